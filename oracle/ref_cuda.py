"""Runs the reference's OWN CUDA kernels (oracle/_ref/*.cubin, compiled unmodified from native/*.cu of
GilesBathgate/ManagedLlama2 by `make -C oracle ref`) with the launch shapes of its C# Module classes.

Test infrastructure: the second checker for the GPU parity tests ("the reference CUDA build") and the
"reference CUDA kernels" timing reported beside the product in bench.py. Kernels are loaded through the CUDA
driver API (cuda-python) and launched on torch's current stream, on torch tensors.
"""
import ctypes
import math
import os

import numpy as np

REF_DIR = os.path.join(os.path.dirname(os.path.abspath(__file__)), "_ref")
KERNELS = {
    "mat_vec_kernel": ["mat_vec_kernel", "mat_vec_strided_kernel", "mat_vec_residual_int4_kernel", "qkv_mat_vec_kernel",
                       "mat_vec_swiglu_kernel"],
    "vec_mat_kernel": ["vec_mat_kernel"],
    "softmax_kernel": ["softmax_kernel"],
    "rmsnorm_kernel": ["rmsnorm_kernel"],
    "rope_kernel": ["rope_kernel"],
    "embedding_kernel": ["embedding_kernel"],
    "argmax_kernel": ["argmax_kernel"],
    "softmax_logits_kernel": ["softmax_logits_kernel"],
    "sort_kernel": ["sort_kernel"],
    "cumulative_sum_kernel": ["cumulative_sum_kernel"],
    "sample_top_p_kernel": ["sample_top_p_kernel"],
}


def available():
    return all(os.path.exists(os.path.join(REF_DIR, m + ".cubin")) for m in KERNELS)


def ceil_div(a, b):
    return (a + (b - 1)) // b


class RefKernels:
    """One driver-API function handle per reference kernel."""

    def __init__(self):
        import torch
        from cuda.bindings import driver
        self.drv = driver
        torch.cuda.init()
        torch.zeros(1, device="cuda")  # make torch's primary context current on this thread
        self.fn = {}
        self._mods = []
        for mod, names in KERNELS.items():
            err, m = driver.cuModuleLoad(os.path.join(REF_DIR, mod + ".cubin").encode())
            if err != driver.CUresult.CUDA_SUCCESS:
                raise RuntimeError("cuModuleLoad(%s): %s" % (mod, err))
            self._mods.append(m)
            for n in names:
                err, f = driver.cuModuleGetFunction(m, n.encode())
                if err != driver.CUresult.CUDA_SUCCESS:
                    raise RuntimeError("cuModuleGetFunction(%s): %s" % (n, err))
                self.fn[n] = f
        self.launches = 0

    def launch(self, name, grid, block, args, types):
        import torch
        stream = torch.cuda.current_stream().cuda_stream
        g = tuple(grid) + (1,) * (3 - len(grid))
        b = tuple(block) + (1,) * (3 - len(block))
        err, = self.drv.cuLaunchKernel(self.fn[name], g[0], g[1], g[2], b[0], b[1], b[2], 0, stream, (tuple(args), tuple(types)), 0)
        if err != self.drv.CUresult.CUDA_SUCCESS:
            raise RuntimeError("cuLaunchKernel(%s): %s" % (name, err))
        self.launches += 1


P, I, F, B = ctypes.c_void_p, ctypes.c_int, ctypes.c_float, ctypes.c_bool


def _sizes(rows):
    scales = ceil_div(rows, 128)
    return ceil_div(scales, 8), scales, ceil_div(rows, 32) * 4  # zeros, scales, weights (src/QKVMatVec.cs:22-24)


class RefModules:
    """The launch geometry of src/*.cs, one method per Module.Forward."""

    def __init__(self, cfg, kernels=None):
        self.k = kernels or RefKernels()
        self.cfg = cfg
        self.kvDim = cfg.dim * cfg.numKVHeads // cfg.numHeads
        self.headSize = cfg.dim // cfg.numHeads

    def matvec(self, out, x, matrix, rows, cols):                      # src/MatVec.cs:11-16
        self.k.launch("mat_vec_kernel", (ceil_div(cols, 4), 1), (32, 4), (out, x, matrix, rows, cols), (P, P, P, I, I))

    def qkv(self, q, k, v, x, qw, kw, vw, rows, cols):                  # src/QKVMatVec.cs:15-30
        z, s, w = _sizes(rows)
        self.k.launch("qkv_mat_vec_kernel", (ceil_div(cols, 4), 3), (32, 4),
                      (q, k, v, x, qw[0], qw[1], qw[2], kw[0], kw[1], kw[2], vw[0], vw[1], vw[2], rows, cols, z, s, w),
                      (P,) * 13 + (I,) * 5)

    def swiglu(self, out, x, g, u, rows, cols):                        # src/MatVecSwiGLU.cs:11-23
        z, s, w = _sizes(rows)
        self.k.launch("mat_vec_swiglu_kernel", (ceil_div(cols, 4), 1), (32, 4),
                      (out, x, g[0], g[1], g[2], u[0], u[1], u[2], rows, cols, z, s, w), (P,) * 8 + (I,) * 5)

    def residual(self, out, x, m, rows, cols):                         # src/MatVecResidual.cs:11-23
        z, s, w = _sizes(rows)
        self.k.launch("mat_vec_residual_int4_kernel", (ceil_div(cols, 4), 1), (32, 4),
                      (out, x, m[0], m[1], m[2], rows, cols, z, s, w), (P,) * 5 + (I,) * 5)

    def scores(self, att, q, key, seq, scale, grid_seq=None):          # src/MatVecStrided.cs:12-18
        hs, dim = self.headSize, self.cfg.dim
        gs = grid_seq if grid_seq is not None else self.cfg.seqLength   # the reference sizes the grid by the max length
        self.k.launch("mat_vec_strided_kernel", (ceil_div(gs, 32), self.cfg.numHeads), (32, 32),
                      (att, q, key, hs, seq, hs, hs, dim, seq, scale), (P, P, P, I, I, I, I, I, I, F))

    def softmax(self, att, seq):                                       # src/Softmax.cs:10-15
        self.k.launch("softmax_kernel", (self.cfg.numHeads,), (1024,), (att, seq), (P, I))

    def vecmat(self, out, value, att, seq):                            # src/VecMat.cs:13-19
        hs, dim = self.headSize, self.cfg.dim
        self.k.launch("vec_mat_kernel", (ceil_div(hs, 32), self.cfg.numHeads), (32, 32),
                      (out, att, value, hs, seq, hs, hs, dim), (P, P, P, I, I, I, I, I))

    def rmsnorm(self, out, x, w, size, eps=1e-5):                      # src/RMSNorm.cs:10-15
        self.k.launch("rmsnorm_kernel", (1,), (1024,), (out, x, w, size, eps), (P, P, P, I, F))

    def rope(self, q, key, pos, theta):                                # src/RoPERotation.cs:15-23
        self.k.launch("rope_kernel", (self.cfg.numHeads,), (self.headSize // 2,),
                      (q, key, self.cfg.numKVHeads, self.headSize, pos, theta), (P, P, I, I, I, F))

    def embedding(self, out, table, size, tokens, pos):                # src/Embedding.cs:10-15
        self.k.launch("embedding_kernel", (ceil_div(size, 256),), (256,), (out, table, size, tokens, pos), (P, P, I, P, I))

    def argmax(self, logits, vocab, tokens, next_pos, write):          # src/Argmax.cs:10-15
        self.k.launch("argmax_kernel", (1,), (1024,), (logits, vocab, tokens, next_pos, bool(write)), (P, I, P, I, B))

    # the sampling chain (src/Sampler.cs:49-66) with the launch shapes of its Module classes
    def softmax_logits(self, logits, size, temperature, indices):     # src/SoftmaxLogits.cs:9-15
        self.k.launch("softmax_logits_kernel", (1,), (1024,), (logits, size, temperature, indices), (P, I, F, P))

    def sort(self, keys, values, size):                                # src/Sort.cs:9-15: size must be 125 * block
        assert size % 125 == 0 and size // 125 <= 1024
        self.k.launch("sort_kernel", (1,), (size // 125,), (keys, values, size), (P, P, I))

    def cumulative_sum(self, values, size):                            # src/CumulativeSum.cs:9-15: size must be 32 * block
        assert size % 32 == 0 and size // 32 <= 1024
        self.k.launch("cumulative_sum_kernel", (1,), (size // 32,), (values, size), (P, I))

    def sample_top_p(self, values, indices, size, threshold, tokens, pos):   # src/SampleTopP.cs:9-15
        self.k.launch("sample_top_p_kernel", (1,), (1024,), (values, indices, size, threshold, tokens, pos), (P, P, I, F, P, I))


class RefTransformer:
    """Transformer.Forward (src/Transformer.cs:158-190) driven with the reference kernels; RunState as src/RunState.cs."""

    def __init__(self, cfg, weights, kernels=None):
        import torch
        self.cfg = cfg
        self.w = weights
        self.m = RefModules(cfg, kernels)
        dev = "cuda"
        f16 = torch.float16
        self.x = torch.zeros(cfg.dim, dtype=f16, device=dev)
        self.xb = torch.zeros(cfg.dim, dtype=f16, device=dev)
        self.h = torch.zeros(cfg.hiddenDim, dtype=f16, device=dev)
        self.q = torch.zeros(cfg.dim, dtype=f16, device=dev)
        self.attention = torch.zeros(cfg.numHeads * max(cfg.seqLength, cfg.dim), dtype=f16, device=dev)
        self.logits = torch.zeros(cfg.vocabSize, dtype=f16, device=dev)
        kv = cfg.numLayers * cfg.seqLength * self.m.kvDim
        self.keyCache = torch.zeros(kv, dtype=f16, device=dev)
        self.valueCache = torch.zeros(kv, dtype=f16, device=dev)
        self.tokens = torch.zeros(cfg.seqLength + 1, dtype=torch.int32, device=dev)

    @staticmethod
    def _qw(q):
        return (q.Weight.data_ptr(), q.Zeros.data_ptr(), q.Scales.data_ptr())

    def forward(self, pos, next_pos, write_token=True):
        c, m, w = self.cfg, self.m, self.w
        hs = c.dim // c.numHeads
        scale = 1.0 / math.sqrt(hs)
        p = lambda t, off=0: t.data_ptr() + 2 * off
        m.embedding(p(self.x), p(w.tokenEmbeddingTable), c.dim, self.tokens.data_ptr(), pos)
        for i, L in enumerate(w.layers):
            m.rmsnorm(p(self.xb), p(self.x), p(L.rmsAttentionWeight), c.dim)
            loff = i * c.seqLength * m.kvDim
            off = loff + pos * m.kvDim
            m.qkv(p(self.q), p(self.keyCache, off), p(self.valueCache, off), p(self.xb), self._qw(L.queryWeight),
                  self._qw(L.keyWeight), self._qw(L.valueWeight), c.dim, c.dim)
            m.rope(p(self.q), p(self.keyCache, off), pos, c.ropeTheta)
            m.scores(p(self.attention), p(self.q), p(self.keyCache, loff), next_pos, scale)
            m.softmax(p(self.attention), next_pos)
            m.vecmat(p(self.xb), p(self.valueCache, loff), p(self.attention), next_pos)
            m.residual(p(self.x), p(self.xb), self._qw(L.outputWeight), c.dim, c.dim)
            m.rmsnorm(p(self.xb), p(self.x), p(L.rmsFeedForwardWeight), c.dim)
            m.swiglu(p(self.h), p(self.xb), self._qw(L.gateWeight), self._qw(L.upWeight), c.dim, c.hiddenDim)
            m.residual(p(self.x), p(self.h), self._qw(L.downWeight), c.hiddenDim, c.dim)
        m.rmsnorm(p(self.x), p(self.x), p(w.rmsFinalWeight), c.dim)
        m.matvec(p(self.logits), p(self.x), p(w.classifierWeights), c.dim, c.vocabSize)
        m.argmax(p(self.logits), c.vocabSize, self.tokens.data_ptr(), next_pos, write_token)

    def set_tokens(self, toks, first=0):
        import torch
        t = torch.from_numpy(np.ascontiguousarray(toks, dtype=np.int32)).cuda()
        self.tokens[first:first + t.numel()] = t

    def read_token(self, pos):
        return int(self.tokens[pos].item())

    def logits_host(self):
        return self.logits.cpu().numpy()
