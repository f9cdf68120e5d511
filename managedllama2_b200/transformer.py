"""Host-side mirror of the reference's model classes over the model-level C ABI.

``Transformer`` stands for src/Transformer.cs (constructor minus file reading, ``Forward``, ``Generate`` on
token ids), ``TransformerWeights`` / ``PerLayerWeight`` for src/TransformerWeights.cs and
src/PerLayerWeight.cs, ``RunState`` for src/RunState.cs. Weights are torch CUDA tensors owned by Python
and borrowed by the library; the run state is owned by the library.
"""
import ctypes
from dataclasses import dataclass, field
from typing import List

import numpy as np

from . import _lib
from .modules import Config, CudaContext, QWeight, qweight_sizes

GROUP = 128

# tensor ids of the synthetic model (any fixed enumeration works; shards use the same ids)
TID_EMBED, TID_CLASSIFIER, TID_RMS_FINAL = 1, 2, 3
LAYER_TIDS = {"query": 0, "key": 1, "value": 2, "output": 3, "up": 4, "gate": 5, "down": 6, "rms_att": 7, "rms_ffn": 8}


def layer_tid(layer, name):
    return 16 + 16 * layer + LAYER_TIDS[name]


class _LayerStruct(ctypes.Structure):
    _fields_ = [(n, _lib.QWeightStruct) for n in ("query", "key", "value", "output", "gate", "up", "down")] + \
               [("rms_attention", ctypes.c_void_p), ("rms_feed_forward", ctypes.c_void_p)]


class _RunStateStruct(ctypes.Structure):
    _fields_ = [(n, ctypes.c_void_p) for n in ("x", "xb", "h", "q", "logits", "key_cache", "value_cache", "tokens")]


@dataclass
class PerLayerWeight:
    """src/PerLayerWeight.cs:5-16."""
    rmsAttentionWeight: object
    rmsFeedForwardWeight: object
    queryWeight: QWeight
    keyWeight: QWeight
    valueWeight: QWeight
    outputWeight: QWeight
    gateWeight: QWeight
    upWeight: QWeight
    downWeight: QWeight


@dataclass
class TransformerWeights:
    """src/TransformerWeights.cs:8-16. Under tensor parallelism the tensors are this rank's shards."""
    tokenEmbeddingTable: object
    classifierWeights: object
    rmsFinalWeight: object
    layers: List[PerLayerWeight] = field(default_factory=list)


def tp_shapes(config, tp_size, tp_rank):
    """Shard geometry: (dim_local, hidden_group0, hidden_groups, vocab_row0, vocab_local)."""
    lib = _lib.load()
    g0, ng = ctypes.c_int(), ctypes.c_int()
    lib.ml2_tp_hidden_groups.restype = None
    lib.ml2_tp_hidden_groups(config.hiddenDim, tp_size, tp_rank, ctypes.byref(g0), ctypes.byref(ng))
    dim_local = config.dim // tp_size
    vocab_local = config.vocabSize // tp_size
    return dim_local, g0.value, ng.value, vocab_local * tp_rank, vocab_local


def _qw_window(rows_full, ncols, g0, ngroups):
    rows = min(ngroups * GROUP, rows_full - g0 * GROUP)
    ws, zs, ss = qweight_sizes(rows)
    return rows, ncols * ws, ncols * zs, ncols * ss


def synthetic_weights(ctx, config, seed=31415, tp_size=1, tp_rank=0, sigma=0.02):
    """Random-init model (nibbles uniform in 0..15, zero points near 8, scales about 0.01, fp16 normal elsewhere), generated on the device shard by shard.

    int4 weights and zero points uniform in [0,15], scales fp16 uniform in [0.001,0.02]; embeddings,
    classifier and norm weights fp16 ~ N(0, sigma^2). Values depend only on (seed, tensor id, logical
    coordinates), so every rank's shard equals the slice of the one-GPU model.
    """
    import torch
    lib = ctx._lib
    dev = "cuda:%d" % ctx.device
    dim, hid = config.dim, config.hiddenDim
    dim_local, hg0, hng, vrow0, vlocal = tp_shapes(config, tp_size, tp_rank)
    hidden_local = hng * GROUP

    def qweight(tid, rows_full, col0, ncols, g0, ngroups):
        _, nw, nz, ns = _qw_window(rows_full, ncols, g0, ngroups)
        w = torch.empty(nw, dtype=torch.int32, device=dev)
        z = torch.empty(nz, dtype=torch.int32, device=dev)
        s = torch.empty(ns, dtype=torch.float16, device=dev)
        _lib.check(lib.ml2_synth_qweight(ctx.handle, ctypes.c_void_p(w.data_ptr()), ctypes.c_void_p(z.data_ptr()),
                                         ctypes.c_void_p(s.data_ptr()), rows_full, col0, ncols, g0, ngroups,
                                         ctypes.c_uint64(seed), ctypes.c_uint32(tid)))
        return QWeight(w, z, s)

    def normal(tid, row0, nrows, width):
        t = torch.empty(nrows * width, dtype=torch.float16, device=dev)
        _lib.check(lib.ml2_synth_normal_f16(ctx.handle, ctypes.c_void_p(t.data_ptr()), ctypes.c_longlong(row0),
                                            ctypes.c_longlong(nrows), width, ctypes.c_float(sigma),
                                            ctypes.c_uint64(seed), ctypes.c_uint32(tid)))
        return t

    w = TransformerWeights(normal(TID_EMBED, 0, config.vocabSize, dim), normal(TID_CLASSIFIER, vrow0, vlocal, dim),
                           normal(TID_RMS_FINAL, 0, 1, dim))
    gd = dim // GROUP
    for l in range(config.numLayers):
        w.layers.append(PerLayerWeight(
            rmsAttentionWeight=normal(layer_tid(l, "rms_att"), 0, 1, dim),
            rmsFeedForwardWeight=normal(layer_tid(l, "rms_ffn"), 0, 1, dim),
            queryWeight=qweight(layer_tid(l, "query"), dim, tp_rank * dim_local, dim_local, 0, gd),
            keyWeight=qweight(layer_tid(l, "key"), dim, tp_rank * dim_local, dim_local, 0, gd),
            valueWeight=qweight(layer_tid(l, "value"), dim, tp_rank * dim_local, dim_local, 0, gd),
            outputWeight=qweight(layer_tid(l, "output"), dim, 0, dim, tp_rank * (dim_local // GROUP), dim_local // GROUP),
            gateWeight=qweight(layer_tid(l, "gate"), dim, hg0 * GROUP, hidden_local, 0, gd),
            upWeight=qweight(layer_tid(l, "up"), dim, hg0 * GROUP, hidden_local, 0, gd),
            downWeight=qweight(layer_tid(l, "down"), hid, 0, dim, hg0, hng)))
    ctx.synchronize()
    return w


def synthetic_weights_host(config, seed=31415, sigma=0.02):
    """The same model as ``synthetic_weights`` (one GPU) as numpy arrays, for the CPU oracle."""
    lib = _lib.load()
    dim, hid = config.dim, config.hiddenDim

    def qweight(tid, rows_full, ncols):
        ngroups = rows_full // GROUP
        _, nw, nz, ns = _qw_window(rows_full, ncols, 0, ngroups)
        w, z, s = np.empty(nw, np.uint32), np.empty(nz, np.uint32), np.empty(ns, np.float16)
        _lib.check(lib.ml2_synth_qweight_host(w.ctypes.data_as(ctypes.c_void_p), z.ctypes.data_as(ctypes.c_void_p),
                                              s.ctypes.data_as(ctypes.c_void_p), rows_full, 0, ncols, 0, ngroups,
                                              ctypes.c_uint64(seed), ctypes.c_uint32(tid)))
        return w, z, s

    def normal(tid, nrows, width):
        t = np.empty(nrows * width, np.float16)
        _lib.check(lib.ml2_synth_normal_f16_host(t.ctypes.data_as(ctypes.c_void_p), ctypes.c_longlong(0),
                                                 ctypes.c_longlong(nrows), width, ctypes.c_float(sigma),
                                                 ctypes.c_uint64(seed), ctypes.c_uint32(tid)))
        return t

    out = {"embed": normal(TID_EMBED, config.vocabSize, dim), "classifier": normal(TID_CLASSIFIER, config.vocabSize, dim),
           "rms_final": normal(TID_RMS_FINAL, 1, dim), "layers": []}
    for l in range(config.numLayers):
        out["layers"].append({
            "q": qweight(layer_tid(l, "query"), dim, dim), "k": qweight(layer_tid(l, "key"), dim, dim),
            "v": qweight(layer_tid(l, "value"), dim, dim), "o": qweight(layer_tid(l, "output"), dim, dim),
            "gate": qweight(layer_tid(l, "gate"), dim, hid), "up": qweight(layer_tid(l, "up"), dim, hid),
            "down": qweight(layer_tid(l, "down"), hid, dim),
            "rms_att": normal(layer_tid(l, "rms_att"), 1, dim), "rms_ffn": normal(layer_tid(l, "rms_ffn"), 1, dim)})
    return out


# tensor ids of ml2_model_file_tensor (include/ml2b200.h)
T_EMBED, T_CLASSIFIER, T_RMS_FINAL = 0, 1, 2
T_QUERY, T_KEY, T_VALUE, T_OUTPUT, T_UP, T_GATE, T_DOWN, T_RMS_ATT, T_RMS_FFN = range(9)


class ModelFile:
    """A ``model.bin`` of the reference (written by src/ModelConverter.cs:130-177), mapped read-only.

    Stands for ``Config.LoadConfig`` (src/Config.cs:21-31) plus the tensor walk of the ``TransformerWeights``
    constructor (src/TransformerWeights.cs:20-41): a wrong ``ropeTheta`` and a file that is not consumed exactly
    raise, as they do there. Needs no GPU.
    """

    def __init__(self, path):
        self.lib = _lib.load()
        h = ctypes.c_void_p()
        _lib.check(self.lib.ml2_model_file_open(str(path).encode(), ctypes.byref(h)))
        self.handle = h
        cfg = _lib.ConfigStruct()
        _lib.check(self.lib.ml2_model_file_config(h, ctypes.byref(cfg)))
        self.config = Config(cfg.dim, cfg.hidden_dim, cfg.n_layers, cfg.n_heads, cfg.n_kv_heads, cfg.vocab_size, cfg.seq_len,
                             cfg.rope_theta)

    def tensor(self, layer, tensor, part=0):
        """numpy view (uint32 for Weight / Zeros, float16 otherwise) of one array of the file."""
        data, nbytes = ctypes.c_void_p(), ctypes.c_uint64()
        _lib.check(self.lib.ml2_model_file_tensor(self.handle, layer, tensor, part, ctypes.byref(data), ctypes.byref(nbytes)))
        is_u32 = layer >= 0 and tensor <= T_DOWN and part < 2
        buf = (ctypes.c_ubyte * nbytes.value).from_address(data.value)
        return np.frombuffer(buf, dtype=np.uint32 if is_u32 else np.float16)

    def close(self):
        if getattr(self, "handle", None):
            self.lib.ml2_model_file_close(self.handle)
            self.handle = None

    def __enter__(self):
        return self

    def __exit__(self, *a):
        self.close()

    def __del__(self):
        try:
            self.close()
        except Exception:
            pass


class DeviceWeights:
    """This rank's shard of a ``ModelFile`` in device memory (one allocation owned by the library)."""

    def __init__(self, ctx, model_file, tp_size=1, tp_rank=0):
        self.lib = ctx._lib
        h = ctypes.c_void_p()
        _lib.check(self.lib.ml2_weights_upload(ctx.handle, model_file.handle, tp_size, tp_rank, ctypes.byref(h)))
        self.handle = h
        self.n_layers = model_file.config.numLayers

    def layer(self, i):
        s = _FileLayerStruct()
        _lib.check(self.lib.ml2_weights_layer(self.handle, i, ctypes.byref(s)))
        return s

    def device_bytes(self):
        n = ctypes.c_uint64()
        _lib.check(self.lib.ml2_weights_globals(self.handle, None, None, None, ctypes.byref(n)))
        return n.value

    def globals(self):
        e, c, r = ctypes.c_void_p(), ctypes.c_void_p(), ctypes.c_void_p()
        _lib.check(self.lib.ml2_weights_globals(self.handle, ctypes.byref(e), ctypes.byref(c), ctypes.byref(r), None))
        return e.value, c.value, r.value

    def close(self):
        if getattr(self, "handle", None):
            self.lib.ml2_weights_free(self.handle)
            self.handle = None

    def __del__(self):
        try:
            self.close()
        except Exception:
            pass


class _FileLayerStruct(ctypes.Structure):
    _fields_ = _LayerStruct._fields_


def tp_forward_counts_agree(dist, count):
    """True when every rank of `dist` reports the same number of Forward calls; raises RuntimeError otherwise."""
    import torch
    mine = torch.tensor([int(count)], dtype=torch.int64)
    world = dist.get_world_size()
    all_counts = [torch.zeros(1, dtype=torch.int64) for _ in range(world)]
    dist.all_gather(all_counts, mine)
    counts = [int(t.item()) for t in all_counts]
    if len(set(counts)) != 1:
        raise RuntimeError("tensor-parallel ranks are out of step: Forward counts per rank %s" % counts)
    return True


class Transformer:
    """src/Transformer.cs on token ids. ``Forward`` is one CUDA-graph replay of the fused per-token sequence."""

    @classmethod
    def FromFile(cls, modelPath, cudaContext=None, tp_size=1, tp_rank=0, nccl_id=None):
        """``new Transformer(modelPath, ...)`` (src/Transformer.cs:46-61): config and weights come from ``model.bin``."""
        ctx = cudaContext or CudaContext(0)
        with ModelFile(modelPath) as mf:
            dw = DeviceWeights(ctx, mf, tp_size, tp_rank)
            tr = cls(mf.config, dw, ctx, tp_size, tp_rank, nccl_id)
        return tr

    def __init__(self, config: Config, weights: TransformerWeights, cudaContext: CudaContext = None, tp_size=1, tp_rank=0,
                 nccl_id: bytes = None):
        self.config = config
        self.ctx = cudaContext or CudaContext(0)
        self.lib = self.ctx._lib
        self.weights = weights  # keeps the borrowed tensors alive
        self.tp_size, self.tp_rank = tp_size, tp_rank
        kv_dim = config.dim * config.numKVHeads // config.numHeads
        if kv_dim != config.dim:  # src/Transformer.cs:53-56
            raise NotImplementedError("Differing kvDim dimention not currently supported.")
        cfg = config.to_struct()
        h = ctypes.c_void_p()
        idbuf = ctypes.create_string_buffer(nccl_id, 128) if nccl_id is not None else None
        _lib.check(self.lib.ml2_model_create(self.ctx.handle, ctypes.byref(cfg), tp_size, tp_rank, idbuf, ctypes.byref(h)))
        self.handle = h
        if isinstance(weights, DeviceWeights):
            _lib.check(self.lib.ml2_weights_bind(weights.handle, h))
            _lib.check(self.lib.ml2_model_alloc_runstate(h))
            self.lib.ml2_model_launches_per_token.restype = ctypes.c_longlong
            return
        _lib.check(self.lib.ml2_model_bind_globals(h, ctypes.c_void_p(weights.tokenEmbeddingTable.data_ptr()),
                                                   ctypes.c_void_p(weights.classifierWeights.data_ptr()),
                                                   ctypes.c_void_p(weights.rmsFinalWeight.data_ptr())))
        for i, L in enumerate(weights.layers):
            s = _LayerStruct(L.queryWeight.struct(), L.keyWeight.struct(), L.valueWeight.struct(), L.outputWeight.struct(),
                             L.gateWeight.struct(), L.upWeight.struct(), L.downWeight.struct(),
                             L.rmsAttentionWeight.data_ptr(), L.rmsFeedForwardWeight.data_ptr())
            _lib.check(self.lib.ml2_model_bind_layer(h, i, ctypes.byref(s)))
        _lib.check(self.lib.ml2_model_alloc_runstate(h))
        self.lib.ml2_model_launches_per_token.restype = ctypes.c_longlong

    @staticmethod
    def nccl_unique_id():
        buf = ctypes.create_string_buffer(128)
        _lib.check(_lib.load().ml2_nccl_unique_id(buf))
        return buf.raw

    # -- tensor-parallel persistent kernel: peer memory -----------------------------------------------
    def comm_handle(self):
        """64-byte CUDA IPC handle of this rank's peer-visible buffer (tensor parallel models only)."""
        buf = ctypes.create_string_buffer(64)
        _lib.check(self.lib.ml2_model_comm_handle(self.handle, buf))
        return buf.raw

    def attach_peers(self, handles):
        """``handles``: the comm_handle() bytes of every rank, in rank order. Enables the one-launch-per-token path."""
        blob = b"".join(handles)
        assert len(blob) == 64 * self.tp_size
        _lib.check(self.lib.ml2_model_comm_attach(self.handle, ctypes.create_string_buffer(blob, len(blob)), self.tp_size))

    def attach_peers_with(self, dist):
        """Exchanges the handles over an initialised ``torch.distributed`` group and attaches them."""
        import torch
        mine = torch.frombuffer(bytearray(self.comm_handle()), dtype=torch.uint8).cuda()
        allh = [torch.empty_like(mine) for _ in range(self.tp_size)]
        dist.all_gather(allh, mine)
        self.attach_peers([bytes(t.cpu().numpy().tobytes()) for t in allh])
        dist.barrier()

    # -- reference API ---------------------------------------------------------------------------
    def Forward(self, position, nextPosition, generateToken=True):
        _lib.check(self.lib.ml2_model_forward(self.handle, position, nextPosition, 1 if generateToken else 0))

    def Generate(self, promptTokens, steps):
        """Transformer.Generate (src/Transformer.cs:89-112): returns the ids it would yield (stops on id < 3)."""
        prompt = np.ascontiguousarray(promptTokens, dtype=np.int32)
        out = np.zeros(max(steps, 1), dtype=np.int32)
        n = ctypes.c_int(0)
        _lib.check(self.lib.ml2_model_generate(self.handle, prompt.ctypes.data_as(ctypes.c_void_p), int(prompt.size),
                                               int(steps), out.ctypes.data_as(ctypes.c_void_p), ctypes.byref(n)))
        return out[:n.value].tolist()

    def Sample(self, nextPosition, temperature, topP, coin):
        """Sampler.Sample for temperature != 0 (src/Sampler.cs:49-66), after ``Forward(pos, next, False)``."""
        _lib.check(self.lib.ml2_model_sample(self.handle, nextPosition, ctypes.c_float(temperature), ctypes.c_float(topP),
                                             ctypes.c_float(coin)))

    def GenerateSampled(self, promptTokens, steps, temperature=0.5, topP=0.9, seed=0):
        """Transformer.Generate with the reference's default sampler settings (src/Transformer.cs:42, 89-112): prompt
        tokens are forced, then one uniform draw per sampled token (``numpy`` generator instead of System.Random)."""
        if temperature == 0.0:
            return self.Generate(promptTokens, steps)
        rng = np.random.default_rng(seed)
        prompt = [int(t) for t in promptTokens]
        self.set_tokens(np.array(prompt, np.int32))
        out = []
        for pos in range(steps):
            self.Forward(pos, pos + 1, False)
            if pos + 1 >= len(prompt):
                self.Sample(pos + 1, temperature, topP, float(rng.random(dtype=np.float32)))
                tok = self.read_token(pos + 1)
            else:
                tok = prompt[pos + 1]
            if tok < 3:
                break
            out.append(tok)
        return out

    # -- access to the run state -------------------------------------------------------------------
    def set_tokens(self, tokens, first=0):
        t = np.ascontiguousarray(tokens, dtype=np.int32)
        _lib.check(self.lib.ml2_model_set_tokens(self.handle, t.ctypes.data_as(ctypes.c_void_p), first, int(t.size)))

    def read_token(self, pos):
        v = ctypes.c_int(0)
        _lib.check(self.lib.ml2_model_read_token(self.handle, pos, ctypes.byref(v)))
        return v.value

    def logits(self):
        out = np.empty(self.config.vocabSize, dtype=np.float16)
        _lib.check(self.lib.ml2_model_read_logits(self.handle, out.ctypes.data_as(ctypes.c_void_p)))
        return out

    def synchronize(self):
        _lib.check(self.lib.ml2_model_synchronize(self.handle))

    def forward_count_in_step(self, dist, count):
        """Host rule of the tensor-parallel persistent kernel: every rank calls Forward the same number of times (a
        rank that skipped one leaves its peers waiting for arrivals that never come). Gathers the ranks' counts over
        `dist` (any backend) and raises on the first mismatch, before anything is launched."""
        return tp_forward_counts_agree(dist, count)

    def set_split_attention_from(self, min_seq):
        """Sequence length from which the persistent kernel splits a head's attention over several CTAs (default 704)."""
        _lib.check(self.lib.ml2_model_set_split_attention_from(self.handle, ctypes.c_int(int(min_seq))))

    def reset(self):
        """After an Ml2Error with code ML2_E_DEVICE (a kernel's bounded wait ran out): clears the error and the
        counters the persistent kernel keeps between tokens. Under tensor parallelism every rank calls it."""
        _lib.check(self.lib.ml2_model_reset(self.handle))

    @property
    def launches_per_token(self):
        return int(self.lib.ml2_model_launches_per_token(self.handle))

    def runstate_ptrs(self):
        rs = _RunStateStruct()
        _lib.check(self.lib.ml2_model_runstate(self.handle, ctypes.byref(rs)))
        return rs

    def close(self):
        if getattr(self, "handle", None):
            self.lib.ml2_model_destroy(self.handle)
            self.handle = None

    def __del__(self):
        try:
            self.close()
        except Exception:
            pass
