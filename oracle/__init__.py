"""ctypes binding of the CPU oracle (``oracle/ml2_oracle.c``).

Test infrastructure: imported by ``tests/``, by ``__graft_entry__.smoke()`` and by the CPU-baseline
legs of ``bench.py`` only. The product package never imports it.

All arrays are numpy: fp16 as ``np.float16``, packed words as ``np.uint32``.
"""
import ctypes
import os
import subprocess

import numpy as np

_HERE = os.path.dirname(os.path.abspath(__file__))
_LIB_PATH = os.path.join(_HERE, "libml2oracle.so")
REF_DIR = os.path.join(_HERE, "_ref")


def build(force=False):
    """Compiles the C oracle with gcc (and the reference's CUDA kernels when the checkout exists)."""
    src = os.path.join(_HERE, "ml2_oracle.c")
    if force or not os.path.exists(_LIB_PATH) or os.path.getmtime(_LIB_PATH) < os.path.getmtime(src):
        subprocess.check_call(["make", "-s", "-C", _HERE])
    return _LIB_PATH


def reference_root():
    """Where the reference checkout lives: ML2_REFERENCE_ROOT, else a ``reference`` directory beside this repository."""
    return os.environ.get("ML2_REFERENCE_ROOT") or os.path.join(os.path.dirname(os.path.dirname(_HERE)), "reference")


def build_ref(reference_root=None, force=False):
    """Compiles the reference's own .cu files (in place, outputs into oracle/_ref/) if the checkout is there."""
    if reference_root is None:
        reference_root = globals()["reference_root"]()
    if not os.path.isdir(os.path.join(reference_root, "native")):
        return False
    if force or not os.path.exists(os.path.join(REF_DIR, "mat_vec_kernel.cubin")):
        subprocess.check_call(["make", "-s", "-C", _HERE, "ref", "REF=" + reference_root])
    return True


_lib = None


def lib():
    global _lib
    if _lib is None:
        build()
        _lib = ctypes.CDLL(_LIB_PATH)
    return _lib


def _p(a):
    return a.ctypes.data_as(ctypes.c_void_p)


def _f16(a):
    a = np.ascontiguousarray(a, dtype=np.float16)
    return a


def _u32(a):
    return np.ascontiguousarray(a, dtype=np.uint32)


def set_threads(n):
    lib().orc_set_threads(ctypes.c_int(int(n)))


def ceil_div(a, b):
    return (a + b - 1) // b


def qweight_sizes(rows):
    """(weightsSize, zerosSize, scalesSize) per output, src/QKVMatVec.cs:22-24."""
    scales = ceil_div(rows, 128)
    return ceil_div(rows, 32) * 4, ceil_div(scales, 8), scales


def unpack_flat(weight, zeros, scales):
    weight, zeros, scales = _u32(weight), _u32(zeros), _f16(scales)
    out = np.empty(weight.size * 8, dtype=np.float16)
    lib().orc_unpack_flat(_p(weight), _p(zeros), _p(scales), ctypes.c_int(weight.size), _p(out))
    return out


def pack_flat(data, scales, zeros_unpacked):
    data = _f16(data)
    scales = np.ascontiguousarray(scales, dtype=np.float32)
    zeros_unpacked = _u32(zeros_unpacked)
    n_scales = scales.size
    assert data.size == n_scales * 128 and zeros_unpacked.size == n_scales
    weight = np.zeros(data.size // 8, dtype=np.uint32)
    zeros = np.zeros(max(n_scales // 8, 1), dtype=np.uint32)
    scales_out = np.zeros(n_scales, dtype=np.float16)
    lib().orc_pack_flat(_p(data), _p(scales), _p(zeros_unpacked), ctypes.c_int(n_scales), _p(weight), _p(zeros),
                        _p(scales_out))
    return weight, zeros, scales_out


def unpack_rows(w, z, s, rows, cols):
    w, z, s = _u32(w), _u32(z), _f16(s)
    out = np.empty((cols, rows), dtype=np.float16)
    lib().orc_unpack_rows(_p(w), _p(z), _p(s), ctypes.c_int(rows), ctypes.c_int(cols), _p(out))
    return out


def matvec_int4_f32(x, w, z, s, rows, cols, mode=0):
    x, w, z, s = _f16(x), _u32(w), _u32(z), _f16(s)
    out = np.empty(cols, dtype=np.float32)
    lib().orc_matvec_int4_f32(_p(out), _p(x), _p(w), _p(z), _p(s), ctypes.c_int(rows), ctypes.c_int(cols),
                              ctypes.c_int(mode))
    return out


def matvec_residual_int4(res, x, w, z, s, rows, cols, mode=0):
    out = _f16(res).copy()
    x, w, z, s = _f16(x), _u32(w), _u32(z), _f16(s)
    lib().orc_matvec_residual_int4(_p(out), _p(x), _p(w), _p(z), _p(s), ctypes.c_int(rows), ctypes.c_int(cols),
                                   ctypes.c_int(mode))
    return out


def qkv_matvec_int4(x, q, k, v, rows, cols, mode=0):
    """q, k, v are (w, z, s) triples; returns the three fp16 outputs."""
    x = _f16(x)
    outs = [np.empty(cols, dtype=np.float16) for _ in range(3)]
    trip = []
    keep = []
    for w, z, s in (q, k, v):
        a = (_u32(w), _u32(z), _f16(s))
        keep.append(a)
        trip += [_p(a[0]), _p(a[1]), _p(a[2])]
    lib().orc_qkv_matvec_int4(_p(outs[0]), _p(outs[1]), _p(outs[2]), _p(x), *trip, ctypes.c_int(rows),
                              ctypes.c_int(cols), ctypes.c_int(mode))
    return outs


def matvec_swiglu_int4(x, g, u, rows, cols, mode=0):
    x = _f16(x)
    out = np.empty(cols, dtype=np.float16)
    ga = (_u32(g[0]), _u32(g[1]), _f16(g[2]))
    ua = (_u32(u[0]), _u32(u[1]), _f16(u[2]))
    lib().orc_matvec_swiglu_int4(_p(out), _p(x), _p(ga[0]), _p(ga[1]), _p(ga[2]), _p(ua[0]), _p(ua[1]), _p(ua[2]),
                                 ctypes.c_int(rows), ctypes.c_int(cols), ctypes.c_int(mode))
    return out


def matvec_f16(x, w, rows, cols):
    x, w = _f16(x), _f16(w)
    out = np.empty(cols, dtype=np.float16)
    lib().orc_matvec_f16(_p(out), _p(x), _p(w), ctypes.c_int(rows), ctypes.c_int(cols))
    return out


def attn_scores(q, k, dim, n_heads, n_kv_heads, seq_len):
    q, k = _f16(q), _f16(k)
    att = np.empty(n_heads * seq_len, dtype=np.float16)
    lib().orc_attn_scores(_p(att), _p(q), _p(k), ctypes.c_int(dim), ctypes.c_int(n_heads), ctypes.c_int(n_kv_heads),
                          ctypes.c_int(seq_len))
    return att


def softmax(att, n_heads, size):
    out = _f16(att).copy()
    lib().orc_softmax(_p(out), ctypes.c_int(n_heads), ctypes.c_int(size))
    return out


def attn_values(att, v, dim, n_heads, n_kv_heads, seq_len):
    att, v = _f16(att), _f16(v)
    out = np.empty(dim, dtype=np.float16)
    lib().orc_attn_values(_p(out), _p(att), _p(v), ctypes.c_int(dim), ctypes.c_int(n_heads), ctypes.c_int(n_kv_heads),
                          ctypes.c_int(seq_len))
    return out


def rmsnorm(x, gamma, eps=1e-5, fp16_square=False):
    x, gamma = _f16(x), _f16(gamma)
    out = np.empty_like(x)
    lib().orc_rmsnorm(_p(out), _p(x), _p(gamma), ctypes.c_int(x.size), ctypes.c_float(eps),
                      ctypes.c_int(1 if fp16_square else 0))
    return out


def rope(q, k_row, dim, n_heads, n_kv_heads, pos, theta=10000.0):
    q, k_row = _f16(q).copy(), _f16(k_row).copy()
    lib().orc_rope(_p(q), _p(k_row), ctypes.c_int(dim), ctypes.c_int(n_heads), ctypes.c_int(n_kv_heads),
                   ctypes.c_int(pos), ctypes.c_float(theta))
    return q, k_row


def argmax(logits):
    logits = _f16(logits)
    f = lib().orc_argmax
    f.restype = ctypes.c_int
    return int(f(_p(logits), ctypes.c_int(logits.size)))


class _QW(ctypes.Structure):
    _fields_ = [("w", ctypes.c_void_p), ("z", ctypes.c_void_p), ("s", ctypes.c_void_p)]


class _Config(ctypes.Structure):
    _fields_ = [("dim", ctypes.c_int), ("hidden_dim", ctypes.c_int), ("n_layers", ctypes.c_int),
                ("n_heads", ctypes.c_int), ("n_kv_heads", ctypes.c_int), ("vocab_size", ctypes.c_int),
                ("seq_len", ctypes.c_int), ("rope_theta", ctypes.c_float)]


class _Layer(ctypes.Structure):
    _fields_ = [(n, _QW) for n in ("q", "k", "v", "o", "gate", "up", "down")] + [("rms_att", ctypes.c_void_p),
                                                                                 ("rms_ffn", ctypes.c_void_p)]


class _Model(ctypes.Structure):
    _fields_ = [("cfg", _Config), ("embed", ctypes.c_void_p), ("classifier", ctypes.c_void_p),
                ("rms_final", ctypes.c_void_p), ("layers", ctypes.c_void_p)] + \
               [(n, ctypes.c_void_p) for n in ("x", "xb", "h", "q", "att", "logits", "key_cache", "value_cache")] + \
               [("eps", ctypes.c_float), ("mode", ctypes.c_int)]


class CpuModel:
    """Whole-model CPU forward, composed like Transformer.Forward (src/Transformer.cs:158-190).

    ``weights`` is a dict: embed, classifier, rms_final (fp16 arrays) and ``layers``: list of dicts with
    q,k,v,o,gate,up,down -> (w,z,s) triples and rms_att, rms_ffn.
    """

    def __init__(self, cfg, weights, mode=1, eps=1e-5):
        self.cfg = dict(cfg)
        self._keep = []
        c = self.cfg
        kv_dim = c["dim"] * c["n_kv_heads"] // c["n_heads"]

        def hold(a, dt):
            a = np.ascontiguousarray(a, dtype=dt)
            self._keep.append(a)
            return a.ctypes.data

        layers = (_Layer * c["n_layers"])()
        for i, lw in enumerate(weights["layers"]):
            for n in ("q", "k", "v", "o", "gate", "up", "down"):
                w, z, s = lw[n]
                setattr(layers[i], n, _QW(hold(w, np.uint32), hold(z, np.uint32), hold(s, np.float16)))
            layers[i].rms_att = hold(lw["rms_att"], np.float16)
            layers[i].rms_ffn = hold(lw["rms_ffn"], np.float16)
        self._layers = layers
        self.x = np.zeros(c["dim"], np.float16)
        self.xb = np.zeros(c["dim"], np.float16)
        self.h = np.zeros(c["hidden_dim"], np.float16)
        self.q = np.zeros(c["dim"], np.float16)
        self.att = np.zeros(c["n_heads"] * c["seq_len"], np.float16)
        self.logits = np.zeros(c["vocab_size"], np.float16)
        self.key_cache = np.zeros(c["n_layers"] * c["seq_len"] * kv_dim, np.float16)
        self.value_cache = np.zeros_like(self.key_cache)
        m = _Model()
        m.cfg = _Config(c["dim"], c["hidden_dim"], c["n_layers"], c["n_heads"], c["n_kv_heads"], c["vocab_size"],
                        c["seq_len"], c.get("rope_theta", 10000.0))
        m.embed = hold(weights["embed"], np.float16)
        m.classifier = hold(weights["classifier"], np.float16)
        m.rms_final = hold(weights["rms_final"], np.float16)
        m.layers = ctypes.addressof(layers)
        for n in ("x", "xb", "h", "q", "att", "logits", "key_cache", "value_cache"):
            setattr(m, n, getattr(self, n).ctypes.data)
        m.eps = eps
        m.mode = mode
        self._m = m

    def forward(self, token, pos):
        lib().orc_forward(ctypes.byref(self._m), ctypes.c_int(int(token)), ctypes.c_int(int(pos)))
        return self.logits.copy()


# ---- sampling chain (numpy restatement of src/Sampler.cs:40-70 and its four kernels) --------------------------

def softmax_logits(logits, temperature):
    """native/softmax_logits_kernel.cu:10-54: returns (probabilities fp16, indices). fp16 rounding after the division
    by the temperature, of every exponential (the sum uses the unrounded ones) and of the final quotient."""
    x = (_f16(logits).astype(np.float32) / np.float32(temperature)).astype(np.float16)
    mx = x.astype(np.float32).max()
    v = np.exp(x.astype(np.float32) - mx, dtype=np.float32)
    total = np.float32(v.sum(dtype=np.float32))
    probs = (v.astype(np.float16).astype(np.float32) / total).astype(np.float16)
    return probs, np.arange(x.size, dtype=np.int32)


def sort_desc(keys, values):
    """native/sort_kernel.cu:13-45: keys descending, values carried, ties in their original order (stable radix sort)."""
    keys = _f16(keys)
    order = np.argsort(-keys.astype(np.float32), kind="stable")
    return keys[order], np.asarray(values, np.int32)[order]


def cumulative_sum(values):
    """native/cumulative_sum_kernel.cu:9-28 / test/CumulativeSumTests.cs:44-56: running fp32 sum, each rounded to fp16."""
    with np.errstate(over="ignore"):   # sums beyond the fp16 range become infinities, as the kernel's cast makes them
        return np.cumsum(_f16(values).astype(np.float32), dtype=np.float32).astype(np.float16)


def sample_top_p(values, indices, threshold):
    """native/sample_top_p_kernel.cu:9-24: indices[first t with values[t] >= threshold], the last entry if none."""
    hit = np.nonzero(_f16(values).astype(np.float32) >= np.float32(threshold))[0]
    return int(np.asarray(indices)[hit[0] if hit.size else len(values) - 1])


def sample(logits, temperature, top_p, coin):
    """Sampler.Sample for temperature != 0 (src/Sampler.cs:49-66)."""
    probs, idx = softmax_logits(logits, temperature)
    threshold = np.float32(coin)
    if 0.0 < top_p < 1.0:
        probs, idx = sort_desc(probs, idx)
        threshold = np.float32(coin) * np.float32(top_p)
    return sample_top_p(cumulative_sum(probs), idx, threshold)


# ---- AWQ -> QWeight repacking (restatement of src/ModelConverter.cs:19, 286-332) ------------------------------

AWQ_ORDER_MAP = (0, 2, 4, 6, 1, 3, 5, 7)   # src/ModelConverter.cs:19


def awq_repack_qdata_loops(q_in, height, width):
    """RepackQData (src/ModelConverter.cs:286-321) as the plain loops it is written in, spare elements of the scratch
    array included. The reference keeps four (:288), enough for the group counts of Llama-2 (32, 40, 86, 108); a
    column count whose remainder modulo 8 is 1, 2 or 3 would run past them there. Seven are kept here so that such
    shapes read zeros instead. ``q_in``: uint32 [height][width / 8]. For small cases."""
    q_in = np.ascontiguousarray(q_in, np.uint32).reshape(-1)
    packed = [0] * (width * height + 7)
    for y in range(height):
        for x in range(0, width, 8):
            offset = height * x + y
            word = int(q_in[(y * width + x) // 8])
            q = [0] * 8
            for i in range(8):
                q[AWQ_ORDER_MAP[i]] = word & 0xF
                word >>= 4
            for i in range(8):
                packed[offset + height * i] = q[i]
    h8 = (height + 7) // 8
    out = np.zeros(width * h8, np.uint32)
    for x in range(width):
        for y in range(0, height, 8):
            offset = height * x + y
            val = 0
            for i in range(8):
                val |= packed[offset + i] << (4 * i)
            out[x * h8 + y // 8] = val
    return out


def awq_repack_qdata(q_in, height, width):
    """The same, vectorised."""
    q_in = np.ascontiguousarray(q_in, np.uint32).reshape(height, width // 8)
    nib = np.zeros((height, width // 8, 8), np.uint32)
    for j in range(8):
        nib[:, :, AWQ_ORDER_MAP[j]] = (q_in >> np.uint32(4 * j)) & np.uint32(0xF)
    vals = nib.reshape(height, width).T.reshape(-1)          # column-major scratch: index = height * x + y
    h8 = (height + 7) // 8
    flat = np.concatenate([vals, np.zeros(8, np.uint32)])
    idx = (np.arange(width)[:, None, None] * height + np.arange(h8)[None, :, None] * 8 + np.arange(8)[None, None, :])
    idx = np.minimum(idx, vals.size + 7)                      # beyond the last output: the spare zeros
    g = flat[idx]
    return (g << (np.arange(8, dtype=np.uint32) * np.uint32(4))[None, None, :]).sum(axis=2, dtype=np.uint64).astype(np.uint32).reshape(-1)


def awq_repack_scales(s_in, meta_height, width):
    """RepackScales (src/ModelConverter.cs:323-332): [meta_height][width] -> [width][meta_height]."""
    return np.ascontiguousarray(_f16(s_in).reshape(meta_height, width).T).reshape(-1)


def awq_pack_v0(values, height, width):
    """Inverse of the first step: 4-bit ``values`` [height][width] -> AutoAWQ words [height][width / 8] (test helper)."""
    v = np.asarray(values, np.uint32).reshape(height, width // 8, 8)
    out = np.zeros((height, width // 8), np.uint32)
    for j in range(8):
        out |= (v[:, :, AWQ_ORDER_MAP[j]] & np.uint32(0xF)) << np.uint32(4 * j)
    return out.reshape(-1)


# ---- synthetic model of the benchmark's value distributions (numpy only) ---------------------------------------------

def synthetic_weights(cfg, seed=31415, sigma=0.02):
    """A model of the benchmark construction made with numpy alone (the CPU arm of the benchmark must not need the
    product library): int4 nibbles and zero points uniform in [0, 15], group scales uniform in [0.001, 0.02],
    embeddings / classifier / norm weights ~ N(0, sigma^2), in the QWeight layout of src/QWeight.cs:5-10 with the
    per-row sizes of src/TransformerWeights.cs:54-69. The values are not those of the device generator (nor need they
    be: the arm is timed, not compared)."""
    rng = np.random.default_rng(seed)
    dim, hid, vocab = cfg["dim"], cfg["hidden_dim"], cfg["vocab_size"]

    def qweight(rows, cols):
        nw, nz, ns = qweight_sizes(rows)
        w = rng.integers(0, 1 << 32, size=cols * nw, dtype=np.uint32)
        z = rng.integers(0, 1 << 32, size=cols * nz, dtype=np.uint32)
        s = (0.001 + 0.019 * rng.random(cols * ns, dtype=np.float32)).astype(np.float16)
        return w, z, s

    def normal(n):
        return (rng.standard_normal(n, dtype=np.float32) * sigma).astype(np.float16)

    out = {"embed": normal(vocab * dim), "classifier": normal(vocab * dim), "rms_final": normal(dim), "layers": []}
    for _ in range(cfg["n_layers"]):
        out["layers"].append({"q": qweight(dim, dim), "k": qweight(dim, dim), "v": qweight(dim, dim), "o": qweight(dim, dim),
                              "gate": qweight(dim, hid), "up": qweight(dim, hid), "down": qweight(hid, dim),
                              "rms_att": normal(dim), "rms_ffn": normal(dim)})
    return out
