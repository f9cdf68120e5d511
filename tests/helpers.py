"""Shared helpers for the parity tests: seeded inputs in the value distributions of random-init AWQ weights (nibbles uniform, zeros near 8, scales about 0.01), device upload, error metric."""
import numpy as np

import oracle


def rand_qweight(rng, rows, cols, scale_lo=0.001, scale_hi=0.02, zero_max=15):
    """Weights/zero points uniform int4 in [0,15], scales fp16 uniform in [0.001,0.02], QWeight layout."""
    ws, zs, ss = oracle.qweight_sizes(rows)
    w = rng.integers(0, 2**32, size=(cols, ws), dtype=np.uint64).astype(np.uint32)
    # nibbles past `rows` in the padded last vector stay random on purpose: they must not be read as weights
    zn = rng.integers(0, zero_max + 1, size=(cols, zs * 8), dtype=np.uint32)
    z = np.zeros((cols, zs), dtype=np.uint32)
    for n in range(8):
        z |= (zn[:, n::8] & 0xF) << np.uint32(4 * n)
    s = (scale_lo + rng.random((cols, ss)) * (scale_hi - scale_lo)).astype(np.float16)
    return w.reshape(-1), z.reshape(-1), s.reshape(-1)


def rand_vec(rng, n, sigma=1.0):
    return (rng.standard_normal(n) * sigma).astype(np.float16)


def to_dev(a):
    import torch
    a = np.ascontiguousarray(a)
    if a.dtype == np.uint32:
        return torch.from_numpy(a.view(np.int32)).cuda()
    return torch.from_numpy(a).cuda()


def dev_qweight(w, z, s):
    import managedllama2_b200 as ml2
    return ml2.QWeight(to_dev(w), to_dev(z), to_dev(s))


def to_host(t):
    return t.detach().cpu().numpy()


def rel_err(got, want):
    """max |got - want| / max(|want|, rms(want)): relative error that does not blow up on outputs near zero."""
    got = np.asarray(got, dtype=np.float64)
    want = np.asarray(want, dtype=np.float64)
    rms = np.sqrt(np.mean(want * want)) if want.size else 0.0
    den = np.maximum(np.abs(want), max(rms, 1e-30))
    return float(np.max(np.abs(got - want) / den)) if want.size else 0.0


def write_model_bin(path, cfg, hw):
    """Writes a ``model.bin`` in the reference's layout (src/ModelConverter.cs:130-177; read back by
    src/TransformerWeights.cs:33-41, 81-95): 32-byte Config header, embedding, classifier, final norm, then per layer
    the QWeights query, key, value, output, UP, GATE, down (Weight, Zeros, Scales each) and the two norm vectors.
    ``hw`` is the dict of ``synthetic_weights_host``."""
    import struct
    with open(path, "wb") as f:
        f.write(struct.pack("<7if", cfg.dim, cfg.hiddenDim, cfg.numLayers, cfg.numHeads, cfg.numKVHeads, cfg.vocabSize,
                            cfg.seqLength, cfg.ropeTheta))
        for name in ("embed", "classifier", "rms_final"):
            f.write(np.ascontiguousarray(hw[name], np.float16).tobytes())
        for L in hw["layers"]:
            for name in ("q", "k", "v", "o", "up", "gate", "down"):
                w, z, s = L[name]
                f.write(np.ascontiguousarray(w, np.uint32).tobytes())
                f.write(np.ascontiguousarray(z, np.uint32).tobytes())
                f.write(np.ascontiguousarray(s, np.float16).tobytes())
            f.write(np.ascontiguousarray(L["rms_att"], np.float16).tobytes())
            f.write(np.ascontiguousarray(L["rms_ffn"], np.float16).tobytes())
