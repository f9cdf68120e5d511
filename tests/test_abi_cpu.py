"""CPU-only checks of the boundary: the library loads, exports every declared symbol, refuses to run without a GPU,
and the host-side generators / shard geometry are consistent. No compute kernel is launched here."""
import ctypes
import os

import numpy as np
import pytest

import managedllama2_b200 as ml2
from managedllama2_b200 import _lib


def test_library_exports_every_declared_symbol():
    lib = ml2.load()
    names = ml2.declared_symbols()
    assert len(names) >= 40
    missing = [s for s in names if not hasattr(lib, s)]
    assert not missing, missing
    assert lib.ml2_version() >= 100


def test_no_cpu_fallback_without_gpu():
    import torch
    if torch.cuda.is_available():
        pytest.skip("a GPU is present")
    with pytest.raises(ml2.Ml2Error) as e:
        ml2.CudaContext(0)
    assert e.value.code == -2  # ML2_E_CUDA: no device, and no silent fallback


def test_missing_library_fails_loudly(monkeypatch):
    monkeypatch.setattr(_lib, "_lib", None)
    monkeypatch.setattr(_lib, "LIB_PATH", os.path.join(os.path.dirname(_lib.LIB_PATH), "does_not_exist.so"))
    with pytest.raises(ImportError):
        _lib.load()


def test_config_struct_layout_matches_reference_header():
    # src/Config.cs:6-17: seven ints and one float, 32 bytes
    assert ctypes.sizeof(_lib.ConfigStruct) == 32
    c = ml2.Config(5120, 13824, 40, 40, 40, 32000, 4096).to_struct()
    raw = bytes(c)
    assert np.frombuffer(raw[:28], dtype=np.int32).tolist() == [5120, 13824, 40, 40, 40, 32000, 4096]
    assert np.frombuffer(raw[28:], dtype=np.float32)[0] == 10000.0


def test_qweight_sizes_formula():
    # src/QKVMatVec.cs:22-24 on the benchmark shapes
    assert ml2.qweight_sizes(4096) == (512, 4, 32)
    assert ml2.qweight_sizes(5120) == (640, 5, 40)
    assert ml2.qweight_sizes(11008) == (1376, 11, 86)
    assert ml2.qweight_sizes(13824) == (1728, 14, 108)


@pytest.mark.parametrize("tp", [1, 2, 4, 8])
def test_tp_hidden_groups_partition(tp):
    cfg = ml2.Config(5120, 13824, 40, 40, 40, 32000, 64)
    total, nxt = 0, 0
    sizes = []
    for r in range(tp):
        dim_local, g0, ng, vrow0, vlocal = ml2.tp_shapes(cfg, tp, r)
        assert g0 == nxt and dim_local == 5120 // tp and vrow0 == r * vlocal
        nxt += ng
        total += ng
        sizes.append(ng)
    assert total == 108
    assert max(sizes) - min(sizes) <= 1
    if tp == 8:
        assert sizes == [14, 14, 14, 14, 13, 13, 13, 13]


def test_synthetic_shard_equals_slice_of_full_tensor():
    """Every rank's QWeight shard is the slice of the one-GPU tensor (values depend on logical coordinates only)."""
    lib = ml2.load()
    rows_full, cols, seed, tid = 1024, 24, 9, 5
    ws, zs, ss = ml2.qweight_sizes(rows_full)

    def gen(col0, ncols, g0, ng):
        rows = ng * 128
        w_, z_, s_ = ml2.qweight_sizes(rows)
        w, z, s = np.empty(ncols * w_, np.uint32), np.empty(ncols * z_, np.uint32), np.empty(ncols * s_, np.float16)
        _lib.check(lib.ml2_synth_qweight_host(w.ctypes.data_as(ctypes.c_void_p), z.ctypes.data_as(ctypes.c_void_p),
                                              s.ctypes.data_as(ctypes.c_void_p), rows_full, col0, ncols, g0, ng,
                                              ctypes.c_uint64(seed), ctypes.c_uint32(tid)))
        return w.reshape(ncols, w_), z.reshape(ncols, z_), s.reshape(ncols, s_)

    import oracle
    fw, fz, fs = gen(0, cols, 0, 8)
    full = oracle.unpack_rows(fw, fz, fs, rows_full, cols)
    # column shard (QKV / gate / up)
    cw, cz, cs = gen(8, 8, 0, 8)
    assert np.array_equal(cw, fw[8:16]) and np.array_equal(cz, fz[8:16]) and np.array_equal(cs, fs[8:16])
    # row shard (o-proj / down): groups 3..5 -> a valid QWeight with rows = 384 whose zero nibbles are re-based
    rw, rz, rs = gen(0, cols, 3, 3)
    shard = oracle.unpack_rows(rw, rz, rs, 384, cols)
    assert np.array_equal(shard.view(np.uint16), full[:, 384:768].view(np.uint16))
    # distributions
    nib = (fw[:, :, None] >> (np.arange(8, dtype=np.uint32) * 4)) & 0xF
    assert nib.min() == 0 and nib.max() == 15 and abs(nib.mean() - 7.5) < 0.2
    assert fs.astype(np.float32).min() >= 0.00099 and fs.astype(np.float32).max() <= 0.02001


def test_argument_validation_without_device():
    lib = ml2.load()
    # null context is rejected before anything touches CUDA
    q = _lib.QWeightStruct(0, 0, 0)
    assert lib.ml2_matvec_residual_int4(None, None, None, ctypes.byref(q), 128, 128) == -1
    assert b"null" in lib.ml2_last_error()
    assert lib.ml2_model_create(None, None, 1, 0, None, None) == -1
