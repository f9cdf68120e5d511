"""Parity of the int4 / fp16 mat-vec family on the GPU against the CPU oracle, through the C ABI.

Mirrors test/MatVecInt4Tests.cs, QKVMatVecInt4Tests.cs, SwiGLUMatVecInt4Tests.cs and MatVecTests.cs of
the reference, and adds what they leave out: non-zero zero points, realistic scales, multi-row matrices
whose d_in is not a multiple of 1024, ragged output counts, the 4096 x 4096 and Llama-2-7B layer shapes.

Tolerance: relative error <= 1e-3 against the fp32-accumulate CPU arithmetic, measured as
|got-want| / max(|want|, rms(want)).
"""
import numpy as np
import pytest

import oracle
from helpers import dev_qweight, rand_qweight, rand_vec, rel_err, to_dev, to_host

pytestmark = pytest.mark.gpu
TOL = 1e-3


@pytest.fixture(scope="module")
def ctx():
    import managedllama2_b200 as ml2
    c = ml2.CudaContext(0)
    yield c
    err, _ = c.status()
    assert err == 0
    c.close()


def test_reference_case_128x128_bit_exact(ctx):
    """test/MatVecInt4Tests.cs:72-93: ints in [0,15), scale 1, zero 0 -> every product and sum is exact: bit equality."""
    import managedllama2_b200 as ml2
    rng = np.random.default_rng(31415)
    rows = cols = 128
    vals = rng.integers(0, 15, size=rows * cols).astype(np.float16)
    w = np.zeros(rows * cols // 8, np.uint32)
    z = np.zeros(cols, np.uint32)
    s = np.ones(cols, np.float16)
    for c in range(cols):
        ww, _, _ = oracle.pack_flat(vals[c * rows:(c + 1) * rows], np.ones(1, np.float32), np.zeros(1, np.uint32))
        w[c * 16:(c + 1) * 16] = ww
    x = rng.integers(-8, 8, size=rows).astype(np.float16)  # integer inputs keep fp32 sums exact
    res = rng.integers(-8, 8, size=cols).astype(np.float16)
    want = oracle.matvec_residual_int4(res, x, w, z, s, rows, cols, mode=0)
    d_res = to_dev(res)
    ml2.MatVecResidual(ctx).Forward(d_res, to_dev(x), dev_qweight(w, z, s), rows, cols)
    assert np.array_equal(to_host(d_res).view(np.uint16), want.view(np.uint16))


@pytest.mark.parametrize("rows,cols", [(128, 128), (4096, 4096), (11008, 4096), (5120, 5120), (13824, 5120),
                                        (640, 5120), (1728, 333), (4096, 37), (96, 8), (5504, 64), (1024, 3)])
def test_matvec_residual_int4(ctx, rows, cols):
    import managedllama2_b200 as ml2
    rng = np.random.default_rng(rows * 7 + cols)
    w, z, s = rand_qweight(rng, rows, cols)
    x, res = rand_vec(rng, rows), rand_vec(rng, cols)
    want_k = oracle.matvec_residual_int4(res, x, w, z, s, rows, cols, mode=1)   # kernel arithmetic, exact sum
    want_cs = oracle.matvec_residual_int4(res, x, w, z, s, rows, cols, mode=0)  # C# test reference
    d_res = to_dev(res)
    ml2.MatVecResidual(ctx).Forward(d_res, to_dev(x), dev_qweight(w, z, s), rows, cols)
    got = to_host(d_res)
    assert rel_err(got, want_k) <= TOL
    # the C# reference rounds every dequantised weight to fp16 first (src/QWeight.cs:53): allow that on top
    assert rel_err(got, want_cs) <= 2 * TOL


@pytest.mark.parametrize("rows,cols", [(128, 128), (4096, 4096), (5120, 5120), (1024, 100)])
def test_qkv_matvec_int4(ctx, rows, cols):
    import torch
    import managedllama2_b200 as ml2
    rng = np.random.default_rng(rows + 3 * cols)
    qs = [rand_qweight(rng, rows, cols) for _ in range(3)]
    x = rand_vec(rng, rows)
    want = oracle.qkv_matvec_int4(x, *qs, rows, cols, mode=1)
    cfg = ml2.Config(cols, 4 * cols, 1, max(cols // 128, 1), max(cols // 128, 1), 32, 8)
    q_out = torch.zeros(cols, dtype=torch.float16, device="cuda")
    kc = torch.zeros(8 * cols, dtype=torch.float16, device="cuda")
    vc = torch.zeros(8 * cols, dtype=torch.float16, device="cuda")
    pos = 5
    ml2.QKVMatVec(ctx, cfg).Forward(q_out, kc, vc, to_dev(x), *[dev_qweight(*t) for t in qs], rows, cols, 0, pos)
    got = [to_host(q_out), to_host(kc)[pos * cols:(pos + 1) * cols], to_host(vc)[pos * cols:(pos + 1) * cols]]
    for g, w_ in zip(got, want):
        assert rel_err(g, w_) <= TOL
    # nothing but row `pos` of the caches was written
    assert not to_host(kc)[:pos * cols].any() and not to_host(kc)[(pos + 1) * cols:].any()
    assert not to_host(vc)[:pos * cols].any() and not to_host(vc)[(pos + 1) * cols:].any()


@pytest.mark.parametrize("rows,cols", [(128, 128), (4096, 11008), (5120, 13824), (512, 90)])
def test_matvec_swiglu_int4(ctx, rows, cols):
    """The gate and up mat-vecs are each held to the 1e-3 of every mat-vec output (through ml2_matvec_int4 on the same
    weights and input); the fused output silu(g) * u then carries both errors: with |dg|, |du| <= 1e-3 (relative to the
    larger of the value and the vector's rms) and |d silu / dg| <= 1.1, the product is within (1.1 + 1) * 1e-3 = 2.1e-3
    plus its own fp16 rounding (4.9e-4): the bound asserted below is 2.6e-3."""
    import ctypes
    import torch
    import managedllama2_b200 as ml2
    from managedllama2_b200 import _lib
    rng = np.random.default_rng(rows + 5 * cols)
    g, u = rand_qweight(rng, rows, cols), rand_qweight(rng, rows, cols)
    x = rand_vec(rng, rows, 0.3)
    xd = to_dev(x)
    for q in (g, u):
        dq = dev_qweight(*q)
        qs = dq.struct()
        part = torch.zeros(cols, dtype=torch.float16, device="cuda")
        _lib.check(ctx._lib.ml2_matvec_int4(ctx.handle, ctypes.c_void_p(part.data_ptr()), ctypes.c_void_p(xd.data_ptr()),
                                            ctypes.byref(qs), rows, cols))
        zero = np.zeros(cols, np.float16)
        assert rel_err(to_host(part), oracle.matvec_residual_int4(zero, x, *q, rows, cols, mode=1)) <= TOL
    want = oracle.matvec_swiglu_int4(x, g, u, rows, cols, mode=1)
    out = torch.zeros(cols, dtype=torch.float16, device="cuda")
    ml2.MatVecSwiGLU(ctx).Forward(out, xd, dev_qweight(*g), dev_qweight(*u), rows, cols)
    assert rel_err(to_host(out), want) <= 2.6 * TOL


@pytest.mark.parametrize("rows,cols", [(4096, 64), (4096, 32000), (5120, 1000), (264, 7)])
def test_matvec_f16(ctx, rows, cols):
    """test/MatVecTests.cs:58-75 shape (4096 x 64) plus the classifier shapes."""
    import torch
    import managedllama2_b200 as ml2
    rng = np.random.default_rng(rows + cols)
    w = (rng.standard_normal((cols, rows)) * 0.02).astype(np.float16)
    x = rand_vec(rng, rows)
    want = oracle.matvec_f16(x, w, rows, cols)
    out = torch.zeros(cols, dtype=torch.float16, device="cuda")
    ml2.MatVec(ctx).Forward(out, to_dev(x), to_dev(w), rows, cols)
    assert rel_err(to_host(out), want) <= TOL


@pytest.mark.parametrize("rows,cols", [(1024, 1), (4096, 16), (11008, 5), (13824, 3), (96, 4)])
def test_dequant_bit_exact(ctx, rows, cols):
    import ctypes
    import torch
    import managedllama2_b200 as ml2
    from managedllama2_b200 import _lib
    rng = np.random.default_rng(rows * 3 + cols)
    w, z, s = rand_qweight(rng, rows, cols)
    want = oracle.unpack_rows(w, z, s, rows, cols)
    out = torch.zeros(cols * rows, dtype=torch.float16, device="cuda")
    q = dev_qweight(w, z, s)
    qs = q.struct()
    _lib.check(ctx._lib.ml2_dequant_int4(ctx.handle, ctypes.c_void_p(out.data_ptr()), ctypes.byref(qs), rows, cols))
    assert np.array_equal(to_host(out).view(np.uint16), want.reshape(-1).view(np.uint16))


def test_dequant_golden_vector(ctx, golden_dir):
    """The reference's literal QWeight vector (test/QWeightTestData.cs) through the device unpacking."""
    import ctypes
    import json
    import os
    import torch
    from managedllama2_b200 import _lib
    g = json.load(open(os.path.join(golden_dir, "qweight_fromdata.json")))
    scales = np.array(g["scales_f32_bits"], dtype=np.uint32).view(np.float32).astype(np.float16)
    w = np.array(g["weights"], dtype=np.uint32)
    z = np.array([g["zero_packed"]], dtype=np.uint32)
    want = np.array(g["checks_f32_bits"], dtype=np.uint32).view(np.float32).astype(np.float16)
    out = torch.zeros(1024, dtype=torch.float16, device="cuda")
    qs = dev_qweight(w, z, scales)
    st = qs.struct()
    _lib.check(ctx._lib.ml2_dequant_int4(ctx.handle, ctypes.c_void_p(out.data_ptr()), ctypes.byref(st), 1024, 1))
    assert np.array_equal(to_host(out).view(np.uint16), want.view(np.uint16))


def test_host_buffer_entry_point(ctx):
    import ctypes
    from managedllama2_b200 import _lib
    rng = np.random.default_rng(5)
    rows, cols = 4096, 4096
    w, z, s = rand_qweight(rng, rows, cols)
    x, res = rand_vec(rng, rows), rand_vec(rng, cols)
    want = oracle.matvec_residual_int4(res, x, w, z, s, rows, cols, mode=1)
    q = dev_qweight(w, z, s)
    st = q.struct()
    buf = res.copy()
    _lib.check(ctx._lib.ml2_matvec_residual_int4_host(ctx.handle, buf.ctypes.data_as(ctypes.c_void_p),
                                                     x.ctypes.data_as(ctypes.c_void_p), ctypes.byref(st), rows, cols))
    assert rel_err(buf, want) <= TOL


def test_argument_checks(ctx):
    import torch
    import managedllama2_b200 as ml2
    x = torch.zeros(4096, dtype=torch.float16, device="cuda")
    q = dev_qweight(*rand_qweight(np.random.default_rng(0), 128, 8))
    with pytest.raises(ml2.Ml2Error):
        ml2.MatVecResidual(ctx).Forward(x, x, q, 128, 8)          # aliasing
    with pytest.raises(ml2.Ml2Error):
        ml2.MatVecResidual(ctx).Forward(x, x[1:], q, 128, 8)      # misaligned input
    with pytest.raises(ml2.Ml2Error):
        ml2.MatVecResidual(ctx).Forward(x, x[8:], q, 0, 8)        # bad size
