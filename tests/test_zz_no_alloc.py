"""The allocation-free host-buffer mat-vec against the allocating one (collected last on purpose).

`ml2_matvec_residual_int4_host_static` serves hosts that own all device memory themselves (as the
reference's C# side does) and must not see the library call cudaMalloc: it stages its vectors in a fixed
array inside the library. It must give exactly what `ml2_matvec_residual_int4_host` gives, on repeated
calls that reuse the shared array, and refuse vectors larger than the array.
"""
import ctypes

import numpy as np
import pytest

import oracle
from helpers import dev_qweight, rand_qweight, rand_vec, rel_err

pytestmark = pytest.mark.gpu


def _call(ctx, name, res, x, st, rows, cols):
    from managedllama2_b200 import _lib
    buf = res.copy()
    _lib.check(getattr(ctx._lib, name)(ctx.handle, buf.ctypes.data_as(ctypes.c_void_p), x.ctypes.data_as(ctypes.c_void_p),
                                       ctypes.byref(st), rows, cols))
    return buf


def test_static_scratch_matches_allocating_entry_point_twice():
    import torch
    import managedllama2_b200 as ml2
    ctx = ml2.CudaContext(0)
    rng = np.random.default_rng(2024)
    # two calls in a row with different shapes: the second reuses the array the first one filled
    for rows, cols in [(4096, 4096), (11008, 512)]:
        w, z, s = rand_qweight(rng, rows, cols)
        x, res = rand_vec(rng, rows), rand_vec(rng, cols)
        q = dev_qweight(w, z, s)
        st = q.struct()
        want = _call(ctx, "ml2_matvec_residual_int4_host", res, x, st, rows, cols)
        free_before = torch.cuda.mem_get_info()[0]
        got = _call(ctx, "ml2_matvec_residual_int4_host_static", res, x, st, rows, cols)
        assert torch.cuda.mem_get_info()[0] == free_before  # nothing was allocated on the device
        assert np.array_equal(got.view(np.uint16), want.view(np.uint16))
        assert rel_err(got, oracle.matvec_residual_int4(res, x, w, z, s, rows, cols, mode=1)) <= 1e-3
    assert ctx.status() == (0, 0)
    ctx.close()


def test_static_scratch_rejects_oversized_vectors():
    import managedllama2_b200 as ml2
    ctx = ml2.CudaContext(0)
    rng = np.random.default_rng(1)
    w, z, s = rand_qweight(rng, 128, 8)
    st = dev_qweight(w, z, s).struct()
    big = np.zeros(20000, np.float16)
    with pytest.raises(ml2.Ml2Error) as e:
        _call(ctx, "ml2_matvec_residual_int4_host_static", big, big, st, 16384 + 128, 8)
    assert "exceed" in str(e.value)
    ctx.close()
