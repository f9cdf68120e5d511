"""Two contexts in one process, one per GPU (skipped on a single GPU): every entry point makes its context's device
current itself, so a caller that switched the current device in between still launches on the right GPU with the right
buffers (the reference binds one CudaContext per process and has no such case)."""
import ctypes

import numpy as np
import pytest

import oracle
from helpers import dev_qweight, rand_qweight, rand_vec, rel_err

pytestmark = pytest.mark.gpu


def _residual_host(ctx, res, x, st, rows, cols):
    from managedllama2_b200 import _lib
    buf = res.copy()
    _lib.check(ctx._lib.ml2_matvec_residual_int4_host(ctx.handle, buf.ctypes.data_as(ctypes.c_void_p), x.ctypes.data_as(ctypes.c_void_p),
                                                      ctypes.byref(st), rows, cols))
    return buf


def test_calls_land_on_their_contexts_device_whatever_device_is_current():
    import torch
    import managedllama2_b200 as ml2
    if torch.cuda.device_count() < 2:
        pytest.skip("needs 2 GPUs")
    rows, cols = 4096, 1024
    rng = np.random.default_rng(77)
    cases = []
    for dev in (0, 1):
        w, z, s = rand_qweight(rng, rows, cols)
        x, res = rand_vec(rng, rows), rand_vec(rng, cols)
        with torch.cuda.device(dev):
            q = dev_qweight(w, z, s)            # this matrix lives on GPU `dev`
            ctx = ml2.CudaContext(dev)
        cases.append((dev, ctx, q, x, res, oracle.matvec_residual_int4(res, x, w, z, s, rows, cols, mode=1)))
    # call each context while the OTHER GPU is the current device of the thread
    for dev, ctx, q, x, res, want in cases:
        torch.cuda.set_device(1 - dev)
        got = _residual_host(ctx, res, x, q.struct(), rows, cols)
        assert rel_err(got, want) <= 1e-3, dev
        got = _residual_host(ctx, res, x, q.struct(), rows, cols)       # and again, attributes and scratch cached per device
        assert rel_err(got, want) <= 1e-3, dev
        assert ctx.status() == (0, 0)
    torch.cuda.set_device(0)
    for _, ctx, *_ in cases:
        ctx.close()
