"""Host-side logic of the tensor-parallel split with two gloo ranks on the CPU: each rank runs the oracle on its
shard (column shards of QKV / gate / up, row shards of o-proj / down), partials are all-reduced in fp32 and rounded
once; the result must match the unsharded oracle."""
import os
import sys

import numpy as np
import pytest


def _worker(rank, world, port, q):
    import ctypes
    import torch
    import torch.distributed as dist
    sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
    import managedllama2_b200 as ml2
    from managedllama2_b200 import _lib
    import oracle
    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    dist.init_process_group("gloo", rank=rank, world_size=world)
    lib = ml2.load()
    dim, hidden, seed = 512, 5 * 128, 3          # 5 hidden groups over 2 ranks: 3 + 2
    cfg = ml2.Config(dim, hidden, 1, 4, 4, 64, 8)
    dim_local, hg0, hng, _, _ = ml2.tp_shapes(cfg, world, rank)

    def gen(tid, rows_full, col0, ncols, g0, ng):
        rows = ng * 128
        w_, z_, s_ = ml2.qweight_sizes(rows)
        w, z, s = np.empty(ncols * w_, np.uint32), np.empty(ncols * z_, np.uint32), np.empty(ncols * s_, np.float16)
        _lib.check(lib.ml2_synth_qweight_host(w.ctypes.data_as(ctypes.c_void_p), z.ctypes.data_as(ctypes.c_void_p),
                                              s.ctypes.data_as(ctypes.c_void_p), rows_full, col0, ncols, g0, ng,
                                              ctypes.c_uint64(seed), ctypes.c_uint32(tid)))
        return w, z, s

    rng = np.random.default_rng(0)
    x = (rng.standard_normal(dim) * 0.5).astype(np.float16)
    res = rng.standard_normal(dim).astype(np.float16)
    # gate/up column shard -> local slice of h; down row shard -> fp32 partial; all-reduce; one rounding
    g = gen(1, dim, hg0 * 128, hng * 128, 0, dim // 128)
    u = gen(2, dim, hg0 * 128, hng * 128, 0, dim // 128)
    h_local = oracle.matvec_swiglu_int4(x, g, u, dim, hng * 128, mode=1)
    d = gen(3, hidden, 0, dim, hg0, hng)
    part = oracle.matvec_int4_f32(h_local, *d, hng * 128, dim, mode=1)
    t = torch.from_numpy(part.copy())
    dist.all_reduce(t)
    got = (res.astype(np.float32) + t.numpy()).astype(np.float16)
    # every rank ends with identical bits
    chk = torch.from_numpy(got.view(np.int16).astype(np.int32))
    lo, hi = chk.clone(), chk.clone()
    dist.all_reduce(lo, op=dist.ReduceOp.MIN)
    dist.all_reduce(hi, op=dist.ReduceOp.MAX)
    same = bool((lo == hi).all())
    if rank == 0:
        gf, uf = gen(1, dim, 0, hidden, 0, dim // 128), gen(2, dim, 0, hidden, 0, dim // 128)
        hf = oracle.matvec_swiglu_int4(x, gf, uf, dim, hidden, mode=1)
        df = gen(3, hidden, 0, dim, 0, hidden // 128)
        want = oracle.matvec_residual_int4(res, hf, *df, hidden, dim, mode=1)
        den = np.maximum(np.abs(want.astype(np.float64)), np.sqrt(np.mean(want.astype(np.float64) ** 2)))
        err = float(np.max(np.abs(got.astype(np.float64) - want.astype(np.float64)) / den))
        q.put((same, err, hng))
    dist.barrier()
    dist.destroy_process_group()


def test_two_rank_sharded_ffn_matches_unsharded():
    import torch.multiprocessing as mp
    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    port = 29511
    procs = [ctx.Process(target=_worker, args=(r, 2, port, q)) for r in range(2)]
    for p in procs:
        p.start()
    same, err, hng = q.get(timeout=120)
    for p in procs:
        p.join(timeout=60)
        assert p.exitcode == 0
    assert same
    assert hng == 3
    assert err <= 1e-3


def _lockstep_worker(rank, world, port, q):
    import torch.distributed as dist
    sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
    from managedllama2_b200.transformer import tp_forward_counts_agree
    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    dist.init_process_group("gloo", rank=rank, world_size=world)
    ok_equal = tp_forward_counts_agree(dist, 7)
    # rank 1 "skipped" a forward: every rank must find out on the host, before any launch
    try:
        tp_forward_counts_agree(dist, 8 if rank == 0 else 7)
        caught = False
    except RuntimeError as e:
        caught = "out of step" in str(e)
    q.put((rank, ok_equal, caught))
    dist.barrier()
    dist.destroy_process_group()


def test_ranks_out_of_step_are_found_on_the_host():
    """Host rule of the fused tensor-parallel path: all ranks call Forward the same number of times. A rank that skips
    one would leave its peers' kernels waiting for arrivals that never come (they give up after the wait limit); the
    check finds the mismatch on the host, with no GPU involved."""
    import torch.multiprocessing as mp
    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    procs = [ctx.Process(target=_lockstep_worker, args=(r, 2, 29512, q)) for r in range(2)]
    for p in procs:
        p.start()
    got = sorted(q.get(timeout=120) for _ in range(2))
    for p in procs:
        p.join(timeout=60)
        assert p.exitcode == 0
    assert got == [(0, True, True), (1, True, True)]
