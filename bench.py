#!/usr/bin/env python
"""Decode benchmark: batch-1 greedy decoding of a Llama-2-13B-shape AWQ int4 (group 128) model.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl ours|reference] [--config 13b|7b]

A step is one decoded token (one pass of the per-token operator sequence + the greedy sample). With
--gpus N > 1 the script is started once per GPU by torch.distributed.run and the model runs tensor
parallel over the N ranks (total work fixed: strong scaling). Rank 0 prints ONE JSON line.

  value          tokens/s with everything resident on the device (CUDA events on the model's stream)
  e2e            tokens/s through the host-buffer API: per step the token id goes host->device (4 B, pinned),
                 the forward runs, and the sampled id comes back device->host (4 B), as a host-driven loop does
  roofline       the persistent per-token kernel: algorithmic bytes of one launch / its duration
  long_context   the same decode after a 4032-token prompt prefilled token by token (64 steps up to position 4096)
  matvec_single  one 4096 -> 4096 int4 mat-vec over 32 rotating weight sets (independent launches and a chain with
                 programmatic dependent launch), and the mat-vec set of one 7B-shape layer
  kernels_timed_alone   every per-operator kernel of the graph path swept over all layers, chained as that path runs them
  tp_check       (N > 1) a 2-layer cut of the same shape, sharded like the timed model, against the CPU oracle
  cpu_baseline   the CPU oracle (C restatement of the reference's C# CPU code) on this box's cores: whole tokens

--impl reference times that CPU restatement on whole tokens of the same configuration (the reference's C# cannot be
built here and its CUDA kernels are not a CPU implementation); it needs neither a GPU nor the product library.
"""
import argparse
import ctypes
import hashlib
import json
import os
import re
import subprocess
import sys
import threading
import time

import numpy as np

ROOT = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, ROOT)

CONFIGS = {
    "13b": dict(dim=5120, hiddenDim=13824, numLayers=40, numHeads=40, numKVHeads=40, vocabSize=32000),
    "7b": dict(dim=4096, hiddenDim=11008, numLayers=32, numHeads=32, numKVHeads=32, vocabSize=32000),
}
PROMPT_LEN = 16
LONG_PROMPT = 4032
LONG_STEPS = 64
SEED = 31415


def measured_peak_gbs():
    p = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.exists(p):
        try:
            return float(json.load(open(p))["hbm_gbs"]), "measured"
        except Exception:
            pass
    return 6650.0, "fallback"


def profiled_traffic_ratio():
    """DRAM bytes moved per algorithmic byte of the persistent kernel, from the kept ncu summary (None when absent)."""
    p = os.path.join(ROOT, "profiles", "decode_token_kernel_13b_8layers.md")
    try:
        m = re.search(r"dram_bytes_per_algorithmic_byte\s*=\s*([0-9.]+)", open(p).read())
        return float(m.group(1)) if m else None
    except Exception:
        return None


class ClockSampler:
    """Samples SM clocks and throttle reasons with nvidia-smi while the timed region runs."""

    def __init__(self, index):
        self.index = index
        self.proc = None
        self.lines = []

    def start(self):
        q = ("clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.hw_slowdown,clocks_event_reasons.hw_thermal_slowdown,"
             "clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap")
        try:
            self.proc = subprocess.Popen(["nvidia-smi", "-i", str(self.index), "--query-gpu=" + q, "--format=csv,noheader,nounits",
                                          "-lms", "100"], stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True)
            threading.Thread(target=self._read, daemon=True).start()
        except Exception:
            self.proc = None

    def _read(self):
        for line in self.proc.stdout:
            self.lines.append(line.strip())

    def stop(self):
        if not self.proc:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["nvidia-smi unavailable"]}
        self.proc.terminate()
        try:
            self.proc.wait(timeout=5)
        except Exception:
            self.proc.kill()
        sm, mx, reasons = [], [], set()
        names = ["hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"]
        for ln in self.lines:
            f = [x.strip() for x in ln.split(",")]
            if len(f) < 7:
                continue
            try:
                sm.append(float(f[0]))
                mx.append(float(f[1]))
            except ValueError:
                continue
            for n, v in zip(names, f[3:7]):
                if v.lower().startswith("active"):
                    reasons.add(n)
        if not sm:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["no samples"]}
        return {"sm_mhz": float(np.median(sm)), "sm_max_mhz": max(mx), "reasons": sorted(reasons), "samples": len(sm)}


def qweight_bytes(rows, cols):
    ss = -(-rows // 128)
    return cols * ((-(-rows // 32)) * 16 + (-(-ss // 8)) * 4 + ss * 2)


def token_bytes(cfg, tp=1):
    """Algorithmic bytes one token reads on one rank (weights + classifier + norms + embedding row), KV excluded."""
    d, h, L, V = cfg["dim"], cfg["hiddenDim"], cfg["numLayers"], cfg["vocabSize"]
    per_layer = 3 * qweight_bytes(d, d // tp) + qweight_bytes(d // tp, d) + 2 * qweight_bytes(d, h // tp) + qweight_bytes(h // tp, d) + 2 * d * 2
    return L * per_layer + (V // tp) * d * 2 + d * 2 + d * 2


def config_block(args, cfg, world):
    """The `config` object of the JSON line: the same for both arms of one command line."""
    tb = token_bytes(cfg, world)
    return {"workload": "llama2-%s-shape%s AWQ int4 g128, batch-1 greedy decode, %d-token prompt then decode" %
                        (args.config, (" cut to %d layers" % args.layers) if args.layers else "", PROMPT_LEN) +
                        ((" from position %d" % args.context) if args.context else ""),
            "parallelism": "tp%d" % world, "l2": "per-token working set %.2f GB per GPU, far larger than L2" % (tb / 1e9),
            "bytes_per_token_per_gpu": tb}


def oracle_cfg(cfg, seq_len):
    return dict(dim=cfg["dim"], hidden_dim=cfg["hiddenDim"], n_layers=cfg["numLayers"], n_heads=cfg["numHeads"],
                n_kv_heads=cfg["numKVHeads"], vocab_size=cfg["vocabSize"], seq_len=seq_len, rope_theta=10000.0)


# --------------------------------------------------------------------------------------------------
# CPU arm: the oracle (C restatement of the reference's C# CPU reference) on the host cores, WHOLE tokens
# --------------------------------------------------------------------------------------------------
def cpu_whole_tokens(cfg, threads, max_tokens, budget_s, warm_tokens=0):
    """Decodes whole tokens of `cfg` with the oracle in the reference's CPU arithmetic (every weight unpacked to fp16,
    sequential fp32 dot: test/MatVecInt4Tests.cs:48-70 with src/QWeight.cs:29-54), `threads` threads over output rows.
    Returns (seconds per token list, seconds spent building the model)."""
    import oracle
    oracle.build()
    oracle.set_threads(threads)
    t0 = time.perf_counter()
    oc = oracle_cfg(cfg, 64)
    model = oracle.CpuModel(oc, oracle.synthetic_weights(oc, seed=SEED), mode=0)
    t_build = time.perf_counter() - t0
    rng = np.random.default_rng(SEED)
    toks = rng.integers(3, cfg["vocabSize"], size=64)
    pos = 0
    for _ in range(warm_tokens):
        model.forward(int(toks[pos]), pos)
        pos += 1
    times = []
    start = time.perf_counter()
    while len(times) < max_tokens:
        t0 = time.perf_counter()
        model.forward(int(toks[pos]), pos)
        times.append(time.perf_counter() - t0)
        pos += 1
        if time.perf_counter() - start > budget_s:
            break
    return times, t_build


def cpu_single_thread_small_cases():
    """The reference's CPU arithmetic on ONE thread, as the reference runs it: one 4096 -> 4096 int4 mat-vec and the
    seven mat-vecs of a 7B-shape layer (QKV, o-proj with residual, gate/up with SwiGLU, down with residual)."""
    import oracle
    oracle.set_threads(1)
    rng = np.random.default_rng(7)

    def qw(rows, cols):
        nw, nz, ns = oracle.qweight_sizes(rows)
        return (rng.integers(0, 1 << 32, size=cols * nw, dtype=np.uint32), rng.integers(0, 1 << 32, size=cols * nz, dtype=np.uint32),
                (0.001 + 0.019 * rng.random(cols * ns, dtype=np.float32)).astype(np.float16))
    d, h = 4096, 11008
    x = rng.standard_normal(d).astype(np.float16)
    res = rng.standard_normal(d).astype(np.float16)
    hv = (rng.standard_normal(h) * 0.1).astype(np.float16)
    a = qw(d, d)
    oracle.matvec_residual_int4(res, x, *a, d, d, mode=0)
    t0 = time.perf_counter()
    oracle.matvec_residual_int4(res, x, *a, d, d, mode=0)
    t_one = time.perf_counter() - t0
    q, k, v, o, g, u, dn = qw(d, d), qw(d, d), qw(d, d), a, qw(d, h), qw(d, h), qw(h, d)
    t0 = time.perf_counter()
    oracle.qkv_matvec_int4(x, q, k, v, d, d, mode=0)
    oracle.matvec_residual_int4(res, x, *o, d, d, mode=0)
    oracle.matvec_swiglu_int4(x, g, u, d, h, mode=0)
    oracle.matvec_residual_int4(res, hv, *dn, h, d, mode=0)
    t_layer = time.perf_counter() - t0
    return {"threads": 1, "matvec_4096x4096_ms": t_one * 1e3, "matvec_4096x4096_GB/s": qweight_bytes(d, d) / t_one / 1e9,
            "layer_7b_shape_ms": t_layer * 1e3}


def run_reference_arm(args, cfg, rank, world):
    """Whole tokens on the CPU; the printed `steps` is the number of tokens actually decoded (ms_per_step x steps is the
    timed wall-clock)."""
    if rank != 0:
        return
    threads = os.cpu_count() or 1
    # a 13B-shape token takes tens of seconds on a few cores: run what fits a few minutes, at least one token
    times, t_build = cpu_whole_tokens(cfg, threads, max_tokens=max(1, args.steps), budget_s=150.0, warm_tokens=0)
    ms_token = float(np.mean(times)) * 1e3
    value = 1e3 / ms_token
    sample = ("%d whole token(s) of the %s shape through the oracle's Transformer.Forward composition in the C# reference "
              "arithmetic (unpack every weight to fp16, sequential fp32 dot), %d threads over output rows; model built in "
              "%.0f s (not timed); no warm-up token (each costs as much as a timed one)" % (len(times), args.config, threads, t_build))
    line = {
        "impl": "reference", "metric": "decode tokens/s batch-1", "value": value, "unit": "tokens/s", "n_gpus": args.gpus,
        "steps": len(times), "warmup": 0, "ms_per_step": ms_token, "higher_is_better": True, "scaling": "strong",
        "vs_baseline": None, "dtype": "int4 weights, fp16 activations, fp32 accumulate", "data": "synthetic",
        "config": config_block(args, cfg, max(1, args.gpus)),
        "cpu_baseline": {"value": value, "unit": "tokens/s", "cores": threads, "kind": "port", "sample": sample},
        "e2e": {"value": value, "unit": "tokens/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
        "gpu_launches": 0,
    }
    print(json.dumps(line), flush=True)


# --------------------------------------------------------------------------------------------------
# GPU arm
# --------------------------------------------------------------------------------------------------
def time_matvec_single(ctx, torch, ml2, peak, peak_kind):
    """One int4 mat-vec alone (4096 -> 4096, residual epilogue), over 32 distinct weight sets (279 MB, more than twice
    the L2) visited in rotation: as independent launches and as a chain with programmatic dependent launch; then the
    mat-vec set of one 7B-shape layer per round over 8 distinct layers (841 MB)."""
    rng = np.random.default_rng(3)
    d, h = 4096, 11008

    def dev_qw(rows, cols):
        nw, nz, ns = (-(-rows // 32)) * 4, -(-(-(-rows // 128)) // 8), -(-rows // 128)
        w = torch.randint(0, 1 << 31, (cols * nw,), dtype=torch.int32, device="cuda")
        z = torch.randint(0, 1 << 31, (cols * nz,), dtype=torch.int32, device="cuda")
        s = (0.001 + 0.019 * torch.rand(cols * ns, device="cuda")).to(torch.float16)
        return ml2.QWeight(w, z, s)

    x = torch.from_numpy(rng.standard_normal(d).astype(np.float16)).cuda()
    hv = torch.from_numpy((rng.standard_normal(h) * 0.1).astype(np.float16)).cuda()
    outs = [torch.zeros(d, dtype=torch.float16, device="cuda") for _ in range(2)]
    sets = [dev_qw(d, d) for _ in range(32)]
    mv = ml2.MatVecResidual(ctx)
    out = {}
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    for name, pdl in (("independent_launches", False), ("pdl_chain", True)):
        ctx.set_pdl(pdl)
        for q in sets:                       # warm-up round
            mv.Forward(outs[0], x, q, d, d)
        ctx.synchronize()
        rounds = 6
        e0.record()
        for _ in range(rounds):
            for q in sets:
                mv.Forward(outs[0], x, q, d, d)
        e1.record()
        torch.cuda.synchronize()
        us = e0.elapsed_time(e1) * 1e3 / (rounds * len(sets))
        b = qweight_bytes(d, d) + 2 * d + 2 * 2 * d
        out[name] = {"us_per_matvec": us, "GB/s": b / us * 1e-3, "frac_of_8TBps": b / us * 1e-3 / 8000.0,
                     "frac_of_%s_peak" % peak_kind: b / us * 1e-3 / peak}
    # one 7B-shape layer's mat-vec set per round
    layers = [dict(q=dev_qw(d, d), k=dev_qw(d, d), v=dev_qw(d, d), o=dev_qw(d, d), g=dev_qw(d, h), u=dev_qw(d, h), dn=dev_qw(h, d))
              for _ in range(8)]
    cfg1 = ml2.Config(dim=d, hiddenDim=h, numLayers=1, numHeads=32, numKVHeads=32, vocabSize=32, seqLength=4)
    qkv, sw = ml2.QKVMatVec(ctx, cfg1), ml2.MatVecSwiGLU(ctx)
    qo, ko, vo = (torch.zeros(d * 4, dtype=torch.float16, device="cuda") for _ in range(3))
    hout = torch.zeros(h, dtype=torch.float16, device="cuda")

    def layer_set(L):
        qkv.Forward(qo, ko, vo, x, L["q"], L["k"], L["v"], d, d, 0, 0)
        mv.Forward(outs[0], x, L["o"], d, d)
        sw.Forward(hout, x, L["g"], L["u"], d, h)
        mv.Forward(outs[1], hv, L["dn"], h, d)
    for L in layers:
        layer_set(L)
    ctx.synchronize()
    e0.record()
    for _ in range(4):
        for L in layers:
            layer_set(L)
    e1.record()
    torch.cuda.synchronize()
    us = e0.elapsed_time(e1) * 1e3 / (4 * len(layers))
    b = 4 * qweight_bytes(d, d) + 2 * qweight_bytes(d, h) + qweight_bytes(h, d)
    out["layer_7b_shape_pdl_chain"] = {"us_per_layer_set": us, "GB/s": b / us * 1e-3, "frac_of_8TBps": b / us * 1e-3 / 8000.0,
                                       "frac_of_%s_peak" % peak_kind: b / us * 1e-3 / peak}
    ctx.set_pdl(False)
    out["how"] = ("ml2_matvec_residual_int4 / ml2_qkv_matvec_int4 / ml2_matvec_swiglu_int4 (stream_matvec_kernel), CUDA events on "
                  "the context's stream, distinct weights every launch (working set far larger than L2)")
    return out


def run_gpu_arm(args, cfg, rank, world, local_rank):
    import torch
    import managedllama2_b200 as ml2
    from managedllama2_b200 import _lib

    torch.cuda.set_device(local_rank)
    dist = None
    if world > 1:
        import torch.distributed as dist_mod
        dist = dist_mod
        dist.init_process_group("nccl", rank=rank, world_size=world, device_id=torch.device("cuda", local_rank))

    def fresh_nccl_id():
        """A unique id serves ONE communicator: every model gets its own, made on rank 0 and broadcast."""
        if dist is None:
            return None
        idt = torch.zeros(128, dtype=torch.uint8, device="cuda")
        if rank == 0:
            idt = torch.frombuffer(bytearray(ml2.Transformer.nccl_unique_id()), dtype=torch.uint8).cuda()
        dist.broadcast(idt, 0)
        return bytes(idt.cpu().numpy().tobytes())

    fused = os.environ.get("ML2_TP_FUSED", "1") == "1"
    ctx = ml2.CudaContext(local_rank)

    def barrier():
        if dist is not None:
            dist.barrier()
        torch.cuda.synchronize()

    def max_over_ranks(v):
        if dist is None:
            return v
        t = torch.tensor([v], device="cuda", dtype=torch.float64)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        return float(t.item())

    # ---- correctness of the sharded path before anything is timed (N > 1): 2 layers of the same shape -------------
    tp_check = None
    if world > 1:
        import oracle
        c2 = dict(cfg)
        c2["numLayers"] = 2
        conf2 = ml2.Config(seqLength=16, **c2)
        w2 = ml2.synthetic_weights(ctx, conf2, seed=SEED + 1, tp_size=world, tp_rank=rank, sigma=1.0)
        t2 = ml2.Transformer(conf2, w2, ctx, tp_size=world, tp_rank=rank, nccl_id=fresh_nccl_id())
        if fused:
            t2.attach_peers_with(dist)
        toks = [11, 4242, 31999 % conf2.vocabSize, 77]
        t2.set_tokens(np.array(toks, dtype=np.int32))
        cpu = None
        if rank == 0:
            oracle.set_threads(os.cpu_count() or 1)
            cpu = oracle.CpuModel(oracle_cfg(c2, 16), ml2.synthetic_weights_host(conf2, seed=SEED + 1, sigma=1.0), mode=1)
        identical, max_err, ok = True, 0.0, True
        for pos in range(4):
            dist.barrier()   # ranks launch a token together (rank 0 spends seconds in the CPU oracle between tokens)
            t2.Forward(pos, pos + 1, False)
            lg = t2.logits()
            t = torch.from_numpy(lg.view(np.int16).astype(np.int32)).cuda()
            lo, hi = t.clone(), t.clone()
            dist.all_reduce(lo, op=dist.ReduceOp.MIN)
            dist.all_reduce(hi, op=dist.ReduceOp.MAX)
            identical = identical and bool((lo == hi).all().item())
            if rank == 0:
                want = cpu.forward(toks[pos], pos).astype(np.float32)
                err = float(np.abs(lg.astype(np.float32) - want).max())
                max_err = max(max_err, err / max(float(want.std()), 1e-9))
        # max over 4 x 32000 logits, in units of their standard deviation. Rounding level is a few per cent (different
        # summation orders flip fp16 roundings of the activations: measured 2.2e-2 at 2 ranks, 1.2e-2 for the unsharded
        # persistent kernel, 5e-3 for the per-operator kernels on the same tokens); a sharding mistake gives 0.3 and more
        ok = identical and max_err <= 5e-2 and ctx.status() == (0, 0)
        tp_check = {"max_err_over_logit_std": max_err, "rank_identical": identical, "ok": bool(ok),
                    "what": "2-layer cut of the timed shape, unit-scale weights, 4 tokens, logits vs the CPU oracle of the unsharded model"}
        t2.close()
        del w2
        torch.cuda.empty_cache()

    seq_len = LONG_PROMPT + LONG_STEPS + 8 if not args.no_long else PROMPT_LEN + args.warmup + 2 * args.steps + 8
    seq_len = max(seq_len, max(PROMPT_LEN, args.context) + args.warmup + 2 * args.steps + 8)
    config = ml2.Config(seqLength=seq_len, **cfg)
    weights = ml2.synthetic_weights(ctx, config, seed=SEED, tp_size=world, tp_rank=rank)
    tr = ml2.Transformer(config, weights, ctx, tp_size=world, tp_rank=rank, nccl_id=fresh_nccl_id())
    if dist is not None and fused:
        tr.attach_peers_with(dist)   # persistent kernel per GPU, all-reduce fused over peer memory
    sp = ctypes.c_void_p()
    _lib.check(tr.lib.ml2_model_stream(tr.handle, ctypes.byref(sp)))
    stream = torch.cuda.ExternalStream(sp.value)

    rng = np.random.default_rng(SEED)
    prompt = rng.integers(3, config.vocabSize, size=PROMPT_LEN).astype(np.int32)
    tr.set_tokens(prompt)

    # prompt (token by token, as the reference does: src/Transformer.cs:96-104) + warm-up decode steps
    pos = 0
    for _ in range(PROMPT_LEN - 1):
        tr.Forward(pos, pos + 1, False)
        pos += 1
    if args.context > pos:
        # profiling aid only: prefill up to `context` token by token with seeded ids
        filler = rng.integers(3, config.vocabSize, size=args.context + 1).astype(np.int32)
        tr.set_tokens(filler[pos + 1:args.context + 1], first=pos + 1)
        while pos < args.context:
            tr.Forward(pos, pos + 1, False)
            pos += 1
    for _ in range(args.warmup):
        tr.Forward(pos, pos + 1, True)
        pos += 1
    tr.synchronize()

    sampler = ClockSampler(local_rank)
    if rank == 0:
        sampler.start()
        time.sleep(0.3)

    # ---- device-resident timed region: K decode steps, no host round trip --------------------------
    barrier()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    launches0 = ctx.launch_count
    first_timed = pos
    e0.record(stream)
    for _ in range(args.steps):
        tr.Forward(pos, pos + 1, True)
        pos += 1
    e1.record(stream)
    tr.synchronize()
    barrier()
    launches = ctx.launch_count - launches0
    ms = max_over_ranks(e0.elapsed_time(e1))
    # the greedy token ids of the timed steps: identical on every rank (checked). Between different N the hash can differ:
    # the logits of a random-init model are nearly flat, so one fp16 rounding flip (the sharded sums associate
    # differently) changes an arg-max within a few tokens; `tp_check` above is the numerical check of the sharded path
    ids = [tr.read_token(p) for p in range(first_timed + 1, first_timed + 1 + min(args.steps, 64))]
    token_hash = hashlib.sha256(np.array(ids, dtype=np.int32).tobytes()).hexdigest()[:16]
    tokens_identical = True
    if dist is not None:
        t_ids = torch.tensor(ids, dtype=torch.int32, device="cuda")
        lo_ids, hi_ids = t_ids.clone(), t_ids.clone()
        dist.all_reduce(lo_ids, op=dist.ReduceOp.MIN)
        dist.all_reduce(hi_ids, op=dist.ReduceOp.MAX)
        tokens_identical = bool((lo_ids == hi_ids).all().item())

    # ---- end to end: host-driven loop, token id in (pinned, 4 B) and sampled id out (4 B) per step ----
    pinned = torch.zeros(1, dtype=torch.int32).pin_memory()
    tok = tr.read_token(pos)
    barrier()
    t0 = time.perf_counter()
    out_tok = ctypes.c_int(0)
    for _ in range(args.steps):
        pinned[0] = tok
        # one C-ABI call per token: host -> device copy of this step's input token, the decode step, device -> host read
        # of the sampled token (blocking 4-byte read, src/Sampler.cs:69)
        _lib.check(tr.lib.ml2_model_step_host(tr.handle, pos, ctypes.c_void_p(pinned.data_ptr()), ctypes.byref(out_tok)))
        pos += 1
        tok = out_tok.value
    torch.cuda.synchronize()
    e2e_ms = max_over_ranks((time.perf_counter() - t0) * 1e3)
    clocks = sampler.stop() if rank == 0 else None
    short_mid = first_timed + args.steps // 2          # mean position of the device-timed region

    # ---- long context: a 4032-token prompt prefilled token by token, then 64 decode steps up to position 4096 ------
    long_ctx = None
    if not args.no_long and args.context == 0:
        lp = rng.integers(3, config.vocabSize, size=LONG_PROMPT).astype(np.int32)
        tr.set_tokens(lp)
        p2 = 0
        barrier()   # ranks start the prefill together: a sharded token waits for its peers only as long as the wait limit allows
        t0 = time.perf_counter()
        for _ in range(LONG_PROMPT - 1):
            tr.Forward(p2, p2 + 1, False)
            p2 += 1
        tr.synchronize()
        prefill_s = time.perf_counter() - t0
        for _ in range(3):                      # warm-up at this length (generated tokens continue the prompt)
            tr.Forward(p2, p2 + 1, True)
            p2 += 1
        barrier()
        l0, l1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        n_long = LONG_STEPS - 4
        l0.record(stream)
        for _ in range(n_long):
            tr.Forward(p2, p2 + 1, True)
            p2 += 1
        l1.record(stream)
        tr.synchronize()
        barrier()
        lms = max_over_ranks(l0.elapsed_time(l1)) / n_long
        mid = p2 - n_long // 2
        kvb = cfg["numLayers"] * 2 * (mid + 1) * (cfg["dim"] // world) * 2
        lb = token_bytes(cfg, world) + kvb
        peak, peak_kind = measured_peak_gbs()
        long_ctx = {"tokens/s": 1e3 / lms, "ms_per_step": lms, "steps": n_long, "positions": [p2 - n_long, p2 - 1],
                    "prefill": "%d prompt tokens, one forward each (%.1f s)" % (LONG_PROMPT, prefill_s),
                    "algorithmic_bytes_per_launch": lb, "kv_cache_bytes_read_per_launch": kvb,
                    "roofline_frac": lb / (lms * 1e-3) / 1e9 / peak, "peak_kind": peak_kind}

    # ---- per-operator kernels timed alone (graph-path kernels; every kernel's achieved GB/s) ------------------------
    barrier()
    tr.Forward(short_mid, short_mid + 1, False)       # the attention kernel is timed at the bench's mean position
    avg_us = (ctypes.c_double * 6)()
    nbytes = (ctypes.c_double * 6)()
    _lib.check(tr.lib.ml2_model_profile(tr.handle, 5, avg_us, nbytes))
    status = ctx.status()

    # ---- the reference's own CUDA kernels on the same weights (one GPU only) ----------------------------
    ref_cuda = None
    if world == 1 and rank == 0:
        try:
            from oracle import ref_cuda as rc
            if rc.available():
                ref = rc.RefTransformer(config, weights)
                ref.set_tokens(prompt)
                rpos = PROMPT_LEN + args.warmup
                for q in range(3):
                    ref.forward(rpos, rpos + 1, True)
                torch.cuda.synchronize()
                n_ref = min(args.steps, 16)
                r0, r1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
                r0.record()
                for q in range(n_ref):
                    ref.forward(rpos, rpos + 1, True)
                r1.record()
                torch.cuda.synchronize()
                eager_ms = r0.elapsed_time(r1) / n_ref
                g = torch.cuda.CUDAGraph()
                side = torch.cuda.Stream()
                with torch.cuda.graph(g, stream=side):
                    ref.forward(rpos, rpos + 1, True)
                g.replay()
                torch.cuda.synchronize()
                r0.record()
                for q in range(n_ref):
                    g.replay()
                r1.record()
                torch.cuda.synchronize()
                graph_ms = r0.elapsed_time(r1) / n_ref
                ref_cuda = {"tokens/s_graph_replay": 1e3 / graph_ms, "tokens/s_eager_launches": 1e3 / eager_ms,
                            "launches_per_token": 10 * config.numLayers + 4, "position": rpos,
                            "how": "reference native/*.cu compiled unmodified for sm_100a, launch shapes of src/*.cs, "
                                   "Transformer.Forward order; graph replay removes host launch overhead"}
        except Exception as e:  # this leg is informative only
            ref_cuda = {"unavailable": repr(e)[:200]}

    persistent = tr.launches_per_token == 1
    tr.close()
    del weights
    torch.cuda.empty_cache()

    if rank == 0:
        peak, peak_kind = measured_peak_gbs()
        names = ["qkv_rope", "attention", "o_proj", "gate_up_swiglu", "down", "classifier"]
        kernels = {n: {"us": avg_us[i], "GB/s": nbytes[i] / avg_us[i] * 1e-3, "bytes": nbytes[i],
                       "frac_of_%s_peak" % peak_kind: nbytes[i] / avg_us[i] * 1e-3 / peak,
                       "frac_of_8TBps": nbytes[i] / avg_us[i] * 1e-3 / 8000.0} for i, n in enumerate(names)}
        kernels["how"] = ("the per-operator kernels of the CUDA-graph path, swept over all layers (distinct weights every launch), "
                          "chained with programmatic dependent launch as that path runs them; attention at position %d" % short_mid)
        matvec_single = None
        if world == 1:
            try:
                matvec_single = time_matvec_single(ctx, torch, ml2, peak, peak_kind)
            except Exception as e:
                matvec_single = {"unavailable": repr(e)[:200]}
        tokens_per_s = args.steps / ms * 1e3
        tb = token_bytes(cfg, world)
        if persistent:
            # one persistent kernel per token: it is the dominant (only) kernel; its launch duration is the step time
            kv = cfg["numLayers"] * 2 * (short_mid + 1) * (cfg["dim"] // world) * 2
            dom_name = "decode_token_kernel (persistent, whole token)"
            dom_bytes = tb + kv
            achieved = dom_bytes / (ms / args.steps * 1e-3) / 1e9
        else:
            dom = 3
            dom_name = "stream_matvec_kernel<Int4,SwiGLU,RMSNorm> (gate/up)"
            dom_bytes = nbytes[dom]
            achieved = nbytes[dom] / avg_us[dom] * 1e-3
        ratio = profiled_traffic_ratio() if persistent else None
        threads = os.cpu_count() or 1
        cpu_baseline = None
        if world == 1 and not args.no_cpu:
            # whole tokens of the timed shape on all cores (one token is 10-30 s of CPU work), plus the one-thread small cases
            times, t_build = cpu_whole_tokens(cfg, threads, max_tokens=1, budget_s=30.0)
            cpu_baseline = {"value": 1.0 / float(np.mean(times)), "unit": "tokens/s", "cores": threads, "kind": "port",
                            "sample": "%d whole token(s) of the %s shape, C# reference arithmetic (unpack to fp16, sequential fp32 dot), "
                                      "%d threads over output rows; %.1f s per token" % (len(times), args.config, threads, float(np.mean(times))),
                            "single_thread": cpu_single_thread_small_cases()}
        line = {
            "metric": "decode tokens/s batch-1", "value": tokens_per_s, "unit": "tokens/s", "n_gpus": world, "steps": args.steps,
            "warmup": args.warmup, "ms_per_step": ms / args.steps, "higher_is_better": True, "scaling": "strong",
            "vs_baseline": None, "dtype": "int4 weights, fp16 activations, fp32 accumulate", "data": "synthetic",
            "config": config_block(args, cfg, world),
            "positions_timed": [first_timed, first_timed + args.steps - 1],
            "hbm_frac_of_token": {"achieved_GB/s": tb * tokens_per_s / 1e9, "of_%s_peak" % peak_kind: tb * tokens_per_s / 1e9 / peak,
                                  "of_8TBps": tb * tokens_per_s / 1e9 / 8000.0},
            "e2e": {"value": args.steps / e2e_ms * 1e3, "unit": "tokens/s", "h2d_bytes_per_step": 4, "d2h_bytes_per_step": 4},
            "gpu_launches": int(launches),
            "roofline": {"bound": "hbm", "kernel": dom_name, "achieved": achieved, "peak": peak, "unit": "GB/s",
                         "frac": achieved / peak, "peak_kind": peak_kind, "algorithmic_bytes_per_launch": dom_bytes,
                         "frac_of_8TBps": achieved / 8000.0,
                         "traffic": (dom_bytes * ratio) if ratio else None,
                         "traffic_source": ("ncu dram bytes per algorithmic byte of the kept 8-layer capture (profiles/) x the bytes of this launch"
                                            if ratio else "not measured in this run")},
            "long_context": long_ctx,
            "matvec_single": matvec_single,
            "kernels_timed_alone": kernels,
            "reference_cuda_kernels": ref_cuda,
            "cpu_baseline": cpu_baseline,
            "tp_check": tp_check,
            "greedy_token_hash": token_hash,
            "greedy_tokens_identical_on_all_ranks": tokens_identical,
            "clocks": clocks,
            "device_status": list(status),
        }
        print(json.dumps(line), flush=True)
    ctx.close()
    if dist is not None:
        dist.barrier()
        dist.destroy_process_group()


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=256)
    ap.add_argument("--warmup", type=int, default=16)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--config", default="13b", choices=sorted(CONFIGS))
    ap.add_argument("--layers", type=int, default=0, help="profiling aid: run the shape with fewer layers (smaller device footprint)")
    ap.add_argument("--no-cpu", action="store_true", help="profiling aid: skip the CPU baseline leg")
    ap.add_argument("--no-long", action="store_true", help="profiling aid: skip the long-context leg")
    ap.add_argument("--context", type=int, default=0, help="profiling aid: prefill to this position (token by token) before the timed steps")
    args = ap.parse_args()
    if args.warmup < 3:
        args.warmup = 3
    rank = int(os.environ.get("RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    local_rank = int(os.environ.get("LOCAL_RANK", "0"))
    cfg = dict(CONFIGS[args.config])
    if args.layers > 0:
        cfg["numLayers"] = args.layers
    if args.impl == "reference":
        run_reference_arm(args, cfg, rank, world)
        return
    if world != args.gpus:
        if args.gpus > 1:
            raise SystemExit("--gpus %d needs torch.distributed.run with --nproc-per-node %d" % (args.gpus, args.gpus))
    run_gpu_arm(args, cfg, rank, world, local_rank)


if __name__ == "__main__":
    main()
