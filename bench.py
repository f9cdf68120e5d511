#!/usr/bin/env python
"""Decode benchmark: batch-1 greedy decoding of a Llama-2-13B-shape AWQ int4 (group 128) model.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl ours|reference] [--config 13b|7b]

A step is one decoded token (one pass of the per-token operator sequence + the greedy sample). With
--gpus N > 1 the script is started once per GPU by torch.distributed.run and the model runs tensor
parallel over the N ranks (total work fixed: strong scaling). Rank 0 prints ONE JSON line.

  value     tokens/s with everything resident on the device (CUDA events on the model's stream)
  e2e       tokens/s through the host-buffer API: per step the token id goes host->device (4 B, pinned),
            the forward runs, and the sampled id comes back device->host (4 B), as a host-driven loop does
  roofline  the dominant kernel (gate/up int4 mat-vec + SwiGLU) timed alone over all layers
  kernels   the same for every kernel kind
  cpu_baseline  the CPU oracle (C restatement of the reference's C# CPU code) on this box's cores, on a
            bounded sample (a few layers) extrapolated to one token

--impl reference times that CPU restatement as the reference arm (the reference's C# cannot be built
here and its CUDA kernels are not a CPU implementation).
"""
import argparse
import ctypes
import json
import os
import subprocess
import sys
import threading
import time

import numpy as np

ROOT = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, ROOT)

CONFIGS = {
    # BASELINE configs[3] / configs[2]
    "13b": dict(dim=5120, hiddenDim=13824, numLayers=40, numHeads=40, numKVHeads=40, vocabSize=32000),
    "7b": dict(dim=4096, hiddenDim=11008, numLayers=32, numHeads=32, numKVHeads=32, vocabSize=32000),
}
PROMPT_LEN = 16
SEED = 31415


def measured_peak_gbs():
    p = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.exists(p):
        try:
            return float(json.load(open(p))["hbm_gbs"]), "measured"
        except Exception:
            pass
    return 6650.0, "fallback"


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


def token_bytes(cfg, tp=1):
    """Algorithmic bytes one token reads on one rank (weights + classifier + norms + embedding row), KV excluded."""
    def qw(rows, cols):
        ss = -(-rows // 128)
        return cols * ((-(-rows // 32)) * 16 + (-(-ss // 8)) * 4 + ss * 2)
    d, h, L, V = cfg["dim"], cfg["hiddenDim"], cfg["numLayers"], cfg["vocabSize"]
    per_layer = 3 * qw(d, d // tp) + qw(d // tp, d) + 2 * qw(d, h // tp) + qw(h // tp, d) + 2 * d * 2
    return L * per_layer + (V // tp) * d * 2 + d * 2 + d * 2


# --------------------------------------------------------------------------------------------------
# CPU arm: the oracle (C restatement of the reference's C# CPU reference) on the host cores
# --------------------------------------------------------------------------------------------------
def cpu_layer_sampler(cfg, threads):
    """Returns (run_layer, run_classifier): closures timing one layer's mat-vec set / the classifier on the CPU."""
    import oracle
    import managedllama2_b200 as ml2
    oracle.set_threads(threads)
    c = ml2.Config(seqLength=64, **cfg)
    one = ml2.Config(dim=c.dim, hiddenDim=c.hiddenDim, numLayers=1, numHeads=c.numHeads, numKVHeads=c.numKVHeads,
                     vocabSize=256, seqLength=64)
    hw = ml2.synthetic_weights_host(one, seed=SEED)
    L = hw["layers"][0]
    rng = np.random.default_rng(1)
    x = rng.standard_normal(c.dim).astype(np.float16)
    hvec = (rng.standard_normal(c.hiddenDim) * 0.1).astype(np.float16)
    cls = (rng.standard_normal((2000, c.dim)) * 0.02).astype(np.float16)  # a 2000-row slice of the classifier

    def run_layer():
        # the seven int4 mat-vecs of one layer in the C# reference arithmetic (unpack to fp16, fp32 dot) + norms
        xb = oracle.rmsnorm(x, L["rms_att"])
        oracle.qkv_matvec_int4(xb, L["q"], L["k"], L["v"], c.dim, c.dim, mode=0)
        oracle.matvec_residual_int4(x, xb, *L["o"], c.dim, c.dim, mode=0)
        xb = oracle.rmsnorm(x, L["rms_ffn"])
        oracle.matvec_swiglu_int4(xb, L["gate"], L["up"], c.dim, c.hiddenDim, mode=0)
        oracle.matvec_residual_int4(x, hvec, *L["down"], c.hiddenDim, c.dim, mode=0)

    def run_classifier_slice():
        oracle.matvec_f16(x, cls, c.dim, cls.shape[0])

    return run_layer, run_classifier_slice, cls.shape[0]


def cpu_tokens_per_s(cfg, threads, layer_reps):
    run_layer, run_cls, cls_rows = cpu_layer_sampler(cfg, threads)
    run_layer()
    t0 = time.perf_counter()
    for _ in range(layer_reps):
        run_layer()
    t_layer = (time.perf_counter() - t0) / layer_reps
    t0 = time.perf_counter()
    run_cls()
    t_cls = (time.perf_counter() - t0) * cfg["vocabSize"] / cls_rows
    return 1.0 / (cfg["numLayers"] * t_layer + t_cls), t_layer, t_cls


def run_reference_arm(args, cfg, rank, world):
    if rank != 0:
        return
    threads = os.cpu_count() or 1
    run_layer, run_cls, cls_rows = cpu_layer_sampler(cfg, threads)
    for _ in range(max(args.warmup, 1) if args.warmup < 3 else 3):
        run_layer()
    # a step = a bounded sample of one token: `sample_layers` layers' mat-vecs, scaled to all layers + classifier
    t0 = time.perf_counter()
    run_cls()
    t_cls = (time.perf_counter() - t0) * cfg["vocabSize"] / cls_rows
    budget_s = 150.0
    times = []
    start = time.perf_counter()
    for _ in range(args.steps):
        t0 = time.perf_counter()
        run_layer()
        times.append(time.perf_counter() - t0)
        if time.perf_counter() - start > budget_s:
            break
    t_layer = float(np.mean(times))
    ms_token = (cfg["numLayers"] * t_layer + t_cls) * 1e3
    value = 1e3 / ms_token
    sample = "per step: the 7 int4 mat-vecs + 2 RMSNorms of one layer (C# reference arithmetic: unpack to fp16, fp32 dot), " \
             "x%d layers + classifier (timed on %d of %d rows) = one token; %d of %d steps run" % (
                 cfg["numLayers"], cls_rows, cfg["vocabSize"], len(times), args.steps)
    line = {
        "impl": "reference", "metric": "decode tokens/s batch-1", "value": value, "unit": "tokens/s", "n_gpus": args.gpus,
        "steps": len(times), "warmup": args.warmup, "ms_per_step": ms_token, "higher_is_better": True, "scaling": "strong",
        "vs_baseline": None, "dtype": "int4 weights, fp16 activations, fp32 accumulate", "data": "synthetic",
        "config": {"workload": "llama2-%s-shape AWQ int4 g128 batch-1 greedy decode, CPU reference arithmetic" % args.config},
        "cpu_baseline": {"value": value, "unit": "tokens/s", "cores": threads, "kind": "port", "sample": sample},
        "e2e": {"value": value, "unit": "tokens/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
        "gpu_launches": 0,
    }
    print(json.dumps(line), flush=True)


# --------------------------------------------------------------------------------------------------
# GPU arm
# --------------------------------------------------------------------------------------------------
def run_gpu_arm(args, cfg, rank, world, local_rank):
    import torch
    import managedllama2_b200 as ml2
    from managedllama2_b200 import _lib

    torch.cuda.set_device(local_rank)
    dist = None
    nccl_id = None
    if world > 1:
        import torch.distributed as dist_mod
        dist = dist_mod
        dist.init_process_group("nccl", rank=rank, world_size=world, device_id=torch.device("cuda", local_rank))
        idt = torch.zeros(128, dtype=torch.uint8, device="cuda")
        if rank == 0:
            idt = torch.frombuffer(bytearray(ml2.Transformer.nccl_unique_id()), dtype=torch.uint8).cuda()
        dist.broadcast(idt, 0)
        nccl_id = bytes(idt.cpu().numpy().tobytes())

    seq_len = max(PROMPT_LEN, args.context) + args.warmup + 2 * args.steps + 8
    config = ml2.Config(seqLength=seq_len, **cfg)
    ctx = ml2.CudaContext(local_rank)
    weights = ml2.synthetic_weights(ctx, config, seed=SEED, tp_size=world, tp_rank=rank)
    tr = ml2.Transformer(config, weights, ctx, tp_size=world, tp_rank=rank, nccl_id=nccl_id)
    if dist is not None and os.environ.get("ML2_TP_FUSED", "1") == "1":
        tr.attach_peers_with(dist)   # persistent kernel per GPU, all-reduce fused over peer memory
    sp = ctypes.c_void_p()
    _lib.check(tr.lib.ml2_model_stream(tr.handle, ctypes.byref(sp)))
    stream = torch.cuda.ExternalStream(sp.value)

    rng = np.random.default_rng(SEED)
    prompt = rng.integers(3, config.vocabSize, size=PROMPT_LEN).astype(np.int32)
    tr.set_tokens(prompt)

    def barrier():
        if dist is not None:
            dist.barrier()
        torch.cuda.synchronize()

    # prompt (token by token, as the reference does) + warm-up decode steps
    pos = 0
    for _ in range(PROMPT_LEN - 1):
        tr.Forward(pos, pos + 1, False)
        pos += 1
    if args.context > pos:
        # long-context timing aid (BASELINE configs[4]): continue from position `context`; the cache rows in between hold
        # whatever the allocation held, the attention still reads and weighs all of them
        pos = args.context
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
    e0.record(stream)
    for _ in range(args.steps):
        tr.Forward(pos, pos + 1, True)
        pos += 1
    e1.record(stream)
    tr.synchronize()
    barrier()
    launches = ctx.launch_count - launches0
    ms = e0.elapsed_time(e1)
    if dist is not None:
        t = torch.tensor([ms], device="cuda")
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        ms = float(t.item())

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
    e2e_ms = (time.perf_counter() - t0) * 1e3
    if dist is not None:
        t = torch.tensor([e2e_ms], device="cuda")
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        e2e_ms = float(t.item())
    clocks = sampler.stop() if rank == 0 else None

    # ---- per-operator kernels timed alone (every kernel's achieved GB/s) -------------------------------
    avg_us = (ctypes.c_double * 6)()
    nbytes = (ctypes.c_double * 6)()
    _lib.check(tr.lib.ml2_model_profile(tr.handle, 5, avg_us, nbytes))
    status = ctx.status()
    final_pos = pos

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
        except Exception as e:  # the reference arm is informative only
            ref_cuda = {"unavailable": repr(e)[:200]}

    if rank == 0:
        peak, peak_kind = measured_peak_gbs()
        names = ["qkv_rope", "attention", "o_proj", "gate_up_swiglu", "down", "classifier"]
        kernels = {n: {"us": avg_us[i], "GB/s": nbytes[i] / avg_us[i] * 1e-3, "bytes": nbytes[i],
                       "frac_of_%s_peak" % peak_kind: nbytes[i] / avg_us[i] * 1e-3 / peak,
                       "frac_of_8TBps": nbytes[i] / avg_us[i] * 1e-3 / 8000.0} for i, n in enumerate(names)}
        tokens_per_s = args.steps / ms * 1e3
        tb = token_bytes(cfg, world)
        persistent = tr.launches_per_token == 1
        if persistent:
            # one persistent kernel per token: it is the dominant (only) kernel; its launch duration is the step time
            mid = final_pos - args.steps - args.steps // 2          # mean position of the device-timed region
            kv = cfg["numLayers"] * 2 * (mid + 1) * (cfg["dim"] // world) * 2
            dom_name = "decode_token_kernel (persistent, whole token)"
            dom_bytes = tb + kv
            achieved = dom_bytes / (ms / args.steps * 1e-3) / 1e9
        else:
            dom = 3
            dom_name = "stream_matvec_kernel<Int4,SwiGLU,RMSNorm> (gate/up)"
            dom_bytes = nbytes[dom]
            achieved = nbytes[dom] / avg_us[dom] * 1e-3
        threads = os.cpu_count() or 1
        if world == 1 and not args.no_cpu:
            cpu_val, t_layer, t_cls = cpu_tokens_per_s(cfg, threads, 3)
            cpu_baseline = {"value": cpu_val, "unit": "tokens/s", "cores": threads, "kind": "port",
                            "sample": "3 repetitions of one layer's 7 int4 mat-vecs (C# reference arithmetic) x %d layers + "
                                      "classifier slice scaled to %d rows" % (cfg["numLayers"], cfg["vocabSize"])}
        else:
            cpu_baseline = None
        line = {
            "metric": "decode tokens/s batch-1", "value": tokens_per_s, "unit": "tokens/s", "n_gpus": world, "steps": args.steps,
            "warmup": args.warmup, "ms_per_step": ms / args.steps, "higher_is_better": True, "scaling": "strong",
            "vs_baseline": None, "dtype": "int4 weights, fp16 activations, fp32 accumulate", "data": "synthetic",
            "config": {"workload": "llama2-%s-shape%s AWQ int4 g128, batch-1 greedy decode, %d-token prompt then decode" %
                                   (args.config, (" cut to %d layers" % args.layers) if args.layers else "", PROMPT_LEN) +
                                   ((" from position %d" % args.context) if args.context else ""),
                       "parallelism": "tp%d" % world, "l2": "per-token working set %.2f GB per GPU, far larger than L2" % (tb / 1e9),
                       "bytes_per_token_per_gpu": tb},
            "hbm_frac_of_token": {"achieved_GB/s": tb * tokens_per_s / 1e9, "of_%s_peak" % peak_kind: tb * tokens_per_s / 1e9 / peak,
                                  "of_8TBps": tb * tokens_per_s / 1e9 / 8000.0},
            "e2e": {"value": args.steps / e2e_ms * 1e3, "unit": "tokens/s", "h2d_bytes_per_step": 4, "d2h_bytes_per_step": 4},
            "gpu_launches": int(launches),
            "roofline": {"bound": "hbm", "kernel": dom_name, "achieved": achieved, "peak": peak, "unit": "GB/s",
                         "frac": achieved / peak, "peak_kind": peak_kind, "algorithmic_bytes_per_launch": dom_bytes,
                         "frac_of_8TBps": achieved / 8000.0,
                         # dram__bytes_read+write of one launch: ncu capture of the 8-layer case (1.6597 GB moved for
                         # 1.6496 GB algorithmic), scaled by the bytes of this launch
                         "traffic": (dom_bytes * 1.00612) if persistent else None,
                         "traffic_source": "ncu dram bytes of the 8-layer capture x (bytes of this launch / bytes of that launch)"},
            "kernels_timed_alone": kernels,
            "reference_cuda_kernels": ref_cuda,
            "cpu_baseline": cpu_baseline,
            "clocks": clocks,
            "device_status": list(status),
        }
        print(json.dumps(line), flush=True)
    tr.close()
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
    ap.add_argument("--context", type=int, default=0, help="profiling aid: time the decode steps from this position on (long-context case)")
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
