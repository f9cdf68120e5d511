"""Tensor-parallel worker (started by torch.distributed.run, one process per GPU): runs the sharded model for a few
tokens and, on rank 0, compares the logits with the CPU oracle of the unsharded model."""
import os
import sys

import numpy as np

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
# unit-scale embeddings and norm weights: attention scores of order one, so a wrong score or cache row shows in the logits
SIGMA = 1.0
sys.path.insert(0, ROOT)


def main():
    import torch
    import torch.distributed as dist
    import managedllama2_b200 as ml2
    import oracle

    rank, world, local = int(os.environ["RANK"]), int(os.environ["WORLD_SIZE"]), int(os.environ["LOCAL_RANK"])
    torch.cuda.set_device(local)
    dist.init_process_group("nccl", rank=rank, world_size=world, device_id=torch.device("cuda", local))
    idt = torch.zeros(128, dtype=torch.uint8, device="cuda")
    if rank == 0:
        idt = torch.frombuffer(bytearray(ml2.Transformer.nccl_unique_id()), dtype=torch.uint8).cuda()
    dist.broadcast(idt, 0)
    if os.environ.get("ML2_TP_SHAPE") == "13b":
        # the benchmark's shape cut to 2 layers: 40 heads and 108 hidden groups, so 8 ranks see 5 heads and 14 / 13 groups
        cfg = ml2.Config(dim=5120, hiddenDim=13824, numLayers=2, numHeads=40, numKVHeads=40, vocabSize=32000, seqLength=40)
    else:
        # 8 heads, 13 hidden groups: uneven hidden split for 2, 4 and 8 ranks
        cfg = ml2.Config(dim=1024, hiddenDim=13 * 128, numLayers=2, numHeads=8, numKVHeads=8, vocabSize=512, seqLength=40)
    ctx = ml2.CudaContext(local)
    model_bin = os.environ.get("ML2_TP_MODEL_BIN")
    if model_bin:
        # every rank cuts its shard out of one model.bin (rank 0 writes it in the reference's layout)
        sys.path.insert(0, os.path.dirname(os.path.abspath(__file__)))
        from helpers import write_model_bin
        if rank == 0:
            write_model_bin(model_bin, cfg, ml2.synthetic_weights_host(cfg, seed=21, sigma=SIGMA))
        dist.barrier()
        tr = ml2.Transformer.FromFile(model_bin, ctx, tp_size=world, tp_rank=rank, nccl_id=idt.cpu().numpy().tobytes())
    else:
        w = ml2.synthetic_weights(ctx, cfg, seed=21, tp_size=world, tp_rank=rank, sigma=SIGMA)
        tr = ml2.Transformer(cfg, w, ctx, tp_size=world, tp_rank=rank, nccl_id=idt.cpu().numpy().tobytes())
    if os.environ.get("ML2_TP_FUSED", "1") == "1":
        tr.attach_peers_with(dist)   # one persistent kernel per token, all-reduce over peer memory
    toks = [5, 99, 256, 31]
    steps = 8 if os.environ.get("ML2_TP_SHAPE") == "13b" else 12
    tr.set_tokens(np.array(toks, dtype=np.int32))
    cpu = None
    if rank == 0:
        hw = ml2.synthetic_weights_host(cfg, seed=21, sigma=SIGMA)
        cpu = oracle.CpuModel(dict(dim=cfg.dim, hidden_dim=cfg.hiddenDim, n_layers=cfg.numLayers, n_heads=cfg.numHeads,
                                   n_kv_heads=cfg.numKVHeads, vocab_size=cfg.vocabSize, seq_len=cfg.seqLength,
                                   rope_theta=cfg.ropeTheta), hw, mode=1)
    ok = True
    if os.environ.get("ML2_TP_LATE") == "1":
        # Failure made on the host: rank 0 calls Forward long after the others. Their kernels wait for its partial sums
        # until the (shortened) wait limit runs out, record the error word and run to their end; rank 0's kernel then waits
        # in vain for theirs. Every rank must see ML2_E_DEVICE (not a fault), reset, and go on with correct tokens.
        import time
        ctx.set_wait_limit(400_000_000)   # about 0.2 s of SM clock
        dist.barrier()
        if rank == 0:
            time.sleep(1.5)
        failed = False
        try:
            tr.Forward(0, 1, False)
            tr.synchronize()
        except ml2.Ml2Error as e:
            failed = e.code == -4   # ML2_E_DEVICE
        refused = False
        try:
            tr.Forward(0, 1, False)
        except ml2.Ml2Error as e:
            refused = True
        f = torch.tensor([1 if (failed and refused) else 0], device="cuda")
        dist.all_reduce(f, op=dist.ReduceOp.MIN)
        ok = ok and f.item() == 1
        if rank == 0 and f.item() != 1:
            print("late rank: expected ML2_E_DEVICE and a refused forward on every rank", flush=True)
        dist.barrier()
        tr.reset()
        ctx.set_wait_limit(4_000_000_000)
        dist.barrier()
    for pos in range(steps):
        gen = pos + 1 >= len(toks)
        # every rank launches its token together: a rank's kernel waits for the others' partial sums only as long as the
        # context's wait limit allows, and rank 0 spends seconds in the CPU oracle between steps
        dist.barrier()
        tr.Forward(pos, pos + 1, gen)
        logits = tr.logits()
        # every rank must hold the same logits bit for bit
        t = torch.from_numpy(logits.view(np.int16).astype(np.int32)).cuda()
        lo, hi = t.clone(), t.clone()
        dist.all_reduce(lo, op=dist.ReduceOp.MIN)
        dist.all_reduce(hi, op=dist.ReduceOp.MAX)
        same = bool((lo == hi).all().item())
        if not same and rank == 0:
            print("step", pos, "ranks disagree on", int((lo != hi).sum().item()), "logits", flush=True)
        ok = ok and same
        if gen:
            toks.append(tr.read_token(pos + 1))
        if rank == 0:
            want = cpu.forward(toks[pos], pos).astype(np.float32)
            err = float(np.abs(logits.astype(np.float32) - want).max())
            # rounding level: a few per cent of the logits' standard deviation (summation orders differ between the sharded
            # kernel and the oracle and flip fp16 roundings of the activations); a sharding mistake gives 30 % and more
            tol = 3e-2 * want.std()
            if not err <= tol:
                print("step", pos, "max error", err, "tolerance", tol, "status", ctx.status(), flush=True)
            ok = ok and err <= tol
    ok = ok and ctx.status() == (0, 0)
    flag = torch.tensor([1 if ok else 0], device="cuda")
    dist.all_reduce(flag, op=dist.ReduceOp.MIN)
    tr.close()
    dist.barrier()
    dist.destroy_process_group()
    if rank == 0:
        print("TP_OK" if flag.item() == 1 else "TP_FAIL", "world", world, flush=True)
    sys.exit(0 if flag.item() == 1 else 1)


if __name__ == "__main__":
    main()
