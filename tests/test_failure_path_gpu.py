"""The bounded-wait error path of the persistent kernel, exercised without faulting or hanging the GPU.

A host-made condition (the launch number the operator counters are compared with is advanced by one, which is what a
tensor-parallel rank sees when a peer skipped a forward) makes the next forward's dependency waits impossible to meet.
With a short wait limit they run out after a fraction of a millisecond: the kernel records the error word and runs to
its end, the synchronising call returns ML2_E_DEVICE, further forwards are refused until ml2_model_reset, and after the
reset the model decodes correctly again (checked against the CPU oracle).
"""
import numpy as np
import pytest

import oracle

pytestmark = pytest.mark.gpu


def test_wait_runs_out_then_reset_recovers():
    import managedllama2_b200 as ml2
    from managedllama2_b200 import _lib

    cfg = ml2.Config(dim=256, hiddenDim=768, numLayers=2, numHeads=2, numKVHeads=2, vocabSize=512, seqLength=32)
    ctx = ml2.CudaContext(0)
    tr = ml2.Transformer(cfg, ml2.synthetic_weights(ctx, cfg, seed=5, sigma=1.0), ctx)
    hw = ml2.synthetic_weights_host(cfg, seed=5, sigma=1.0)
    cpu = oracle.CpuModel(dict(dim=cfg.dim, hidden_dim=cfg.hiddenDim, n_layers=cfg.numLayers, n_heads=cfg.numHeads,
                               n_kv_heads=cfg.numKVHeads, vocab_size=cfg.vocabSize, seq_len=cfg.seqLength,
                               rope_theta=cfg.ropeTheta), hw, mode=1)
    tokens = [9, 100, 301, 17]
    tr.set_tokens(np.array(tokens, dtype=np.int32))
    if tr.launches_per_token != 0:
        pass
    # two healthy tokens first
    for pos in range(2):
        tr.Forward(pos, pos + 1, False)
        got = tr.logits().astype(np.float32)
        want = cpu.forward(tokens[pos], pos).astype(np.float32)
        assert float(np.abs(got - want).max()) <= 2e-2 * want.std()
    assert tr.launches_per_token == 1, "the persistent kernel is the path under test"

    ctx.set_wait_limit(400_000)          # about 0.2 ms at 1.9 GHz
    _lib.check(tr.lib.ml2_model_debug_skip_launch(tr.handle))
    tr.Forward(2, 3, False)              # its waits cannot be met: they run out, the kernel returns
    with pytest.raises(_lib.Ml2Error) as e:
        tr.synchronize()
    assert e.value.code == -4            # ML2_E_DEVICE
    with pytest.raises(_lib.Ml2Error) as e:
        tr.Forward(2, 3, False)          # refused until the reset
    assert e.value.code == -3            # ML2_E_STATE

    tr.reset()
    ctx.set_wait_limit(4_000_000_000)
    assert ctx.status() == (0, 0)
    # the cache rows of positions 0 and 1 are intact; position 2 is simply run again
    for pos in range(2, 4):
        tr.Forward(pos, pos + 1, False)
        got = tr.logits().astype(np.float32)
        want = cpu.forward(tokens[pos], pos).astype(np.float32)
        assert float(np.abs(got - want).max()) <= 2e-2 * want.std(), pos
    assert ctx.status() == (0, 0)
    tr.close()
    ctx.close()
