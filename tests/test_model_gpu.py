"""Whole-token parity: the fused per-token graph against the CPU oracle's Transformer.Forward composition.

The reference has no runnable model-level test (test/TransformerTests.cs:8-23 is skipped and needs a real
checkpoint), so the arbiter is the oracle's forward (oracle/ml2_oracle.c: orc_forward), which follows
src/Transformer.cs:158-190 with an fp16 store wherever the reference kernels store fp16.

Tolerances: logits within 1e-2 absolute of the reference arithmetic and identical greedy
tokens; here the logits are also held to 2e-2 relative to their own spread, which is much tighter.
"""
import os

import numpy as np
import pytest

import oracle

pytestmark = pytest.mark.gpu


def small_config(ml2, seq=48):
    return ml2.Config(dim=256, hiddenDim=768, numLayers=3, numHeads=2, numKVHeads=2, vocabSize=512, seqLength=seq)


def oracle_model(ml2, cfg, seed):
    hw = ml2.synthetic_weights_host(cfg, seed=seed)
    ocfg = dict(dim=cfg.dim, hidden_dim=cfg.hiddenDim, n_layers=cfg.numLayers, n_heads=cfg.numHeads,
                n_kv_heads=cfg.numKVHeads, vocab_size=cfg.vocabSize, seq_len=cfg.seqLength, rope_theta=cfg.ropeTheta)
    return oracle.CpuModel(ocfg, hw, mode=1), hw


def test_synthetic_device_equals_host():
    import managedllama2_b200 as ml2
    cfg = small_config(ml2)
    ctx = ml2.CudaContext(0)
    dw = ml2.synthetic_weights(ctx, cfg, seed=7)
    hw = ml2.synthetic_weights_host(cfg, seed=7)
    assert np.array_equal(dw.tokenEmbeddingTable.cpu().numpy().view(np.uint16), hw["embed"].view(np.uint16))
    assert np.array_equal(dw.classifierWeights.cpu().numpy().view(np.uint16), hw["classifier"].view(np.uint16))
    for l in range(cfg.numLayers):
        L, H = dw.layers[l], hw["layers"][l]
        for name, key in (("queryWeight", "q"), ("outputWeight", "o"), ("gateWeight", "gate"), ("upWeight", "up"),
                          ("downWeight", "down")):
            q = getattr(L, name)
            assert np.array_equal(q.Weight.cpu().numpy().view(np.uint32), H[key][0]), (l, name)
            assert np.array_equal(q.Zeros.cpu().numpy().view(np.uint32), H[key][1]), (l, name)
            assert np.array_equal(q.Scales.cpu().numpy().view(np.uint16), H[key][2].view(np.uint16)), (l, name)
        assert np.array_equal(L.rmsAttentionWeight.cpu().numpy().view(np.uint16), H["rms_att"].view(np.uint16))
    # value distributions of the random-init construction the benchmark uses
    s = hw["layers"][0]["q"][2].astype(np.float32)
    assert 0.00099 <= s.min() and s.max() <= 0.02001
    e = hw["embed"].astype(np.float32)
    assert abs(e.std() - 0.02) < 0.002 and abs(e.mean()) < 0.001
    ctx.close()


@pytest.mark.parametrize("mode", ["persistent", "graph", "eager"])
def test_greedy_decode_matches_oracle(mode):
    """The three ways the per-token sequence can run: one persistent kernel, a CUDA graph of per-operator kernels,
    or those kernels launched eagerly. All must match the oracle."""
    import managedllama2_b200 as ml2
    env = {"persistent": {}, "graph": {"ML2_NO_MEGA": "1"}, "eager": {"ML2_NO_MEGA": "1", "ML2_NO_GRAPH": "1"}}[mode]
    os.environ.update(env)
    try:
        cfg = small_config(ml2)
        ctx = ml2.CudaContext(0)
        tr = ml2.Transformer(cfg, ml2.synthetic_weights(ctx, cfg, seed=11), ctx)
    finally:
        for k in env:
            os.environ.pop(k, None)
    cpu, _ = oracle_model(ml2, cfg, 11)
    rng = np.random.default_rng(3)
    prompt = rng.integers(3, cfg.vocabSize, size=8).astype(np.int32)
    steps = 32
    tr.set_tokens(prompt)
    tokens = list(prompt)
    worst = 0.0
    for pos in range(steps):
        generate = pos + 1 >= len(prompt)
        tr.Forward(pos, pos + 1, generate)
        got = tr.logits().astype(np.float32)
        want = cpu.forward(tokens[pos], pos).astype(np.float32)
        spread = want.std()
        err = np.abs(got - want).max()
        worst = max(worst, err / spread)
        assert err <= 1e-2, (pos, err)
        assert err <= 2e-2 * spread, (pos, err, spread)
        if generate:
            tok = tr.read_token(pos + 1)
            # greedy token: equal to the oracle's unless the oracle's own top two are within the logits error
            o = oracle.argmax(want.astype(np.float16))
            if tok != o:
                top2 = np.sort(want)[-2:]
                assert top2[1] - top2[0] <= 2 * err + 1e-7, (pos, tok, o)
            tokens.append(tok)
    assert tr.launches_per_token == (1 if mode == "persistent" else 5 * cfg.numLayers + 3)
    err, _ = ctx.status()
    assert err == 0
    tr.close()
    ctx.close()


def test_generate_host_api_and_determinism():
    import managedllama2_b200 as ml2
    cfg = small_config(ml2)
    ctx = ml2.CudaContext(0)
    tr = ml2.Transformer(cfg, ml2.synthetic_weights(ctx, cfg, seed=5), ctx)
    prompt = np.array([5, 17, 300, 44], dtype=np.int32)
    a = tr.Generate(prompt, 40)
    b = tr.Generate(prompt, 40)
    assert a == b and len(a) > 0
    assert a[:3] == [17, 300, 44]  # prompt tokens are yielded as they are consumed (src/Transformer.cs:102-109)
    tr.close()
    ctx.close()


def test_long_sequence_cluster_path():
    """A sequence of 400 positions (one CTA per head in the persistent kernel) against the oracle."""
    import managedllama2_b200 as ml2
    cfg = ml2.Config(dim=256, hiddenDim=384, numLayers=1, numHeads=2, numKVHeads=2, vocabSize=256, seqLength=400)
    ctx = ml2.CudaContext(0)
    tr = ml2.Transformer(cfg, ml2.synthetic_weights(ctx, cfg, seed=2), ctx)
    cpu, _ = oracle_model(ml2, cfg, 2)
    rng = np.random.default_rng(1)
    toks = rng.integers(3, cfg.vocabSize, size=cfg.seqLength).astype(np.int32)
    tr.set_tokens(toks)
    for pos in range(cfg.seqLength - 1):
        tr.Forward(pos, pos + 1, False)
        want = cpu.forward(toks[pos], pos).astype(np.float32)
        if pos in (0, 127, 128, 129, 200, 257, 398):
            got = tr.logits().astype(np.float32)
            assert np.abs(got - want).max() <= 2e-2 * want.std(), pos
    tr.close()
    ctx.close()


@pytest.mark.parametrize("heads", [2, 5])
def test_split_attention_in_the_persistent_kernel(heads):
    """Several CTAs per head (the long-context path of the persistent kernel), forced on from the second position so
    that parts without any cache row, one-row parts and uneven parts all occur; logits against the oracle."""
    import managedllama2_b200 as ml2
    cfg = ml2.Config(dim=128 * heads, hiddenDim=384, numLayers=2, numHeads=heads, numKVHeads=heads, vocabSize=256, seqLength=300)
    ctx = ml2.CudaContext(0)
    tr = ml2.Transformer(cfg, ml2.synthetic_weights(ctx, cfg, seed=6), ctx)
    tr.set_split_attention_from(2)
    cpu, _ = oracle_model(ml2, cfg, 6)
    rng = np.random.default_rng(3)
    toks = rng.integers(3, cfg.vocabSize, size=cfg.seqLength).astype(np.int32)
    tr.set_tokens(toks)
    for pos in range(cfg.seqLength - 1):
        tr.Forward(pos, pos + 1, False)
        want = cpu.forward(toks[pos], pos).astype(np.float32)
        if pos < 20 or pos in (31, 32, 63, 64, 100, 167, 255, 298):
            got = tr.logits().astype(np.float32)
            assert np.abs(got - want).max() <= 2e-2 * want.std(), pos
    assert ctx.status() == (0, 0)
    tr.close()
    ctx.close()


@pytest.mark.parametrize("mode", ["persistent", "persistent_split", "graph", "eager"])
def test_peaked_attention_matches_oracle(mode):
    """Weights of unit scale (embeddings and norm weights ~ N(0, 1)) give attention scores of order one, so the
    softmax is far from uniform and a wrong score, rotation or cache row shows in the logits at once; with the small
    weights of the benchmark construction every position gets nearly the same probability and such an error hides."""
    import managedllama2_b200 as ml2
    env = {"persistent": {}, "persistent_split": {}, "graph": {"ML2_NO_MEGA": "1"},
           "eager": {"ML2_NO_MEGA": "1", "ML2_NO_GRAPH": "1"}}[mode]
    os.environ.update(env)
    try:
        cfg = ml2.Config(dim=384, hiddenDim=640, numLayers=2, numHeads=3, numKVHeads=3, vocabSize=320, seqLength=200)
        ctx = ml2.CudaContext(0)
        tr = ml2.Transformer(cfg, ml2.synthetic_weights(ctx, cfg, seed=13, sigma=1.0), ctx)
        if mode == "persistent_split":
            tr.set_split_attention_from(2)
    finally:
        for k in env:
            os.environ.pop(k, None)
    hw = ml2.synthetic_weights_host(cfg, seed=13, sigma=1.0)
    cpu = oracle.CpuModel(dict(dim=cfg.dim, hidden_dim=cfg.hiddenDim, n_layers=cfg.numLayers, n_heads=cfg.numHeads,
                               n_kv_heads=cfg.numKVHeads, vocab_size=cfg.vocabSize, seq_len=cfg.seqLength,
                               rope_theta=cfg.ropeTheta), hw, mode=1)
    rng = np.random.default_rng(5)
    toks = rng.integers(3, cfg.vocabSize, size=cfg.seqLength).astype(np.int32)
    tr.set_tokens(toks)
    for pos in range(cfg.seqLength - 1):
        tr.Forward(pos, pos + 1, False)
        want = cpu.forward(toks[pos], pos).astype(np.float32)
        if pos < 12 or pos % 16 == 0 or pos in (127, 128, 129, 198):
            got = tr.logits().astype(np.float32)
            assert np.abs(got - want).max() <= 2e-2 * want.std(), (mode, pos)
    assert ctx.status() == (0, 0)
    tr.close()
    ctx.close()


def test_step_host_equals_forward_and_read():
    """ml2_model_step_host (token in from host memory, step, token out) gives the tokens of Forward + read_token."""
    import ctypes
    import torch
    import managedllama2_b200 as ml2
    from managedllama2_b200 import _lib
    cfg = small_config(ml2)
    ctx = ml2.CudaContext(0)
    w = ml2.synthetic_weights(ctx, cfg, seed=8, sigma=1.0)
    a, b = ml2.Transformer(cfg, w, ctx), ml2.Transformer(cfg, w, ctx)
    a.set_tokens(np.array([7], np.int32))
    pinned = torch.zeros(1, dtype=torch.int32).pin_memory()
    out = ctypes.c_int(0)
    tok_a, tok_b = 7, 7
    for pos in range(20):
        a.set_tokens(np.array([tok_a], np.int32), first=pos)
        a.Forward(pos, pos + 1, True)
        tok_a = a.read_token(pos + 1)
        pinned[0] = tok_b
        _lib.check(b.lib.ml2_model_step_host(b.handle, pos, ctypes.c_void_p(pinned.data_ptr()), ctypes.byref(out)))
        tok_b = out.value
        assert tok_a == tok_b, pos
    a.close()
    b.close()
    ctx.close()


def test_long_context_to_4096_through_the_split_attention():
    """The longest context of the benchmark configurations (4096 positions) on a small model: one CTA per head up to 703
    cache rows, several CTAs per head from 704 on (the default threshold). Logits against the oracle around the switch
    and over the last 64 positions; unit-scale weights, so the attention is peaked and every cache row matters."""
    import managedllama2_b200 as ml2
    cfg = ml2.Config(dim=256, hiddenDim=384, numLayers=1, numHeads=2, numKVHeads=2, vocabSize=256, seqLength=4096)
    ctx = ml2.CudaContext(0)
    tr = ml2.Transformer(cfg, ml2.synthetic_weights(ctx, cfg, seed=17, sigma=1.0), ctx)
    hw = ml2.synthetic_weights_host(cfg, seed=17, sigma=1.0)
    cpu = oracle.CpuModel(dict(dim=cfg.dim, hidden_dim=cfg.hiddenDim, n_layers=cfg.numLayers, n_heads=cfg.numHeads,
                               n_kv_heads=cfg.numKVHeads, vocab_size=cfg.vocabSize, seq_len=cfg.seqLength,
                               rope_theta=cfg.ropeTheta), hw, mode=1)
    rng = np.random.default_rng(9)
    toks = rng.integers(3, cfg.vocabSize, size=cfg.seqLength).astype(np.int32)
    tr.set_tokens(toks)
    checked = 0
    for pos in range(cfg.seqLength - 1):
        tr.Forward(pos, pos + 1, False)
        want = cpu.forward(toks[pos], pos).astype(np.float32)
        if pos in (0, 1, 702, 703, 704, 705, 1500, 2047, 2048) or pos >= 4031:
            got = tr.logits().astype(np.float32)
            assert np.abs(got - want).max() <= 2e-2 * want.std(), pos
            checked += 1
    assert checked >= 70 and tr.launches_per_token == 1
    assert ctx.status() == (0, 0)
    tr.close()
    ctx.close()
