"""The sampling chain (Sampler.Sample, src/Sampler.cs:40-70) through the C ABI: each step against the numpy oracle with
the inputs of the reference's own tests (test/SoftmaxLogitsTests.cs, SortTests.cs, CumulativeSumTests.cs,
SampleTopPTests.cs), against the reference's own kernels where they are built, and the chain as a whole.

Tolerances: index work (sort order, carried ids, picked token) is exact; probabilities and cumulative sums are fp16
values of fp32 sums whose association differs between implementations, so they may differ by one fp16 step; sums of
integers (the reference's cumulative-sum test) are exact.
"""
import numpy as np
import pytest

import oracle
from helpers import to_dev, to_host

pytestmark = pytest.mark.gpu


@pytest.fixture(scope="module")
def ctx():
    import managedllama2_b200 as ml2
    c = ml2.CudaContext(0)
    yield c
    assert c.status() == (0, 0)
    c.close()


@pytest.fixture(scope="module")
def ref():
    from oracle import ref_cuda
    if not ref_cuda.available():
        pytest.skip("reference kernels not built (make -C oracle ref)")
    import managedllama2_b200 as ml2
    return ref_cuda.RefModules(ml2.Config(5120, 13824, 1, 40, 40, 32000, 64))


def half_steps(a, b):
    """Distance in fp16 steps between two arrays of non-negative fp16 values."""
    return np.abs(a.view(np.uint16).astype(np.int32) - b.view(np.uint16).astype(np.int32))


def dev_i32(a):
    import torch
    return torch.from_numpy(np.ascontiguousarray(a, np.int32)).cuda()


@pytest.mark.parametrize("size,temperature", [(16, 1.0), (16, 0.5), (1000, 0.7), (32000, 0.5), (32000, 1.0), (32003, 1.3)])
def test_softmax_logits(ctx, size, temperature):
    """test/SoftmaxLogitsTests.cs:75-91 (16 values in [0,1), temperature 1) and vocabulary-sized inputs."""
    import torch
    import managedllama2_b200 as ml2
    rng = np.random.default_rng(size)
    x = rng.random(size).astype(np.float16) if size == 16 else (rng.standard_normal(size) * 3).astype(np.float16)
    d = to_dev(x)
    idx = torch.full((size,), -1, dtype=torch.int32, device="cuda")
    ml2.SoftmaxLogits(ctx).Forward(d, size, temperature, idx)
    want, want_idx = oracle.softmax_logits(x, temperature)
    got = to_host(d)
    assert np.array_equal(idx.cpu().numpy(), want_idx)
    assert half_steps(got, want).max() <= 1
    assert abs(float(got.astype(np.float32).sum()) - 1.0) < 2e-2


@pytest.mark.parametrize("size", [1, 2, 17, 1000, 4096, 32000, 32768])
def test_sort_is_descending_and_stable(ctx, size):
    """test/SortTests.cs:52-70 (integers 0..1023 as fp16, so many ties) at several sizes; ids exact (stable order)."""
    import managedllama2_b200 as ml2
    rng = np.random.default_rng(size)
    keys = rng.integers(0, 1024, size).astype(np.float16)
    vals = rng.permutation(size).astype(np.int32)
    dk, dv = to_dev(keys), dev_i32(vals)
    ml2.Sort(ctx).Forward(dk, dv, size)
    wk, wv = oracle.sort_desc(keys, vals)
    assert np.array_equal(to_host(dk).view(np.uint16), wk.view(np.uint16))
    assert np.array_equal(dv.cpu().numpy(), wv)


def test_sort_signed_keys(ctx):
    import managedllama2_b200 as ml2
    rng = np.random.default_rng(3)
    keys = (rng.standard_normal(5000) * 100).astype(np.float16)
    vals = np.arange(5000, dtype=np.int32)
    dk, dv = to_dev(keys), dev_i32(vals)
    ml2.Sort(ctx).Forward(dk, dv, 5000)
    wk, wv = oracle.sort_desc(keys, vals)
    assert np.array_equal(to_host(dk).view(np.uint16), wk.view(np.uint16)) and np.array_equal(dv.cpu().numpy(), wv)


@pytest.mark.parametrize("size", [1, 31, 1025, 32000])
def test_cumulative_sum_of_integers_is_exact(ctx, size):
    """test/CumulativeSumTests.cs:58-75: integers in [-1000, 1000] as fp16; expected = sequential fp32 sum -> fp16."""
    import managedllama2_b200 as ml2
    rng = np.random.default_rng(size)
    x = rng.integers(-1000, 1001, size).astype(np.float16)
    d = to_dev(x)
    ml2.CumulativeSum(ctx).Forward(d, size)
    assert np.array_equal(to_host(d).view(np.uint16), oracle.cumulative_sum(x).view(np.uint16))


def test_cumulative_sum_of_probabilities(ctx):
    import managedllama2_b200 as ml2
    rng = np.random.default_rng(8)
    p, _ = oracle.softmax_logits((rng.standard_normal(32000) * 3).astype(np.float16), 0.5)
    p, _ = oracle.sort_desc(p, np.arange(32000))
    d = to_dev(p)
    ml2.CumulativeSum(ctx).Forward(d, 32000)
    assert half_steps(to_host(d), oracle.cumulative_sum(p)).max() <= 1


def test_sample_top_p_reference_case_and_edges(ctx):
    """test/SampleTopPTests.cs:49-64: 16 values in [0,1), ids in 0..15, threshold 0.9; plus 'nothing reaches it'."""
    import torch
    import managedllama2_b200 as ml2
    rng = np.random.default_rng(31415)
    for _ in range(10):
        x = rng.random(16).astype(np.float16)
        ids = rng.integers(0, 16, 16).astype(np.int32)
        tokens = torch.full((4,), -1, dtype=torch.int32, device="cuda")
        ml2.SampleTopP(ctx).Forward(to_dev(x), dev_i32(ids), 16, 0.9, tokens, 2)
        assert int(tokens[2].item()) == oracle.sample_top_p(x, ids, 0.9)
        assert int(tokens[1].item()) == -1 and int(tokens[3].item()) == -1
    x = np.linspace(0, 0.5, 32000).astype(np.float16)
    ids = np.arange(32000, dtype=np.int32)[::-1].copy()
    tokens = torch.full((1,), -1, dtype=torch.int32, device="cuda")
    ml2.SampleTopP(ctx).Forward(to_dev(x), dev_i32(ids), 32000, 0.75, tokens, 0)
    assert int(tokens[0].item()) == ids[-1]
    ml2.SampleTopP(ctx).Forward(to_dev(x), dev_i32(ids), 32000, 0.25, tokens, 0)
    assert int(tokens[0].item()) == oracle.sample_top_p(x, ids, 0.25)


def run_chain(ctx, logits, temperature, top_p, coin):
    """Sampler.Sample (src/Sampler.cs:49-66) step by step through the Module mirrors; returns every intermediate."""
    import torch
    import managedllama2_b200 as ml2
    n = logits.size
    d = to_dev(logits)
    idx = torch.empty(n, dtype=torch.int32, device="cuda")
    tokens = torch.full((2,), -1, dtype=torch.int32, device="cuda")
    ml2.SoftmaxLogits(ctx).Forward(d, n, temperature, idx)
    threshold = coin
    if 0.0 < top_p < 1.0:
        ml2.Sort(ctx).Forward(d, idx, n)
        threshold = float(np.float32(coin) * np.float32(top_p))
    sorted_p = to_host(d).copy()
    ml2.CumulativeSum(ctx).Forward(d, n)
    ml2.SampleTopP(ctx).Forward(d, idx, n, threshold, tokens, 1)
    return sorted_p, to_host(d), idx.cpu().numpy(), int(tokens[1].item()), threshold


@pytest.mark.parametrize("temperature,top_p", [(0.5, 0.9), (1.0, 0.0), (0.8, 1.0), (1.2, 0.5)])
def test_chain_step_by_step(ctx, temperature, top_p):
    rng = np.random.default_rng(int(temperature * 10))
    agree = 0
    for trial in range(20):
        logits = (rng.standard_normal(32000) * 2.5).astype(np.float16)
        coin = float(rng.random(dtype=np.float32))
        sorted_p, cum, ids, tok, thr = run_chain(ctx, logits, temperature, top_p, coin)
        # the pick is exact given the arrays the device itself produced
        assert tok == oracle.sample_top_p(cum, ids, thr)
        assert half_steps(cum, oracle.cumulative_sum(sorted_p)).max() <= 1
        if 0.0 < top_p < 1.0:
            assert np.all(np.diff(sorted_p.astype(np.float32)) <= 0) and sorted(ids.tolist()) == list(range(32000))
        agree += tok == oracle.sample(logits, temperature, top_p, coin)
    # a coin within one fp16 step of a cumulative value may legitimately pick the neighbour
    assert agree >= 18


def test_model_sample_matches_module_chain(ctx):
    """ml2_model_sample after Forward(pos, next, False) picks the token the Module chain picks on the same logits."""
    import managedllama2_b200 as ml2
    cfg = ml2.Config(dim=512, hiddenDim=1024, numLayers=2, numHeads=4, numKVHeads=4, vocabSize=2000, seqLength=32)
    tr = ml2.Transformer(cfg, ml2.synthetic_weights(ctx, cfg, seed=4), ctx)
    tr.set_tokens(np.array([5, 17], np.int32))
    rng = np.random.default_rng(0)
    for pos in range(8):
        tr.Forward(pos, pos + 1, False)
        if pos >= 1:
            logits = tr.logits()
            coin = float(rng.random(dtype=np.float32))
            tr.Sample(pos + 1, 0.5, 0.9, coin)
            tok = tr.read_token(pos + 1)
            assert tok == run_chain(ctx, logits, 0.5, 0.9, coin)[3]
            assert 0 <= tok < cfg.vocabSize
    out = tr.GenerateSampled([5, 17], 12, temperature=0.5, topP=0.9, seed=1)
    assert out == tr.GenerateSampled([5, 17], 12, temperature=0.5, topP=0.9, seed=1)   # same draws, same tokens
    assert out[0] == 17 and len(out) <= 12
    tr.close()


_REF_CUMSUM = {}


def ref_cumsum_launches(ref):
    """The reference's cumulative_sum_kernel keeps 32 items per thread in registers and is launched with
    vocabulary / 32 = 1000 threads (src/CumulativeSum.cs:12); compiled for sm_100a that block asks for more registers
    than an SM has and the launch is refused (CUDA_ERROR_LAUNCH_OUT_OF_RESOURCES). Where that happens the numpy oracle
    stands in for this one step."""
    if "ok" not in _REF_CUMSUM:
        import torch
        probe = torch.zeros(32000, dtype=torch.float16, device="cuda")
        try:
            ref.cumulative_sum(probe.data_ptr(), 32000)
            torch.cuda.synchronize()
            _REF_CUMSUM["ok"] = True
        except RuntimeError:
            _REF_CUMSUM["ok"] = False
    return _REF_CUMSUM["ok"]


def test_against_reference_kernels(ctx, ref):
    """The reference's four kernels (compiled unmodified) on the same inputs, vocabulary 32000 (the only size their
    launch shapes allow: 125 * 256 and 32 * 1000)."""
    import torch
    import managedllama2_b200 as ml2
    rng = np.random.default_rng(77)
    n = 32000
    for trial in range(4):
        logits = (rng.standard_normal(n) * 3).astype(np.float16)
        a, b = to_dev(logits), to_dev(logits)
        ia = torch.empty(n, dtype=torch.int32, device="cuda")
        ib = torch.empty(n, dtype=torch.int32, device="cuda")
        ml2.SoftmaxLogits(ctx).Forward(a, n, 0.5, ia)
        ref.softmax_logits(b.data_ptr(), n, 0.5, ib.data_ptr())
        torch.cuda.synchronize()
        pa, pb = to_host(a), to_host(b)
        assert half_steps(pa, pb).max() <= 1 and np.array_equal(ia.cpu().numpy(), ib.cpu().numpy())
        # from here on both sides get the reference's probabilities, so that index work can be compared exactly
        a.copy_(b)
        ml2.Sort(ctx).Forward(a, ia, n)
        ref.sort(b.data_ptr(), ib.data_ptr(), n)
        torch.cuda.synchronize()
        assert np.array_equal(to_host(a).view(np.uint16), to_host(b).view(np.uint16))
        assert np.array_equal(ia.cpu().numpy(), ib.cpu().numpy())
        ml2.CumulativeSum(ctx).Forward(a, n)
        if ref_cumsum_launches(ref):
            ref.cumulative_sum(b.data_ptr(), n)
        else:
            b.copy_(to_dev(oracle.cumulative_sum(to_host(b))))
        torch.cuda.synchronize()
        assert half_steps(to_host(a), to_host(b)).max() <= 1
        a.copy_(b)
        ta = torch.full((1,), -1, dtype=torch.int32, device="cuda")
        tb = torch.full((1,), -1, dtype=torch.int32, device="cuda")
        thr = float(rng.random(dtype=np.float32)) * 0.9
        ml2.SampleTopP(ctx).Forward(a, ia, n, thr, ta, 0)
        ref.sample_top_p(b.data_ptr(), ib.data_ptr(), n, thr, tb.data_ptr(), 0)
        torch.cuda.synchronize()
        assert int(ta.item()) == int(tb.item())
    # integers: exact (the reference's own cumulative-sum test)
    if ref_cumsum_launches(ref):
        x = rng.integers(-1000, 1001, n).astype(np.float16)
        a, b = to_dev(x), to_dev(x)
        ml2.CumulativeSum(ctx).Forward(a, n)
        ref.cumulative_sum(b.data_ptr(), n)
        torch.cuda.synchronize()
        assert np.array_equal(to_host(a).view(np.uint16), to_host(b).view(np.uint16))


def test_argument_checks(ctx):
    import torch
    import managedllama2_b200 as ml2
    t = torch.zeros(64, dtype=torch.float16, device="cuda")
    i = torch.zeros(64, dtype=torch.int32, device="cuda")
    with pytest.raises(ml2.Ml2Error):
        ml2.SoftmaxLogits(ctx).Forward(t, 64, 0.0, i)
    with pytest.raises(ml2.Ml2Error):
        ml2.Sort(ctx).Forward(t, i, 0)
    with pytest.raises(ml2.Ml2Error):
        ml2.Sort(ctx).Forward(t, i, 40000)
    with pytest.raises(ml2.Ml2Error):
        ml2.CumulativeSum(ctx).Forward(t, -1)
