"""The numpy restatement of the sampling chain (oracle.softmax_logits / sort_desc / cumulative_sum / sample_top_p)
against the expectations written in the reference's own tests (test/SoftmaxLogitsTests.cs:34-72,
test/CumulativeSumTests.cs:44-56, test/SampleTopPTests.cs:34-46), restated here as plain loops on small inputs."""
import numpy as np

import oracle


def test_softmax_logits_matches_plain_loops():
    rng = np.random.default_rng(1)
    x = rng.random(16).astype(np.float16)
    for temperature in (1.0, 0.5):
        probs, idx = oracle.softmax_logits(x, temperature)
        scaled = [np.float16(np.float32(v) / np.float32(temperature)) for v in x]
        mx = max(np.float32(v) for v in scaled)
        e = [np.exp(np.float32(v) - mx, dtype=np.float32) for v in scaled]
        tot = np.float32(0)
        for v in e:
            tot = np.float32(tot + v)
        want = np.array([np.float16(np.float32(np.float16(v)) / tot) for v in e], np.float16)
        assert np.max(np.abs(probs.view(np.uint16).astype(int) - want.view(np.uint16).astype(int))) <= 1
        assert idx.tolist() == list(range(16))


def test_cumulative_sum_and_pick():
    rng = np.random.default_rng(2)
    x = rng.integers(-1000, 1001, 500).astype(np.float16)
    cdf, want = np.float32(0), []
    for v in x:
        cdf = np.float32(cdf + np.float32(v))
        want.append(np.float16(cdf))
    assert np.array_equal(oracle.cumulative_sum(x).view(np.uint16), np.array(want, np.float16).view(np.uint16))
    vals = rng.random(16).astype(np.float16)
    ids = rng.integers(0, 16, 16)
    first = next((i for i, v in enumerate(vals) if float(v) >= 0.9), 15)
    assert oracle.sample_top_p(vals, ids, 0.9) == ids[first]
    assert oracle.sample_top_p(np.zeros(8, np.float16), np.arange(8), 0.5) == 7


def test_sort_is_stable_and_sample_respects_top_p():
    keys = np.array([1, 3, 3, 0, 3, 1], np.float16)
    k, v = oracle.sort_desc(keys, np.arange(6))
    assert k.tolist() == [3, 3, 3, 1, 1, 0] and v.tolist() == [1, 2, 4, 0, 5, 3]
    logits = np.array([0.0, 5.0, 1.0, 4.0], np.float16)
    # with top_p = 0.5 only the most likely token can be drawn, whatever the coin
    assert {oracle.sample(logits, 1.0, 0.5, c) for c in np.linspace(0, 0.999, 50)} == {1}
    # without top-p the coin walks the unsorted cumulative distribution
    assert oracle.sample(logits, 1.0, 0.0, 0.0) == 0 and oracle.sample(logits, 1.0, 0.0, 0.999) == 3
