"""The small operators through the C ABI against the CPU oracle, case by case like the reference's own tests:
test/RMSNormTests.cs, RoPETests.cs, SoftmaxTests.cs, ArgmaxTests.cs, EmbeddingTableTests.cs, MatVecStridedTests.cs,
VecMatTests.cs (inputs of the same shapes and ranges; the reference draws them from System.Random(31415), which cannot
be regenerated without .NET). Tolerance: one fp16 rounding of difference at most (relative 1e-3), bit equality where
the arithmetic is exact.
"""
import numpy as np
import pytest

import oracle
from helpers import rel_err, to_dev, to_host

pytestmark = pytest.mark.gpu


@pytest.fixture(scope="module")
def ctx():
    import managedllama2_b200 as ml2
    c = ml2.CudaContext(0)
    yield c
    assert c.status() == (0, 0)
    c.close()


def uniform01(rng, n):
    return rng.random(n).astype(np.float16)  # Generator.NextArray: (Half)random.NextDouble()


@pytest.mark.parametrize("vec,gamma", [([1., 2., 3.], [4., 5., 6.]), ([6., 2., 6.], [1., 9., 7.])])
def test_rmsnorm_reference_cases(ctx, vec, gamma):
    """test/RMSNormTests.cs:63-75: the two inline 3-element cases."""
    import torch
    import managedllama2_b200 as ml2
    x, g = np.array(vec, np.float16), np.array(gamma, np.float16)
    out = torch.zeros(3, dtype=torch.float16, device="cuda")
    ml2.RMSNorm(ctx).Forward(out, to_dev(x), to_dev(g), 3)
    got = to_host(out)
    assert rel_err(got, oracle.rmsnorm(x, g)) <= 1e-3                      # kernel arithmetic (fp32 squares)
    assert rel_err(got, oracle.rmsnorm(x, g, fp16_square=True)) <= 1e-3    # the C# test's variant


@pytest.mark.parametrize("size", [1, 7, 4096, 5120, 11008])
def test_rmsnorm_sizes_and_in_place(ctx, size):
    import managedllama2_b200 as ml2
    rng = np.random.default_rng(size)
    x, g = rng.standard_normal(size).astype(np.float16), (rng.standard_normal(size) * 0.02).astype(np.float16)
    d = to_dev(x)
    ml2.RMSNorm(ctx).Forward(d, d, to_dev(g), size)   # in place, as the final norm is (src/Transformer.cs:187)
    assert rel_err(to_host(d), oracle.rmsnorm(x, g)) <= 1e-3


def test_rope_reference_case(ctx):
    """test/RoPETests.cs:94-118: dim 128, 32 heads (head size 4), 20 cache rows, pos 0..18."""
    import managedllama2_b200 as ml2
    rng = np.random.default_rng(31415)
    dim, heads, seq = 128, 32, 20
    cfg = ml2.Config(dim, 4 * dim, 1, heads, heads, 32, seq)
    q0, k0 = uniform01(rng, dim), uniform01(rng, dim * seq)
    for pos in range(seq - 1):
        q, k = to_dev(q0), to_dev(k0)
        ml2.RoPERotation(ctx, cfg).Forward(q, k, heads, dim // heads, pos, 0, 10000.0)
        wq, wk_row = oracle.rope(q0, k0[pos * dim:(pos + 1) * dim], dim, heads, heads, pos)
        want_k = k0.copy()
        want_k[pos * dim:(pos + 1) * dim] = wk_row
        assert rel_err(to_host(q), wq) <= 1e-3
        assert rel_err(to_host(k), want_k) <= 1e-3
        untouched = np.ones(dim * seq, bool)
        untouched[pos * dim:(pos + 1) * dim] = False
        assert np.array_equal(to_host(k)[untouched].view(np.uint16), k0[untouched].view(np.uint16))


@pytest.mark.parametrize("pos", [0, 1, 18, 2047, 4095])
def test_rope_head128_positions(ctx, pos):
    import managedllama2_b200 as ml2
    rng = np.random.default_rng(pos)
    dim, heads = 512, 4
    cfg = ml2.Config(dim, 4 * dim, 1, heads, heads, 32, 8)
    q0, k0 = rng.standard_normal(dim).astype(np.float16), rng.standard_normal(dim).astype(np.float16)
    q, k = to_dev(q0), to_dev(k0)
    # the key pointer is offset by pos * kvDim inside Forward (src/RoPERotation.cs:22): call the ABI on the row itself
    import ctypes
    from managedllama2_b200 import _lib
    _lib.check(ctx._lib.ml2_rope(ctx.handle, ctypes.c_void_p(q.data_ptr()), ctypes.c_void_p(k.data_ptr()), heads, heads, 128, pos,
                                ctypes.c_float(10000.0)))
    wq, wk = oracle.rope(q0, k0, dim, heads, heads, pos)
    # sinf/cosf of large angles differ between libm and the device by a few ulp of fp32: one fp16 step at most
    assert rel_err(to_host(q), wq) <= 2e-3 and rel_err(to_host(k), wk) <= 2e-3


def test_softmax_reference_cases(ctx):
    """test/SoftmaxTests.cs:61-78: ten vectors of 16 values in [0,1), one head each."""
    import managedllama2_b200 as ml2
    rng = np.random.default_rng(31415)
    cfg = ml2.Config(128, 512, 1, 1, 1, 32, 16)
    for _ in range(10):
        x = uniform01(rng, 16)
        d = to_dev(x)
        ml2.Softmax(ctx, cfg).Forward(d, 16)
        got = to_host(d)
        assert rel_err(got, oracle.softmax(x, 1, 16)) <= 1e-3
        assert abs(float(got.astype(np.float32).sum()) - 1.0) < 5e-3


@pytest.mark.parametrize("heads,size", [(32, 1), (32, 33), (40, 1000), (40, 4096), (2, 9000)])
def test_softmax_sizes(ctx, heads, size):
    """Up to and beyond the reference's 8192-float shared-memory cap (native/softmax_kernel.cu:5)."""
    import managedllama2_b200 as ml2
    rng = np.random.default_rng(size)
    cfg = ml2.Config(128 * heads, 512, 1, heads, heads, 32, size)
    x = (rng.standard_normal(heads * size) * 2).astype(np.float16)
    d = to_dev(x)
    ml2.Softmax(ctx, cfg).Forward(d, size)
    want = oracle.softmax(x, heads, size).astype(np.float64)
    got = to_host(d).astype(np.float64)
    assert np.max(np.abs(got - want)) <= 1e-3 * max(want.max(), 1e-4) + 1e-7


def test_argmax_reference_case_and_ties(ctx):
    """test/ArgmaxTests.cs:48-64 (10 values) plus ties, which must resolve to the first maximum (:33-46)."""
    import torch
    import managedllama2_b200 as ml2
    rng = np.random.default_rng(31415)
    for n in (10, 1000, 32000):
        x = uniform01(rng, n)
        tokens = torch.full((8,), -1, dtype=torch.int32, device="cuda")
        ml2.Argmax(ctx).Forward(to_dev(x), n, tokens, 3, True)
        assert int(tokens[3].item()) == oracle.argmax(x)
        assert int(tokens[2].item()) == -1 and int(tokens[4].item()) == -1
    x = np.zeros(32000, np.float16)
    x[[17, 4000, 31999]] = 2.5
    tokens = torch.full((4,), -1, dtype=torch.int32, device="cuda")
    ml2.Argmax(ctx).Forward(to_dev(x), 32000, tokens, 0, True)
    assert int(tokens[0].item()) == 17
    ml2.Argmax(ctx).Forward(to_dev(x), 32000, tokens, 1, False)   # generateToken = false: nothing written
    assert int(tokens[1].item()) == -1


def test_embedding_reference_case(ctx):
    """test/EmbeddingTableTests.cs:40-50: 256-wide rows gathered by token id."""
    import torch
    import managedllama2_b200 as ml2
    rng = np.random.default_rng(31415)
    size, vocab = 256, 50
    table = uniform01(rng, size * vocab)
    toks = np.array([7, 0, 49, 13], np.int32)
    out = torch.zeros(size, dtype=torch.float16, device="cuda")
    for pos, t in enumerate(toks):
        ml2.Embedding(ctx).Forward(out, to_dev(table), size, to_dev(toks), pos)
        assert np.array_equal(to_host(out).view(np.uint16), table[t * size:(t + 1) * size].view(np.uint16))


@pytest.mark.parametrize("seq", [1, 16, 31, 32, 33, 272, 4096])
def test_scores_and_values_reference_shapes(ctx, seq):
    """test/MatVecStridedTests.cs:74-92 and test/VecMatTests.cs:75-93: dim 4096, 32 heads, seq 16 (and other lengths)."""
    import torch
    import managedllama2_b200 as ml2
    rng = np.random.default_rng(seq)
    dim, heads = 4096, 32
    cfg = ml2.Config(dim, 11008, 1, heads, heads, 32, max(seq, 16))
    q, kc = uniform01(rng, dim), uniform01(rng, dim * seq)
    att = torch.zeros(heads * seq, dtype=torch.float16, device="cuda")
    ml2.MatVecStrided(ctx, cfg).Forward(att, to_dev(q), to_dev(kc), 128, dim, seq, 0, 1.0 / np.sqrt(128.0))
    want = oracle.attn_scores(q, kc, dim, heads, heads, seq)
    assert rel_err(to_host(att), want) <= 1e-3
    a = uniform01(rng, heads * seq)
    vc = uniform01(rng, dim * seq)
    out = torch.zeros(dim, dtype=torch.float16, device="cuda")
    ml2.VecMat(ctx, cfg).Forward(out, to_dev(vc), to_dev(a), 128, dim, seq, 0)
    assert rel_err(to_host(out), oracle.attn_values(a, vc, dim, heads, heads, seq)) <= 1e-3


def test_small_ops_argument_checks(ctx):
    import torch
    import managedllama2_b200 as ml2
    t = torch.zeros(64, dtype=torch.float16, device="cuda")
    cfg = ml2.Config(128, 512, 1, 1, 1, 32, 16)
    with pytest.raises(ml2.Ml2Error):
        ml2.RMSNorm(ctx).Forward(t, t, t, 0)
    with pytest.raises(ml2.Ml2Error):
        ml2.Softmax(ctx, cfg).Forward(t, 0)
    with pytest.raises(ml2.Ml2Error):
        ml2.RoPERotation(ctx, cfg).Forward(t, t, 2, 128, 0, 0, 10000.0)   # more kv heads than heads
