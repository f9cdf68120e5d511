"""model.bin -> device -> decode: a model loaded from a file in the reference's layout gives the same logits, bit for
bit, as the same tensors bound directly, and every tensor-parallel shard cut from the file equals the shard generated
in place."""
import ctypes

import numpy as np
import pytest

import oracle
from helpers import write_model_bin

pytestmark = pytest.mark.gpu


def d2h(ptr, nbytes):
    import torch
    out = np.empty(nbytes, np.uint8)
    rt = ctypes.CDLL("libcudart.so.12")
    rt.cudaMemcpy.argtypes = [ctypes.c_void_p, ctypes.c_void_p, ctypes.c_size_t, ctypes.c_int]
    assert rt.cudaMemcpy(out.ctypes.data, ctypes.c_void_p(ptr), nbytes, 2) == 0
    return out


@pytest.fixture(scope="module")
def setup(tmp_path_factory):
    import managedllama2_b200 as ml2
    cfg = ml2.Config(dim=512, hiddenDim=13 * 128, numLayers=2, numHeads=4, numKVHeads=4, vocabSize=256, seqLength=48)
    hw = ml2.synthetic_weights_host(cfg, seed=9)
    path = tmp_path_factory.mktemp("mfg") / "model.bin"
    write_model_bin(path, cfg, hw)
    ctx = ml2.CudaContext(0)
    yield ml2, cfg, hw, path, ctx
    assert ctx.status() == (0, 0)


def test_decode_from_file_is_bit_identical_to_bound_tensors(setup):
    ml2, cfg, hw, path, ctx = setup
    a = ml2.Transformer.FromFile(path, ctx)
    b = ml2.Transformer(cfg, ml2.synthetic_weights(ctx, cfg, seed=9), ctx)
    assert a.config == cfg
    cpu = oracle.CpuModel(dict(dim=cfg.dim, hidden_dim=cfg.hiddenDim, n_layers=cfg.numLayers, n_heads=cfg.numHeads,
                               n_kv_heads=cfg.numKVHeads, vocab_size=cfg.vocabSize, seq_len=cfg.seqLength,
                               rope_theta=cfg.ropeTheta), hw, mode=1)
    toks = [3, 77, 200]
    for t in (a, b):
        t.set_tokens(np.array(toks, np.int32))
    seq = list(toks)
    for pos in range(10):
        gen = pos + 1 >= len(toks)
        a.Forward(pos, pos + 1, gen)
        b.Forward(pos, pos + 1, gen)
        la, lb = a.logits(), b.logits()
        assert np.array_equal(la.view(np.uint16), lb.view(np.uint16))
        if gen:
            assert a.read_token(pos + 1) == b.read_token(pos + 1)
            seq.append(a.read_token(pos + 1))
        want = cpu.forward(seq[pos], pos).astype(np.float32)
        assert float(np.abs(la.astype(np.float32) - want).max()) <= 1e-2
    a.close()
    b.close()


@pytest.mark.parametrize("tp", [1, 2, 4])
def test_shards_from_file_equal_generated_shards(setup, tp):
    ml2, cfg, hw, path, ctx = setup
    from managedllama2_b200.transformer import GROUP, tp_shapes
    with ml2.ModelFile(path) as mf:
        for rank in range(tp):
            dw = ml2.DeviceWeights(ctx, mf, tp, rank)
            ref = ml2.synthetic_weights(ctx, cfg, seed=9, tp_size=tp, tp_rank=rank)
            dim_local, hg0, hng, vrow0, vlocal = tp_shapes(cfg, tp, rank)
            e, c, r = dw.globals()
            assert np.array_equal(d2h(e, cfg.vocabSize * cfg.dim * 2), ref.tokenEmbeddingTable.cpu().numpy().view(np.uint8))
            assert np.array_equal(d2h(c, vlocal * cfg.dim * 2), ref.classifierWeights.cpu().numpy().view(np.uint8))
            assert np.array_equal(d2h(r, cfg.dim * 2), ref.rmsFinalWeight.cpu().numpy().view(np.uint8))
            for l in range(cfg.numLayers):
                s, L = dw.layer(l), ref.layers[l]
                pairs = [("query", L.queryWeight, cfg.dim // GROUP), ("key", L.keyWeight, cfg.dim // GROUP),
                         ("value", L.valueWeight, cfg.dim // GROUP), ("output", L.outputWeight, dim_local // GROUP),
                         ("gate", L.gateWeight, cfg.dim // GROUP), ("up", L.upWeight, cfg.dim // GROUP), ("down", L.downWeight, hng)]
                for name, qw, ngroups in pairs:
                    q = getattr(s, name)
                    w = qw.Weight.cpu().numpy().view(np.uint8)
                    assert np.array_equal(d2h(q.weight, w.size), w), (tp, rank, l, name)
                    sc = qw.Scales.cpu().numpy().view(np.uint8)
                    assert np.array_equal(d2h(q.scales, sc.size), sc), (tp, rank, l, name)
                    # zero points: compare the nibbles that exist (padding nibbles of a column's last word are never read)
                    z = qw.Zeros.cpu().numpy().view(np.uint32)
                    got = d2h(q.zeros, z.size * 4).view(np.uint32)
                    zs = (ngroups + 7) // 8
                    mask = np.zeros(zs, np.uint32)
                    for g in range(ngroups):
                        mask[g // 8] |= np.uint32(0xF << (4 * (g % 8)))
                    m = np.tile(mask, z.size // zs)
                    assert np.array_equal(got & m, z & m), (tp, rank, l, name)
                assert np.array_equal(d2h(s.rms_attention, cfg.dim * 2), L.rmsAttentionWeight.cpu().numpy().view(np.uint8))
                assert np.array_equal(d2h(s.rms_feed_forward, cfg.dim * 2), L.rmsFeedForwardWeight.cpu().numpy().view(np.uint8))
            dw.close()


def test_upload_refuses_shapes_that_do_not_split(setup):
    ml2, cfg, hw, path, ctx = setup
    with ml2.ModelFile(path) as mf:
        with pytest.raises(ml2.Ml2Error):
            ml2.DeviceWeights(ctx, mf, 3, 0)      # 4 heads over 3 ranks
        with pytest.raises(ml2.Ml2Error):
            ml2.DeviceWeights(ctx, mf, 2, 2)      # rank out of range
