"""AWQ -> QWeight repacking on the device (bit-exact against the oracle) and the converter end to end: a synthetic
AutoAWQ-style checkpoint -> model.bin -> reader -> decode, logits against the CPU oracle on the re-packed weights."""
import ctypes
import json

import numpy as np
import pytest

import oracle

pytestmark = pytest.mark.gpu


@pytest.fixture(scope="module")
def ctx():
    import managedllama2_b200 as ml2
    c = ml2.CudaContext(0)
    yield c
    assert c.status() == (0, 0)
    c.close()


@pytest.mark.parametrize("height,width", [(8, 8), (4, 8), (1, 8), (2, 16), (3, 24), (12, 16), (108, 5120), (86, 4096), (40, 5120), (5120, 1024), (4096, 264)])
def test_repack_qdata_bit_exact(ctx, height, width):
    import torch
    from managedllama2_b200.convert import ModelConverter
    rng = np.random.default_rng(height + width)
    q = rng.integers(0, 2 ** 32, size=height * (width // 8), dtype=np.uint64).astype(np.uint32)
    conv = ModelConverter([], None, ctx)
    got = conv.repack_qdata(torch.from_numpy(q.view(np.int32)), height, width)
    assert np.array_equal(got, oracle.awq_repack_qdata(q, height, width))
    if height * width <= 4096:
        assert np.array_equal(got, oracle.awq_repack_qdata_loops(q, height, width))


@pytest.mark.parametrize("meta_height,width", [(1, 8), (5, 40), (40, 5120), (108, 5120), (33, 1000)])
def test_repack_scales_bit_exact(ctx, meta_height, width):
    import torch
    from managedllama2_b200.convert import ModelConverter
    rng = np.random.default_rng(meta_height)
    s = rng.standard_normal(meta_height * width).astype(np.float16)
    conv = ModelConverter([], None, ctx)
    got = conv.repack_scales(torch.from_numpy(s), meta_height, width)
    assert np.array_equal(got.view(np.uint16), oracle.awq_repack_scales(s, meta_height, width).view(np.uint16))
    padded = ((meta_height + 7) // 8) * 8
    v1 = rng.standard_normal(width * padded).astype(np.float16)
    got = conv.compact_scales_v1(torch.from_numpy(v1), meta_height, padded, width)
    assert np.array_equal(got.view(np.uint16), v1.reshape(width, padded)[:, :meta_height].reshape(-1).view(np.uint16))


def make_checkpoint(tmp, cfg, seed, fmt):
    """A synthetic AutoAWQ-style state dict (format v0) or the v1 layout, plus the QWeights it must convert to."""
    import torch
    rng = np.random.default_rng(seed)
    dim, hid = cfg.dim, cfg.hiddenDim
    state, want = {}, {"layers": []}

    def f16(*shape, sigma=0.05):
        return (rng.standard_normal(shape) * sigma).astype(np.float16)

    for name, key, shape in (("model.embed_tokens.weight", "embed", (cfg.vocabSize, dim)), ("lm_head.weight", "classifier", (cfg.vocabSize, dim)),
                             ("model.norm.weight", "rms_final", (dim,))):
        a = f16(*shape) if key != "rms_final" else (1 + f16(*shape)).astype(np.float16)
        state[name] = torch.from_numpy(a)
        want[key] = a.reshape(-1)
    projs = (("self_attn.q_proj", "q", dim, dim), ("self_attn.k_proj", "k", dim, dim), ("self_attn.v_proj", "v", dim, dim),
             ("self_attn.o_proj", "o", dim, dim), ("mlp.up_proj", "up", dim, hid), ("mlp.gate_proj", "gate", dim, hid),
             ("mlp.down_proj", "down", hid, dim))
    for l in range(cfg.numLayers):
        L = {}
        for pname, key, height, width in projs:
            groups = height // 128
            vals = rng.integers(0, 16, size=(height, width))
            zeros = rng.integers(0, 16, size=(groups, width))
            scales = rng.uniform(0.001, 0.02, size=(groups, width)).astype(np.float16)
            qw, qz = oracle.awq_pack_v0(vals, height, width), oracle.awq_pack_v0(zeros, groups, width)
            tw = oracle.awq_repack_qdata(qw, height, width)
            tz = oracle.awq_repack_qdata(qz, groups, width)
            ts = oracle.awq_repack_scales(scales, groups, width)
            L[key] = (tw, tz, ts)
            p = "model.layers.%d.%s" % (l, pname)
            if fmt == "v0":
                state[p + ".qweight"] = torch.from_numpy(qw.view(np.int32).reshape(height, width // 8))
                state[p + ".qzeros"] = torch.from_numpy(qz.view(np.int32).reshape(groups, width // 8))
                state[p + ".scales"] = torch.from_numpy(scales)
            else:
                padded = ((groups + 7) // 8) * 8
                sp = np.zeros((width, padded), np.float16)
                sp[:, :groups] = ts.reshape(width, groups)
                state[p + ".qweight"] = torch.from_numpy(tw.view(np.int32))
                state[p + ".qzeros"] = torch.from_numpy(tz.view(np.int32))
                state[p + ".scales"] = torch.from_numpy(sp)
        for pname, key in (("input_layernorm.weight", "rms_att"), ("post_attention_layernorm.weight", "rms_ffn")):
            a = (1 + f16(dim)).astype(np.float16)
            state["model.layers.%d.%s" % (l, pname)] = torch.from_numpy(a)
            L[key] = a
        want["layers"].append(L)
    # two checkpoint files, as the 13B download comes in parts (src/ModelConverter.cs:64-70)
    keys = sorted(state)
    half = len(keys) // 2
    paths = [tmp / "pytorch_model.001.pt", tmp / "pytorch_model.002.pt"]
    torch.save({k: state[k] for k in keys[:half]}, paths[0])
    torch.save({k: state[k] for k in keys[half:]}, paths[1])
    cj = tmp / "config.json"
    cj.write_text(json.dumps({"hidden_size": dim, "intermediate_size": hid, "max_position_embeddings": cfg.seqLength,
                              "num_attention_heads": cfg.numHeads, "num_hidden_layers": cfg.numLayers,
                              "num_key_value_heads": cfg.numKVHeads, "vocab_size": cfg.vocabSize}))
    return paths, cj, want


@pytest.mark.parametrize("fmt", ["v0", "v1"])
def test_converter_end_to_end(ctx, tmp_path, fmt):
    import managedllama2_b200 as ml2
    from managedllama2_b200 import transformer as T
    from managedllama2_b200.convert import ModelConverter
    cfg = ml2.Config(dim=256, hiddenDim=640, numLayers=2, numHeads=2, numKVHeads=2, vocabSize=96, seqLength=32)
    paths, cj, want = make_checkpoint(tmp_path, cfg, 11, fmt)
    out = tmp_path / "model.bin"
    got_cfg = ModelConverter(paths, cj, ctx).Convert(out, fmt)
    assert got_cfg == cfg        # rope_theta absent from config.json -> 10000 (src/ModelConverter.cs:107)
    names = {T.T_QUERY: "q", T.T_KEY: "k", T.T_VALUE: "v", T.T_OUTPUT: "o", T.T_UP: "up", T.T_GATE: "gate", T.T_DOWN: "down"}
    with ml2.ModelFile(out) as mf:
        assert mf.config == cfg
        assert np.array_equal(mf.tensor(-1, T.T_EMBED).view(np.uint16), want["embed"].view(np.uint16))
        for l, L in enumerate(want["layers"]):
            for tid, name in names.items():
                for part in range(3):
                    a, b = mf.tensor(l, tid, part), L[name][part]
                    assert np.array_equal(a.view(np.uint16), np.ascontiguousarray(b).view(np.uint16)), (l, name, part)
    tr = ml2.Transformer.FromFile(out, ctx)
    cpu = oracle.CpuModel(dict(dim=cfg.dim, hidden_dim=cfg.hiddenDim, n_layers=cfg.numLayers, n_heads=cfg.numHeads,
                               n_kv_heads=cfg.numKVHeads, vocab_size=cfg.vocabSize, seq_len=cfg.seqLength,
                               rope_theta=cfg.ropeTheta), want, mode=1)
    toks = [5, 40, 77]
    tr.set_tokens(np.array(toks, np.int32))
    for pos in range(6):
        gen = pos + 1 >= len(toks)
        tr.Forward(pos, pos + 1, gen)
        if gen:
            toks.append(tr.read_token(pos + 1))
        w = cpu.forward(toks[pos], pos).astype(np.float32)
        assert np.abs(tr.logits().astype(np.float32) - w).max() <= 2e-2 * max(w.std(), 1e-3)
    tr.close()
