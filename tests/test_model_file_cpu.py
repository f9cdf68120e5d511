"""model.bin reader, host side (no GPU): header, tensor walk, and the reference's two refusals
(src/Config.cs:27-28 ropeTheta, src/TransformerWeights.cs:39-40 exact consumption)."""
import struct

import numpy as np
import pytest

import managedllama2_b200 as ml2
from managedllama2_b200 import transformer as T
from helpers import write_model_bin

CFG = ml2.Config(dim=256, hiddenDim=640, numLayers=2, numHeads=2, numKVHeads=2, vocabSize=96, seqLength=32)


@pytest.fixture(scope="module")
def model(tmp_path_factory):
    hw = ml2.synthetic_weights_host(CFG, seed=5)
    path = tmp_path_factory.mktemp("mf") / "model.bin"
    write_model_bin(path, CFG, hw)
    return path, hw


def test_header_and_every_tensor(model):
    path, hw = model
    with ml2.ModelFile(path) as mf:
        assert mf.config == CFG
        assert np.array_equal(mf.tensor(-1, T.T_EMBED).view(np.uint16), hw["embed"].view(np.uint16))
        assert np.array_equal(mf.tensor(-1, T.T_CLASSIFIER).view(np.uint16), hw["classifier"].view(np.uint16))
        assert np.array_equal(mf.tensor(-1, T.T_RMS_FINAL).view(np.uint16), hw["rms_final"].view(np.uint16))
        names = {T.T_QUERY: "q", T.T_KEY: "k", T.T_VALUE: "v", T.T_OUTPUT: "o", T.T_UP: "up", T.T_GATE: "gate", T.T_DOWN: "down"}
        for l, L in enumerate(hw["layers"]):
            for tid, name in names.items():
                w, z, s = L[name]
                assert np.array_equal(mf.tensor(l, tid, 0), w), (l, name)
                assert np.array_equal(mf.tensor(l, tid, 1), z), (l, name)
                assert np.array_equal(mf.tensor(l, tid, 2).view(np.uint16), s.view(np.uint16)), (l, name)
            assert np.array_equal(mf.tensor(l, T.T_RMS_ATT).view(np.uint16), L["rms_att"].view(np.uint16))
            assert np.array_equal(mf.tensor(l, T.T_RMS_FFN).view(np.uint16), L["rms_ffn"].view(np.uint16))


def test_qweight_sizes_follow_the_reference(model):
    """ReadQWeight (src/TransformerWeights.cs:54-69): weightsSize = ceil(rows/32)*4, scalesSize = ceil(rows/128),
    zerosSize = ceil(scalesSize/8), all times cols; down has rows = hiddenDim."""
    path, _ = model
    with ml2.ModelFile(path) as mf:
        assert mf.tensor(0, T.T_QUERY, 0).size == 8 * 4 * 256 and mf.tensor(0, T.T_QUERY, 1).size == 256
        assert mf.tensor(0, T.T_QUERY, 2).size == 2 * 256
        assert mf.tensor(0, T.T_UP, 0).size == 8 * 4 * 640 and mf.tensor(0, T.T_GATE, 2).size == 2 * 640
        assert mf.tensor(0, T.T_DOWN, 0).size == 20 * 4 * 256 and mf.tensor(0, T.T_DOWN, 1).size == 256
        assert mf.tensor(0, T.T_DOWN, 2).size == 5 * 256


def test_truncated_and_padded_files_are_refused(model, tmp_path):
    path, _ = model
    blob = path.read_bytes()
    short, long_ = tmp_path / "short.bin", tmp_path / "long.bin"
    short.write_bytes(blob[:-2])
    long_.write_bytes(blob + b"\0\0")
    for p in (short, long_):
        with pytest.raises(ml2.Ml2Error, match="Failed to read file"):
            ml2.ModelFile(p)
    tiny = tmp_path / "tiny.bin"
    tiny.write_bytes(blob[:16])
    with pytest.raises(ml2.Ml2Error, match="header"):
        ml2.ModelFile(tiny)
    with pytest.raises(ml2.Ml2Error):
        ml2.ModelFile(tmp_path / "missing.bin")


def test_wrong_rope_theta_is_refused(model, tmp_path):
    path, _ = model
    blob = bytearray(path.read_bytes())
    blob[28:32] = struct.pack("<f", 500000.0)
    bad = tmp_path / "theta.bin"
    bad.write_bytes(bytes(blob))
    with pytest.raises(ml2.Ml2Error, match="Invalid model config"):
        ml2.ModelFile(bad)


def test_bad_tensor_requests(model):
    path, _ = model
    with ml2.ModelFile(path) as mf:
        for args in ((-1, 3, 0), (0, 9, 0), (2, 0, 0), (0, T.T_QUERY, 3), (0, T.T_RMS_ATT, 1)):
            with pytest.raises(ml2.Ml2Error):
                mf.tensor(*args)


@pytest.mark.parametrize("tp", [1, 2])
def test_shards_cut_on_the_host_equal_generated_shards(model, tp):
    """ml2_model_file_shard (no GPU): every rank's part of every QWeight equals the shard the synthetic generator makes
    in place for the same rank - column ranges for query / key / value / up / gate, windows of groups with re-packed
    zero points for output / down (5 hidden groups over 2 ranks: 3 + 2, an uneven split)."""
    import ctypes
    from managedllama2_b200 import _lib
    from managedllama2_b200.transformer import GROUP, layer_tid, tp_shapes, _qw_window
    path, _ = model
    lib = _lib.load()
    dim, hid = CFG.dim, CFG.hiddenDim
    with ml2.ModelFile(path) as mf:
        for rank in range(tp):
            dim_local, hg0, hng, _, _ = tp_shapes(CFG, tp, rank)
            hidden_local = hng * GROUP
            gd = dim // GROUP
            # (tensor id in the file, generator name, rows_full, col0, ncols, g0, ngroups)
            plan = [(T.T_QUERY, "query", dim, rank * dim_local, dim_local, 0, gd), (T.T_KEY, "key", dim, rank * dim_local, dim_local, 0, gd),
                    (T.T_VALUE, "value", dim, rank * dim_local, dim_local, 0, gd),
                    (T.T_OUTPUT, "output", dim, 0, dim, rank * (dim_local // GROUP), dim_local // GROUP),
                    (T.T_UP, "up", dim, hg0 * GROUP, hidden_local, 0, gd), (T.T_GATE, "gate", dim, hg0 * GROUP, hidden_local, 0, gd),
                    (T.T_DOWN, "down", hid, 0, dim, hg0, hng)]
            for l in range(CFG.numLayers):
                for tid, name, rows_full, col0, ncols, g0, ng in plan:
                    _, nw, nz, ns = _qw_window(rows_full, ncols, g0, ng)
                    w, z, s = np.empty(nw, np.uint32), np.empty(nz, np.uint32), np.empty(ns, np.float16)
                    _lib.check(lib.ml2_synth_qweight_host(w.ctypes.data_as(ctypes.c_void_p), z.ctypes.data_as(ctypes.c_void_p),
                                                          s.ctypes.data_as(ctypes.c_void_p), rows_full, col0, ncols, g0, ng,
                                                          ctypes.c_uint64(5), ctypes.c_uint32(layer_tid(l, name))))
                    bw, bz, bs = ctypes.c_uint64(), ctypes.c_uint64(), ctypes.c_uint64()
                    _lib.check(lib.ml2_model_file_shard(mf.handle, l, tid, tp, rank, None, None, None, ctypes.byref(bw), ctypes.byref(bz),
                                                        ctypes.byref(bs)))
                    assert (bw.value, bz.value, bs.value) == (nw * 4, nz * 4, ns * 2), (rank, l, name)
                    gw, gz, gs = np.empty(nw, np.uint32), np.empty(nz, np.uint32), np.empty(ns, np.float16)
                    _lib.check(lib.ml2_model_file_shard(mf.handle, l, tid, tp, rank, gw.ctypes.data_as(ctypes.c_void_p),
                                                        gz.ctypes.data_as(ctypes.c_void_p), gs.ctypes.data_as(ctypes.c_void_p), None, None, None))
                    assert np.array_equal(gw, w), (rank, l, name)
                    assert np.array_equal(gs.view(np.uint16), s.view(np.uint16)), (rank, l, name)
                    zs = (ng + 7) // 8
                    mask = np.zeros(zs, np.uint32)
                    for g in range(ng):
                        mask[g // 8] |= np.uint32(0xF << (4 * (g % 8)))
                    m = np.tile(mask, nz // zs)
                    assert np.array_equal(gz & m, z & m), (rank, l, name)
        with pytest.raises(ml2.Ml2Error):
            lib_rc = lib.ml2_model_file_shard(mf.handle, 0, T.T_QUERY, 3, 0, None, None, None, None, None, None)
            _lib.check(lib_rc)
