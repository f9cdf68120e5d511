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
