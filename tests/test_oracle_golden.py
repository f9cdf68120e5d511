"""Pins the CPU oracle against the reference's own known answers for the QWeight layout.

Mirrors test/QWeightTests.cs of the reference: Test_QWeight_FromData (:29-48, literal vector) and
Test_QWeight_Pack_Unpack (:19-27, round trip on six value ranges).
"""
import json
import os

import numpy as np
import pytest

import oracle


def _golden(golden_dir):
    return json.load(open(os.path.join(golden_dir, "qweight_fromdata.json")))


def test_qweight_fromdata_golden(golden_dir):
    g = _golden(golden_dir)
    combined = 0
    for z, v in enumerate(g["zeros"]):
        combined |= (v & 0xF) << (z * 4)
    assert combined == g["zero_packed"]  # test/QWeightTests.cs:34-38

    scales = np.array(g["scales_f32_bits"], dtype=np.uint32).view(np.float32).astype(np.float16)
    weights = np.array(g["weights"], dtype=np.uint32)
    # HostQWeight(128): Zeros has size/128 = 1 word, Scales size/16 = 8 (src/QWeight.cs:20-21)
    got = oracle.unpack_flat(weights, np.array([combined], dtype=np.uint32), scales)
    want = np.array(g["checks_f32_bits"], dtype=np.uint32).view(np.float32).astype(np.float16)
    assert got.shape == (1024,)
    assert np.array_equal(got.view(np.uint16), want.view(np.uint16))
    # the per-row form used for device-layout matrices agrees on a single 1024-wide row
    rows = oracle.unpack_rows(weights, np.array([combined], dtype=np.uint32), scales, 1024, 1)
    assert np.array_equal(rows.reshape(-1).view(np.uint16), want.view(np.uint16))


def test_fixture_matches_reference_checkout(golden_dir):
    ref = os.path.join(oracle.reference_root(), "test", "QWeightTestData.cs")
    if not os.path.exists(ref):
        pytest.skip("reference checkout not present")
    import importlib.util
    spec = importlib.util.spec_from_file_location("mk", os.path.join(golden_dir, "make_qweight_golden.py"))
    mk = importlib.util.module_from_spec(spec)
    spec.loader.exec_module(mk)
    assert mk.parse(ref) == _golden(golden_dir)


@pytest.mark.parametrize("lo,hi,mul,scale,zero", [
    (0, 15, 1.0, 1.0, 0), (-1, 14, 1.0, 1.0, 1), (-14, 1, 1.0, 1.0, 14), (-7, 8, 1.0, 1.0, 7),
    (0, 15, 10.0, 10.0, 0), (0, 15, None, 0.1, 0),
])
def test_pack_unpack_roundtrip(lo, hi, mul, scale, zero):
    rng = np.random.default_rng(31415)
    ints = rng.integers(lo, hi, size=1024)  # Random.Next(min, max): max exclusive
    if mul is None:
        vals = (ints // 10).astype(np.float16)  # test/QWeightTests.cs:17: integer division
    else:
        vals = (ints * mul).astype(np.float16)
    w, z, s = oracle.pack_flat(vals, np.full(8, scale, np.float32), np.full(8, zero, np.uint32))
    back = oracle.unpack_flat(w, z, s)
    assert np.array_equal(back.view(np.uint16), vals.view(np.uint16))


def test_unpack_rows_padded_zero_words():
    # d_in = 11008 -> 86 groups -> 11 zero words per output (last one half used); 3 outputs
    rng = np.random.default_rng(7)
    rows, cols = 11008, 3
    ws, zs, ss = oracle.qweight_sizes(rows)
    assert (ws, zs, ss) == (1376, 11, 86)
    w = rng.integers(0, 2**32, size=cols * ws, dtype=np.uint64).astype(np.uint32)
    z = rng.integers(0, 2**32, size=cols * zs, dtype=np.uint64).astype(np.uint32)
    s = (0.001 + rng.random(cols * ss) * 0.019).astype(np.float16)
    got = oracle.unpack_rows(w, z, s, rows, cols).astype(np.float32)
    # independent numpy restatement
    wn = ((w.reshape(cols, ws)[:, :, None] >> (np.arange(8, dtype=np.uint32) * 4)) & 0xF).reshape(cols, -1)[:, :rows]
    zn = ((z.reshape(cols, zs)[:, :, None] >> (np.arange(8, dtype=np.uint32) * 4)) & 0xF).reshape(cols, -1)[:, :ss]
    want = ((wn.astype(np.int32) - np.repeat(zn, 128, axis=1)[:, :rows].astype(np.int32)).astype(np.float32)
            * np.repeat(s.reshape(cols, ss).astype(np.float32), 128, axis=1)[:, :rows]).astype(np.float16)
    assert np.array_equal(got.astype(np.float16).view(np.uint16), want.view(np.uint16))
