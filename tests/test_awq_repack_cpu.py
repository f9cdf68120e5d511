"""AWQ -> QWeight repacking, oracle side: the vectorised numpy restatement against the literal loops of RepackQData
(src/ModelConverter.cs:286-321) and against the meaning of the layout (target word (out, in / 8), nibble i = input
8 * word + i). The reference's only pin for its converter is the SHA-256 of a converted 7B download
(test/ConverterTests.cs:22-33), which cannot be reproduced without the network: parity of this step is unpinned."""
import numpy as np
import pytest

import oracle


@pytest.mark.parametrize("height,width", [(8, 8), (4, 8), (1, 8), (2, 16), (3, 24), (12, 16), (108, 24), (86, 8), (40, 32), (128, 64)])
def test_vectorised_equals_loops_and_layout(height, width):
    rng = np.random.default_rng(height * 1000 + width)
    q = rng.integers(0, 2 ** 32, size=height * (width // 8), dtype=np.uint64).astype(np.uint32)
    assert np.array_equal(oracle.awq_repack_qdata(q, height, width), oracle.awq_repack_qdata_loops(q, height, width))
    vals = rng.integers(0, 16, size=(height, width))
    r = oracle.awq_repack_qdata(oracle.awq_pack_v0(vals, height, width), height, width).reshape(width, -1)
    got = np.stack([(r[:, y // 8] >> np.uint32(4 * (y % 8))) & np.uint32(15) for y in range(height)])
    assert np.array_equal(got, vals)


def test_spill_over_of_a_ragged_column_end():
    """108 groups = 13.5 words: the upper half of an output's last zero-point word repeats the first four values of
    the next output, zeros after the last output (src/ModelConverter.cs:288, 308-312)."""
    height, width = 12, 8
    vals = np.arange(height * width).reshape(height, width) % 16
    r = oracle.awq_repack_qdata_loops(oracle.awq_pack_v0(vals, height, width), height, width).reshape(width, 2)
    for x in range(width):
        spill = [(int(r[x, 1]) >> (4 * i)) & 15 for i in range(4, 8)]
        want = [int(vals[i, x + 1]) for i in range(4)] if x + 1 < width else [0, 0, 0, 0]
        assert spill == want


def test_scales_transpose():
    s = np.arange(6, dtype=np.float16).reshape(2, 3)
    assert oracle.awq_repack_scales(s, 2, 3).tolist() == [0, 3, 1, 4, 2, 5]
