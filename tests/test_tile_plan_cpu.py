"""Host side of the persistent kernel's weight streaming, without a GPU: the per-CTA tile lists that `build_mega` hands
to the copy and tail warps. For the shapes the model tests and the benchmark run (13B and 7B, unsharded and sharded over
2 / 4 / 8 ranks with their uneven hidden splits, the small test model) every operator must plan, every output row must be
covered exactly once, and every bulk copy must obey the 16-byte rule and stay inside its ring slot."""
import ctypes

import pytest

from managedllama2_b200 import _lib

SLOT = 43520          # a ring slot of the 4-stage configuration
SLOT_WIDE = 58368     # and of the 3-stage one (8 rows of a 13824-input matrix)


def plan(fmt, rows, cols, nmat, paired, slot, n_cta=148):
    lib = _lib.load()
    out = (ctypes.c_longlong * 8)()
    _lib.check(lib.ml2_debug_tile_plan(fmt, rows, cols, nmat, 1 if paired else 0, slot, n_cta, out))
    return dict(zip(("planned", "covered", "min_tiles", "max_tiles", "bad", "rmax", "kw", "np"), [int(v) for v in out]))


def layer_ops(dim, hidden, tp, hidden_local):
    dl = dim // tp
    return [("qkv", 0, dim, dl, 3, False), ("o", 0, dl, dim, 1, False), ("gate_up", 0, dim, hidden_local, 2, True),
            ("down", 0, hidden_local, dim, 1, False)]


CASES = []
for name, dim, hidden, vocab in (("13b", 5120, 13824, 32000), ("7b", 4096, 11008, 32000), ("small", 1024, 13 * 128, 512)):
    groups = hidden // 128
    for tp in (1, 2, 4, 8):
        if (dim // 128) % tp:
            continue
        for g_local in sorted({groups // tp, -(-groups // tp)}):     # the ranks' uneven shares of the hidden groups
            if g_local == 0:
                continue
            for op in layer_ops(dim, hidden, tp, g_local * 128):
                CASES.append((name, tp) + op)
        CASES.append((name, tp, "classifier", 1, dim, vocab // tp, 1, False))


@pytest.mark.parametrize("model,tp,op,fmt,rows,cols,nmat,paired", CASES)
def test_tile_lists_cover_every_row_once_and_obey_the_copy_rules(model, tp, op, fmt, rows, cols, nmat, paired):
    got = plan(fmt, rows, cols, nmat, paired, SLOT_WIDE)
    assert got["planned"] == 1, got
    assert got["bad"] == 0, got
    assert got["covered"] == cols * (1 if paired else nmat), got
    assert 1 <= got["kw"] <= 21 and got["rmax"] >= 1
    if fmt == 0:
        assert got["rmax"] in (8, 16) and got["np"] >= 2
    # balanced: no CTA streams more than one full tile (plus a boundary remainder per matrix) beyond the fewest
    assert got["max_tiles"] - got["min_tiles"] <= nmat + 1, got


def test_a_slot_too_small_for_eight_rows_is_refused_not_split():
    assert plan(0, 13824, 5120, 1, False, 32768)["planned"] == 0      # 8 rows of 6912 + 56 + 216 bytes do not fit
    assert plan(0, 5120, 5120, 1, False, SLOT)["rmax"] == 16
    assert plan(0, 13824, 5120, 1, False, SLOT_WIDE)["rmax"] == 8     # the wide matrix streams 8-row tiles


def test_inputs_that_are_not_whole_quantisation_groups_are_refused():
    assert plan(0, 5120 + 32, 5120, 1, False, SLOT_WIDE)["planned"] == 0
