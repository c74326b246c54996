"""The thread-to-work mappings of the dense stack kernels (hgq2_b200/csrc/dense_chain.cu: mc_map, mc_rows_product_any, the
unit / split items of the weight-gradient product, the column passes, mc_foreach), restated in Python and checked on the CPU
for EVERY layer width from 1 to 64 and several tile heights: each output element must be produced by exactly one thread, and
nothing may be stored that was not computed.  The GPU parity tests cover a dozen widths; this covers the rest of the index
arithmetic."""

import pytest

T = 512            # kMcThreads
HEIGHTS = (8, 16, 56, 112, 128)


def mc_map(R, width):
    groups = (width + 3) // 4
    rows_per_thread = 4 if groups >= 12 else 2
    slots = min(T // groups, (R + rows_per_thread - 1) // rows_per_thread)
    return groups, slots


@pytest.mark.parametrize('R', HEIGHTS)
def test_row_products_cover_every_output_once(R):
    for width in range(1, 65):
        groups, slots = mc_map(R, width)
        jn = (R + slots - 1) // slots
        assert jn <= 4
        computed_rows = 1 if jn <= 1 else (2 if jn == 2 else 4)   # the instantiation mc_rows_product_any picks
        cover = {}
        for tid in range(T):
            cg, slot = tid % groups, tid // groups
            if not (slot < slots and slot < R):
                continue
            for j in range(4):
                r = slot + j * slots
                if r < R:
                    assert j < computed_rows, (R, width, tid, j)
                    for c in range(4):
                        if cg * 4 + c < width:
                            cover[(r, cg * 4 + c)] = cover.get((r, cg * 4 + c), 0) + 1
        assert len(cover) == R * width and set(cover.values()) == {1}, (R, width)


@pytest.mark.parametrize('R', HEIGHTS)
def test_weight_gradient_items_cover_every_row_of_every_unit_once(R):
    for K in range(1, 65):
        for N in (1, 3, 5, 8, 20, 27, 32, 33, 64):
            units = ((K + 3) // 4) * ((N + 3) // 4)
            splits = max(1, min(T // units, R >> 3))
            rps = (R + splits - 1) // splits
            assert units * splits <= T
            rows = {}
            for tid in range(units * splits):
                unit, sp = tid % units, tid // units
                for r in range(sp * rps, min(R, sp * rps + rps)):
                    rows[(unit, r)] = rows.get((unit, r), 0) + 1
            assert len(rows) == units * R and set(rows.values()) == {1}, (R, K, N)


@pytest.mark.parametrize('R', HEIGHTS)
def test_column_passes_and_element_loops_cover_every_element_once(R):
    for width in range(1, 65):
        subsets = T // width                       # the df / dbq passes
        seen = {}
        for tid in range(subsets * width):
            for r in range(tid // width, R, subsets):
                seen[(r, tid % width)] = seen.get((r, tid % width), 0) + 1
        assert len(seen) == R * width and set(seen.values()) == {1}, ('column pass', R, width)
        seen = {}                                   # mc_foreach
        for tid in range(T):
            if T % width == 0:
                for r in range(tid // width, R, T // width):
                    seen[(r, tid % width)] = seen.get((r, tid % width), 0) + 1
            else:
                for e in range(tid, R * width, T):
                    seen[(e // width, e % width)] = seen.get((e // width, e % width), 0) + 1
        assert len(seen) == R * width and set(seen.values()) == {1}, ('element loop', R, width)
