"""Index arithmetic of the CTA-pair kernel, checked on the CPU.

``eo_debug_pair_schedule`` runs the launcher's planning code and the kernel's own decoders (compiled for the host as
well) over every work item of a launch.  For a range of shapes, tile orders and batch sizes: every tile of every
matrix is covered exactly once, either whole or by K pieces that partition its k-blocks; triangular launches touch
the lower triangle only; the split depends on the matrix shape alone.
"""

import numpy as np
import pytest

from emerging_optimizers_b200 import _native as nat

SHAPES = [
    # M, N, K, tri
    (256, 256, 64, False),
    (512, 768, 4096, False),
    (3072, 3328, 6144, False),  # 156 tiles: the last 8 in two pieces
    (3072, 3328, 24640, False),  # ... in eight pieces of unequal length
    (3000, 3304, 9216, False),  # ragged edges
    (8192, 28672, 8192, False),  # the BX product of the bench workload
    (8192, 8192, 28672, True),  # its Gram product: 528 tiles, 10 of them in 7 pieces
    (8192, 8192, 8192, True),
    (4352, 4352, 15360, True),
    (4096, 4096, 14336, True),  # 136 tiles: last round too full to split
    (2304, 2304, 192, True),  # 9 tile rows: one full band and one tile
    (5000, 5000, 1000, True),  # tile rows not a multiple of the band width
]


def _expected_tiles(M, N, tri):
    tm, tn = -(-M // 256), -(-N // 256)
    return {(i, j) for i in range(tm) for j in range(tn) if not tri or j <= i}


@pytest.fixture
def options():
    changed = []

    def set_option(name, value):
        nat.set_option(name, value)
        changed.append(name)

    yield set_option
    defaults = {"gemm_pair_band": 8, "gemm_pair_group_m": 8, "gemm_split_k": 1}
    for name in changed:
        nat.set_option(name, defaults[name])


@pytest.mark.parametrize("M,N,K,tri", SHAPES)
@pytest.mark.parametrize("batch", [1, 3])
def test_every_tile_is_covered_exactly_once(M, N, K, tri, batch):
    items = nat.pair_schedule(M, N, K, tri, batch)
    num_kb = -(-K // 64)
    want = _expected_tiles(M, N, tri)
    per_matrix = len(items) // batch
    assert per_matrix * batch == len(items)
    first = None
    for b in range(batch):
        rows = items[items[:, 0] == b]
        assert len(rows) == per_matrix
        whole = rows[rows[:, 5] < 0]
        pieces = rows[rows[:, 5] >= 0]
        seen = {(int(r[1]), int(r[2])) for r in whole}
        assert len(seen) == len(whole)  # no whole tile twice
        assert np.all(whole[:, 3] == 0) and np.all(whole[:, 4] == num_kb)
        by_slot = {}
        for r in pieces:
            by_slot.setdefault(int(r[5]), []).append(r)
        for slot, rs in by_slot.items():
            tiles = {(int(r[1]), int(r[2])) for r in rs}
            assert len(tiles) == 1  # one slot, one tile
            tile = tiles.pop()
            assert tile not in seen
            seen.add(tile)
            spans = sorted((int(r[3]), int(r[4])) for r in rs)
            assert spans[0][0] == 0 and spans[-1][1] == num_kb
            assert all(a[1] == b2[0] for a, b2 in zip(spans, spans[1:]))  # the pieces partition the k-blocks
            assert all(hi - lo >= 48 for lo, hi in spans)  # and are long enough to pay for themselves
        assert seen == want
        # slots are numbered consecutively over the batch
        assert sorted(by_slot) == list(range(b * len(by_slot), (b + 1) * len(by_slot)))
        layout = [(int(r[1]), int(r[2]), int(r[3]), int(r[4])) for r in rows]
        if first is None:
            first = layout
        assert layout == first  # every matrix of the batch is cut up like the first: the split ignores the batch


def test_bench_workload_split():
    gram = nat.pair_schedule(8192, 8192, 28672, True)
    assert len(gram) == 518 + 10 * 7 and len(set(gram[gram[:, 5] >= 0][:, 5])) == 10
    bx = nat.pair_schedule(8192, 28672, 8192, False)
    assert len(bx) == 3552 + 32 * 2
    assert len(nat.pair_schedule(4096, 4096, 14336, True)) == 136  # nothing to gain: not split


@pytest.mark.parametrize("band", [0, 1, 5, 8, 12, 64])
@pytest.mark.parametrize("group", [1, 8, 16, 64])
def test_tile_orders_are_permutations(band, group, options):
    options("gemm_pair_band", band)
    options("gemm_pair_group_m", group)
    for M, N, K, tri in ((5000, 5000, 1000, True), (8192, 8192, 8192, True), (3000, 7000, 512, False)):
        items = nat.pair_schedule(M, N, K, tri)
        tiles = [(int(r[1]), int(r[2])) for r in items if r[5] < 0] + list(
            {(int(r[1]), int(r[2])) for r in items if r[5] >= 0}
        )
        assert len(tiles) == len(set(tiles)) and set(tiles) == _expected_tiles(M, N, tri)


def test_band_order_keeps_a_round_compact(options):
    """74 consecutive tiles of the triangular order touch about 9 + 8 row blocks, not all 32."""
    options("gemm_split_k", 0)
    items = nat.pair_schedule(8192, 8192, 28672, True)
    touched = []
    for start in range(0, len(items) - 74, 37):
        chunk = items[start : start + 74]
        touched.append(len(set(chunk[:, 1]) | set(chunk[:, 2])))
    assert sorted(touched)[len(touched) // 2] <= 18 and max(touched) <= 24  # (the worst window straddles two bands)
    options("gemm_pair_band", 0)
    items = nat.pair_schedule(8192, 8192, 28672, True)
    assert len(set(items[:74, 1]) | set(items[:74, 2])) == 32  # whole tile columns: every row block at once


def test_split_off():
    options_before = nat.pair_schedule(8192, 8192, 28672, True)
    nat.set_option("gemm_split_k", 0)
    try:
        items = nat.pair_schedule(8192, 8192, 28672, True)
    finally:
        nat.set_option("gemm_split_k", 1)
    assert len(items) == 528 and np.all(items[:, 5] == -1) and len(options_before) == 588


def test_argument_errors():
    with pytest.raises(nat.NativeLibraryError):
        nat.pair_schedule(128, 256, 64, False)
    with pytest.raises(nat.NativeLibraryError):
        nat.pair_schedule(512, 256, 64, True)
