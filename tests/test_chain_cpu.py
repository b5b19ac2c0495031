"""CPU tests of how a GEMM chain deals its work to the CTAs (twm_chain_partition runs the same
integer code as the kernel): every unit of every tile is taken exactly once, pieces of a tile are
numbered 0..n-1 in K order, and the load is even."""
import pytest

from tensorwarp_b200 import quantize as q

SHAPES = [  # (N, K)
    (4608, 3584), (3584, 3584), (37888, 3584), (3584, 18944),      # 7B layer
    (9728, 896), (152064, 3584), (8192, 1024), (200, 512), (1, 32), (129, 96), (1024, 28672),
]


@pytest.mark.parametrize("n,k", SHAPES)
@pytest.mark.parametrize("grid", [296, 1, 7, 132])
def test_partition_covers_every_unit_once(twm_lib, n, k, grid):
    n_tiles, nkb = (n + 127) // 128, k // 32
    cover = {}                   # tile -> list of (blk0, blk1, slot, n_pieces)
    loads = []
    for rank in range(grid):
        pieces = q.chain_partition(n_tiles, nkb, grid, rank)
        loads.append(sum(b1 - b0 for _, b0, b1, _, _ in pieces))
        for tile, b0, b1, slot, npc in pieces:
            assert 0 <= tile < n_tiles and 0 <= b0 < b1 <= nkb and b0 % 4 == 0
            assert b1 % 4 == 0 or b1 == nkb
            cover.setdefault(tile, []).append((b0, b1, slot, npc))
    assert sorted(cover) == list(range(n_tiles))
    for tile, ps in cover.items():
        ps.sort()
        assert ps[0][0] == 0 and ps[-1][1] == nkb
        for (a0, a1, _, _), (b0, _, _, _) in zip(ps, ps[1:]):
            assert a1 == b0                                   # contiguous, no overlap
        assert [p[2] for p in ps] == list(range(len(ps)))     # slots in K order
        assert all(p[3] == len(ps) for p in ps)               # every piece knows the tile's piece count
    # even load: no rank more than one unit (4 blocks) above the mean
    busy = [x for x in loads if x > 0]
    assert max(busy) - min(busy) <= 4 or grid > n_tiles * ((nkb + 3) // 4)
    assert sum(loads) == n_tiles * nkb
