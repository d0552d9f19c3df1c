"""The work plan of the tcgen05 matrix product, checked on the host: for every way of
dealing the (tile, k-block) units of a product to the blocks of a launch (equal shares of
the line, one whole tile per block when all blocks fit on the GPU at once, the leftover
deal, split-K for the consumer), the blocks' ranges, computed by
the same function the kernel runs, must cover every unit exactly once; shares of one tile
must be consecutive blocks, as the block that adds them assumes.  No GPU is needed: the
library is compiled by nvcc and only its host functions are called."""
import ctypes
import shutil

import pytest

pytestmark = pytest.mark.skipif(shutil.which("nvcc") is None, reason="nvcc is needed to compile the library")

BM, BK = 128, 64


def _lib():
    from grout_b200.kernels.build import module
    lib = module("gemm_tc")
    lib.gb_gemm_tc_plan_for.argtypes = [ctypes.c_int] * 4 + [ctypes.POINTER(ctypes.c_int)]
    lib.gb_gemm_tc_ranges.argtypes = [ctypes.c_int] * 6 + [ctypes.POINTER(ctypes.c_longlong)]
    return lib


def _plan(lib, rows_a, rows_b, k, sms):
    out = (ctypes.c_int * 7)()
    assert lib.gb_gemm_tc_plan_for(rows_a, rows_b, k, sms, out) == 0
    return dict(bn=out[0], blocks=out[1], scratch=out[2], counters=out[3], split=out[4], lead=out[5],
                lean=out[6])


def _ranges(lib, p, blocks, tiles, kblocks, split, lead):
    out = (ctypes.c_longlong * 4)()
    assert lib.gb_gemm_tc_ranges(p, blocks, tiles, kblocks, split, lead, out) == 0
    return [(out[0], out[1]), (out[2], out[3])]


def _cover(lib, blocks, tiles, kblocks, split, lead):
    """Units seen, per tile the list of blocks that touch it, and the longest share."""
    seen = [0] * (tiles * kblocks)
    by_tile = {}
    longest = 0
    for p in range(blocks):
        mine = 0
        for lo, hi in _ranges(lib, p, blocks, tiles, kblocks, split, lead):
            assert 0 <= lo <= hi <= tiles * kblocks
            mine += hi - lo
            for u in range(lo, hi):
                seen[u] += 1
                by_tile.setdefault(u // kblocks, []).append(p)
        longest = max(longest, mine)
    return seen, by_tile, longest


SHAPES = [(19456, 8, 2560), (19456, 64, 2560), (2560, 8, 4096), (2560, 8, 9728), (6144, 1, 2560),
          (151936, 8, 2560), (20000, 40, 520), (21000, 100, 1032), (5120, 1, 8192), (10240, 8, 5120),
          (51200, 8, 5120), (200, 33, 264), (128, 1, 64), (1280, 4096, 520), (24576, 16, 4096)]


@pytest.mark.parametrize("sms", [148, 132, 60])
def test_every_unit_is_worked_exactly_once(sms):
    lib = _lib()
    for rows_a, rows_b, k in SHAPES:
        pl = _plan(lib, rows_a, rows_b, k, sms)
        bn = pl["bn"]
        assert bn in (16, 32, 64, 128, 256) and (bn >= rows_b or bn == 256)
        tiles = -(-rows_a // BM) * -(-rows_b // bn)
        kblocks = -(-k // BK)
        assert pl["counters"] == tiles and 1 <= pl["blocks"]
        assert pl["scratch"] == 2 * pl["blocks"] * bn * BM
        if pl["blocks"] > sms:
            # more blocks than SMs only when every block has whole tiles of its own (one, or
            # for the 32- and 64-column tiles a few) and all blocks fit on the GPU at once: two
            # of the 16-column tiles an SM with the usual ring of stages; three of them, or two
            # of the 32- and 64-column ones, with four
            per_sm = {(16, 0): 2, (16, 1): 3, (32, 1): 2, (64, 1): 2}.get((bn, pl["lean"]))
            assert per_sm is not None and pl["blocks"] <= per_sm * sms and not pl["lead"], pl
            assert tiles % pl["blocks"] == 0 and (pl["blocks"] == tiles or bn in (32, 64)), pl
        else:
            assert not pl["lean"]
        # the launch without split-K: equal shares, or the leftover deal
        seen, by_tile, longest = _cover(lib, pl["blocks"], tiles, kblocks, 0, pl["lead"])
        assert set(seen) == {1}, (rows_a, rows_b, k, sms, pl)
        for t, ps in by_tile.items():
            uniq = sorted(set(ps))
            assert uniq == list(range(uniq[0], uniq[-1] + 1)), (t, uniq)      # consecutive blocks
        if tiles % pl["blocks"] == 0:
            assert all(len(set(ps)) == 1 for ps in by_tile.values())              # no tile is shared
        if pl["lead"]:
            n_left = tiles - pl["blocks"]
            assert pl["blocks"] == sms and 0 < n_left and n_left * pl["lead"] <= sms and pl["lead"] >= 2
            assert kblocks // pl["lead"] >= 4
            assert longest <= kblocks + -(-kblocks // pl["lead"])                # a tile and one share
            for t in range(sms, tiles):                                          # shares of a leftover tile
                first = (t - sms) * pl["lead"]
                assert sorted(set(by_tile[t])) == list(range(first, first + pl["lead"]))
        else:
            assert longest <= -(-tiles * kblocks // pl["blocks"])
        # the split-K launch whose consumer adds the partial products
        s = pl["split"]
        assert s == 0 or 2 <= s <= 8
        if s:
            assert kblocks // s >= 4 and tiles * s <= sms + sms // 6 + tiles
            seen, by_tile, _ = _cover(lib, tiles * s, tiles, kblocks, s, 0)
            assert set(seen) == {1}
            for t, ps in by_tile.items():
                assert sorted(set(ps)) == list(range(t * s, (t + 1) * s))
