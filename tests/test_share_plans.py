"""The tensor-core kernel's sharing of tiles between CTAs, checked on the host (no GPU): every
main k-stage of every tile is multiplied exactly once, a tile split between CTAs is split between
neighbours in ascending order with the last stages on the highest CTA, every CTA dumps at most one
unfinished piece and works on it first, and the CTAs' loads differ by less than one tile."""
import ctypes

import pytest

from unifur_b200 import _lib

SHAPES = [
    (2048, 4096, 14336),   # configuration 3: 896 tiles on 148 CTAs
    (4096, 3584, 3584), (4096, 3584, 512), (4096, 3584, 18944), (4096, 18944, 3584),   # the block's projections
    (4096, 18944, 1792), (4096, 18944, 896), (4096, 18944, 448), (4096, 3584, 64),     # and their shards
    (2048, 4096, 7168), (2048, 4096, 1792),
    (512, 4096, 256), (300, 3072, 200), (768, 1536, 6400), (17, 64, 8), (40, 64, 40000), (257, 192, 136),
]


def _plan(rows, d_in, d_out):
    L = _lib.load()
    ctas = ctypes.c_uint32(0)
    cap = 4096
    seg = (ctypes.c_uint32 * (3 * cap))()
    n0 = L.nf4_prefill_share_plan(rows, d_in, d_out, 0, ctypes.byref(ctas), seg, cap)
    assert n0 >= 0 and 1 <= ctas.value <= 148
    out = []
    for c in range(ctas.value):
        n = L.nf4_prefill_share_plan(rows, d_in, d_out, c, None, seg, cap)
        assert 0 <= n <= cap
        out.append([(seg[3 * j], seg[3 * j + 1], seg[3 * j + 2]) for j in range(n)])
    return out


@pytest.mark.parametrize("rows,d_in,d_out", SHAPES)
def test_every_stage_once_and_neighbours_share(rows, d_in, d_out):
    plan = _plan(rows, d_in, d_out)
    ks = d_in // 64
    tiles = ((rows + 255) // 256) * ((d_out + 127) // 128)
    pieces = {}
    for c, segs in enumerate(plan):
        unfinished = [j for j, (_t, _b, e) in enumerate(segs) if e != ks]
        assert len(unfinished) <= 1 and (not unfinished or unfinished[0] == 0)   # dumped first, at most one
        for tile, b, e in segs:
            assert tile < tiles and 0 <= b < e <= ks
            pieces.setdefault(tile, []).append((b, e, c))
    assert sorted(pieces) == list(range(tiles))
    for tile, ps in pieces.items():
        ps.sort()
        assert ps[0][0] == 0 and ps[-1][1] == ks
        for (b0, e0, c0), (b1, e1, c1) in zip(ps, ps[1:]):
            assert e0 == b1 and c1 == c0 + 1        # contiguous stages, consecutive CTAs
    loads = [sum(e - b for _t, b, e in segs) for segs in plan]
    assert max(loads) - min(loads) <= ks             # nobody has a whole tile more than anybody else


def test_rejects_what_the_kernel_does_not_take():
    L = _lib.load()
    seg = (ctypes.c_uint32 * 3)()
    assert L.nf4_prefill_share_plan(16, 4096, 4096, 0, None, seg, 1) < 0      # decode-sized
    assert L.nf4_prefill_share_plan(64, 100, 4096, 0, None, seg, 1) < 0       # d_in not a multiple of 64
    assert L.nf4_prefill_share_plan(64, 4096, 4096, 500, None, seg, 1) < 0    # no such CTA


@pytest.mark.parametrize("rows,d_in,d_out,rank", [
    (1, 4096, 11008, 16), (16, 4096, 11008, 16), (8, 3584, 3584, 16), (8, 3584, 512, 16), (8, 3584, 18944, 16),
    (8, 18944, 3584, 16), (4, 2048, 64, 0), (5, 1024, 1000, 16), (3, 512, 200, 8), (5, 32768, 48, 32),
    (16, 4096, 160, 64), (1, 8192, 384, 16), (8, 4352, 96, 8), (1, 256, 16, 0),
])
def test_decode_kernel_shares_rows_and_k_exactly(rows, d_in, d_out, rank):
    # every (row of W, k) belongs to exactly one CTA: the parts of K tile [0, d_in), and within a
    # part the CTAs' row ranges tile [0, d_out) in order
    L = _lib.load()
    out = (ctypes.c_uint32 * 4)()
    ctas = L.nf4_decode_share_plan(rows, d_in, d_out, rank, 0, out)
    assert 1 <= ctas <= 148
    parts = {}
    for c in range(ctas):
        assert L.nf4_decode_share_plan(rows, d_in, d_out, rank, c, out) == ctas
        k0, k1, n0, n1 = out[0], out[1], out[2], out[3]
        assert k0 < k1 <= d_in and k1 - k0 <= 4096 and n0 <= n1 <= d_out
        parts.setdefault((k0, k1), []).append((n0, n1))
    ks = sorted(parts)
    assert ks[0][0] == 0 and ks[-1][1] == d_in and all(a[1] == b[0] for a, b in zip(ks, ks[1:]))
    for ranges in parts.values():
        assert ranges[0][0] == 0 and ranges[-1][1] == d_out
        assert all(a[1] == b[0] for a, b in zip(ranges, ranges[1:]))
    assert L.nf4_decode_share_plan(17, 4096, 64, 0, 0, out) < 0 and L.nf4_decode_share_plan(4, 100, 64, 0, 0, out) < 0
