"""The compare-exchange network of the block-wide best-16 (fomoe_b200/csrc/select.cuh), restated lane by lane in
numpy: sixteen 32-lane bitonic sorts, then four levels of 5-stage bitonic merges that keep the better half.  The
order is the reference's top_k order (src/tensor.c:226-252): value descending, lower index first.  Runs without
a GPU; the CUDA code itself is compared with the oracle in test_gpu_router.py."""
import numpy as np
import pytest

PAD_ID = 0x7FFFFFFF


def better(av, ai, bv, bi):
    return (av > bv) | ((av == bv) & (ai < bi))


def cmpx(v, i, d, keep_better):
    """One compare-exchange step of 32 lanes with partner lane ^ d (fb_cmpx)."""
    lanes = np.arange(32)
    ov, oi = v[lanes ^ d], i[lanes ^ d]
    other_better = better(ov, oi, v, i)
    take = other_better == keep_better
    return np.where(take, ov, v), np.where(take, oi, i)


def sort32(v, i):
    lanes = np.arange(32)
    k = 2
    while k <= 32:
        j = k >> 1
        while j > 0:
            up = ((lanes & k) == 0) | (k == 32)
            lower = (lanes & j) == 0
            v, i = cmpx(v, i, j, lower == up)
            j >>= 1
        k <<= 1
    return v, i


def merge_level(lists_v, lists_i):
    out_v, out_i = [], []
    lanes = np.arange(32)
    for w in range(len(lists_v) // 2):
        src = 2 * w + (lanes >> 4)
        pos = np.where(lanes < 16, lanes, 31 - lanes)
        v = np.array([lists_v[s][p] for s, p in zip(src, pos)], dtype=np.float32)
        i = np.array([lists_i[s][p] for s, p in zip(src, pos)], dtype=np.int64)
        d = 16
        while d > 0:
            v, i = cmpx(v, i, d, (lanes & d) == 0)
            d >>= 1
        out_v.append(v[:16])
        out_i.append(i[:16])
    return out_v, out_i


def block_best16(values):
    n = len(values)
    v = np.full(512, -np.inf, dtype=np.float32)
    i = np.full(512, PAD_ID, dtype=np.int64)
    v[:n] = values
    i[:n] = np.arange(n)
    lv, li = [], []
    for w in range(16):
        sv, si = sort32(v[32 * w:32 * w + 32], i[32 * w:32 * w + 32])
        lv.append(sv[:16])
        li.append(si[:16])
    while len(lv) > 1:
        lv, li = merge_level(lv, li)
    return lv[0], li[0]


def expected(values):
    order = sorted(range(len(values)), key=lambda e: (-float(values[e]), e))[:16]
    return [int(e) for e in order]


@pytest.mark.parametrize("n", [512, 384, 128, 60, 17, 16, 3])
def test_random_values(n):
    rng = np.random.default_rng(n)
    for _ in range(5):
        vals = rng.standard_normal(n).astype(np.float32)
        _, ids = block_best16(vals)
        want = expected(vals)
        assert [int(x) for x in ids[:len(want)]] == want
        assert all(int(x) == PAD_ID for x in ids[len(want):])


def test_ties_keep_lower_index():
    rng = np.random.default_rng(7)
    vals = rng.integers(0, 4, size=512).astype(np.float32)   # many exact ties
    _, ids = block_best16(vals)
    assert [int(x) for x in ids] == expected(vals)
    vals = np.ones(512, dtype=np.float32)                     # all equal: the sixteen lowest indices, in order
    _, ids = block_best16(vals)
    assert [int(x) for x in ids] == list(range(16))


def test_best_entries_in_one_warp():
    vals = np.zeros(512, dtype=np.float32)
    vals[64:96] = np.arange(32, 0, -1)                        # one warp holds all of the best 16 (and more)
    _, ids = block_best16(vals)
    assert [int(x) for x in ids] == list(range(64, 80))
