"""Properties of the CPU oracle that hold at any size (the checker is itself checked): ordering rules of top-k,
invariants of the Q8_K quantiser, and what cache-aware routing may and may not change."""
import numpy as np
import pytest

import helpers as H


def _mask(resident, n_experts):
    m = np.zeros(16, dtype=np.uint32)
    for e in resident:
        m[e >> 5] |= np.uint32(1 << (e & 31))
    return m


@pytest.mark.parametrize("n,k", [(8, 8), (33, 5), (512, 10), (512, 1)])
def test_top_k_is_a_stable_sort_prefix(oracle, n, k):
    rng = np.random.default_rng(n + k)
    x = rng.integers(0, 6, n).astype(np.float32) / 4        # many exact ties
    ids, vals = oracle.top_k(x, k)
    order = sorted(range(n), key=lambda i: (-x[i], i))[:k]    # value descending, lower index first (src/tensor.c:226-252)
    assert list(ids) == order
    assert (vals == x[ids]).all()


def test_q8k_quantiser_invariants(oracle):
    rng = np.random.default_rng(5)
    x = (rng.normal(0, 3, 1024) * rng.choice([0.0, 1e-6, 1.0, 1e4], 1024)).astype(np.float32)
    x[256:512] = 0.0                                          # an all-zero block
    x[512] = 127.0
    x[513:516] = [0.5, 1.5, -2.5]                             # exact halves once iscale == 1 (amax 127)
    x[516:768] = np.clip(x[516:768], -126, 126)
    rec = oracle.quantize_q8k(x).reshape(4, 292)
    for b in range(4):
        d = rec[b, :4].view(np.float32)[0]
        qs = rec[b, 4:260].view(np.int8).astype(np.int32)
        bs = rec[b, 260:292].view(np.int16).astype(np.int32)
        assert (bs == qs.reshape(16, 16).sum(axis=1)).all()   # bsums are the sums of 16
        blk = x[256 * b:256 * (b + 1)]
        if np.abs(blk).max() == 0:
            assert d == 0 and (qs == 0).all()
        else:
            assert np.abs(qs).max() == 127                    # the extreme value maps to +-127
            assert np.abs(qs * d - blk).max() <= 0.5 * d * (1 + 1e-5)
    qs2 = rec[2, 4:260].view(np.int8)
    assert list(qs2[:4]) == [127, 1, 2, -3]                   # roundf: halves go away from zero


@pytest.mark.parametrize("dampen", [False, True])
def test_car_invariants(fb, oracle, dampen):
    n_experts, k, seed = 512, 10, 321
    W = H.router_weights(fb, seed, 0, n_experts, 1024)
    for tok in range(6):
        h = H.hidden(fb, seed, tok, 1024)
        base_ids, base_sc, alls, _ = oracle.route(W, h, k)
        assert abs(float(alls.sum()) - 1.0) < 1e-5 and abs(float(base_sc.sum()) - 1.0) < 1e-5
        everything = _mask(range(n_experts), n_experts)
        ids, sc, _, subs = oracle.route(W, h, k, everything, 0.35, dampen)
        assert subs == 0 and (ids == base_ids).all() and (H.bits(sc) == H.bits(base_sc)).all()   # all resident
        mask = H.zipf_resident_mask(seed, tok, n_experts)
        ids1, sc1, _, subs1 = oracle.route(W, h, k, mask, 1.0, dampen)
        assert subs1 == 0 and (ids1 == base_ids).all()                                            # threshold 1: off
        ids2, sc2, _, subs2 = oracle.route(W, h, k, mask, 0.35, dampen)
        res = {e for e in range(n_experts) if (int(mask[e >> 5]) >> (e & 31)) & 1}
        changed = [r for r in range(k) if ids2[r] != base_ids[r]]
        assert len(changed) == subs2 and len(set(ids2)) == k                                      # unique experts
        for r in changed:
            assert base_ids[r] not in res and ids2[r] in res                                      # only misses move
            assert alls[ids2[r]] >= np.float32(0.35) * alls[base_ids[r]]                           # ratio >= threshold
            if dampen:
                assert sc2[r] <= base_sc[r]                                                        # dampened, not raised
        if not dampen and subs2:
            assert abs(float(sc2.sum()) - 1.0) < 1e-5                                             # renormalised
