"""Router -> softmax -> ordered top-k -> CAR on the device against the CPU oracle
(reference src/tensor.c:104-113, 186-252; src/inference.c:496-502; src/car.c:36-264;
classify loop src/gpu_kernels.hip:7097-7187).  Expert ids must match index for index."""
import numpy as np
import pytest

import helpers as H

pytestmark = pytest.mark.gpu

SCORE_TOL = 2e-5  # relative; GPU expf and summation order differ from glibc in the last bits


def _mk(fb, n_layers, n_embd, n_experts, top_k, seed, **kw):
    d = fb.MoeDecoder(n_layers, n_embd, 256, n_experts, top_k, False, [H.Q4] * n_layers, **kw)
    d.generate(seed)
    return d


@pytest.mark.parametrize("n_experts,top_k,n_embd", [(512, 10, 4096), (256, 8, 2048), (64, 4, 512), (8, 3, 256)])
def test_topk_ids_bit_exact(fb, oracle, n_experts, top_k, n_embd):
    d = _mk(fb, 3, n_embd, n_experts, top_k, 31)
    for layer in range(3):
        w = H.router_weights(fb, 31, layer, n_experts, n_embd)
        for tok in range(6):
            h = H.hidden(fb, 31, 100 * layer + tok, n_embd)
            got = d.moe_layer(layer, h)
            ids, scores, alls, _ = oracle.route(w, h, top_k)
            assert (got["ids"] == ids).all(), (layer, tok, got["ids"], ids)
            assert (got["ids_orig"] == ids).all()
            assert np.allclose(got["scores"], scores, rtol=SCORE_TOL, atol=0)
            assert np.allclose(got["all_scores"], alls, rtol=SCORE_TOL, atol=1e-12)
    assert d.status() == 0
    d.close()


@pytest.mark.parametrize("threshold,dampen", [(0.35, True), (0.35, False), (1.0, True), (0.0, True), (0.9, False)])
def test_car_substitutions_match(fb, oracle, threshold, dampen):
    n_experts, top_k, n_embd = 512, 10, 4096
    d = _mk(fb, 2, n_embd, n_experts, top_k, 41, car_threshold=threshold, car_dampen=dampen)
    total = 0
    for layer in range(2):
        mask = H.zipf_resident_mask(41, layer, n_experts)
        d.set_resident_mask(layer, mask)
        w = H.router_weights(fb, 41, layer, n_experts, n_embd)
        for tok in range(8):
            h = H.hidden(fb, 41, 50 * layer + tok, n_embd)
            got = d.moe_layer(layer, h)
            ids, scores, alls, subs = oracle.route(w, h, top_k, mask, threshold, dampen)
            ids0, _, _, _ = oracle.route(w, h, top_k)
            assert (got["ids_orig"] == ids0).all()
            assert (got["ids"] == ids).all(), (layer, tok, got["ids"], ids)
            assert np.allclose(got["scores"], scores, rtol=SCORE_TOL, atol=0)
            total += subs
    assert d.substitutions() == total
    if threshold in (1.0, 0.0):
        assert total == 0
    if threshold == 0.35:
        assert total > 0
    d.close()


def test_car_reference_scenarios(fb, oracle):
    """The reference's own CAR scenario (src/test_v2.c:201-246): 8 experts, selected {0,5,6}, resident
    {0,1,2,3}: experts 5 and 6 are replaced by 1 and 2.  The raw car_evaluate answers are pinned on the
    CPU side; here the device must agree with the oracle on the same router."""
    n_embd = 256
    d = fb.MoeDecoder(1, n_embd, 256, 8, 3, False, [H.Q4], car_threshold=0.45)
    d.generate(1)
    target = np.array([0.5, 0.15, 0.12, 0.08, 0.05, 0.3, 0.2, 0.01], dtype=np.float64)
    w = np.zeros((8, n_embd), dtype=np.float32)
    w[:, 0] = np.log(target / target.sum()).astype(np.float32)
    h = np.zeros(n_embd, dtype=np.float32)
    h[0] = 1.0
    d.upload_router(0, w)
    mask = np.zeros(16, dtype=np.uint32)
    mask[0] = 0b1111
    d.set_resident_mask(0, mask)
    for thr, damp, expect in ((0.45, False, [0, 1, 2]), (0.45, True, [0, 1, 2]), (0.9, False, [0, 5, 6])):
        d.set_car(thr, damp)
        got = d.moe_layer(0, h)
        ids, scores, _, subs = oracle.route(w, h, 3, mask, thr, damp)
        assert list(got["ids_orig"]) == [0, 5, 6]
        assert list(got["ids"]) == expect == list(ids)
        assert np.allclose(got["scores"], scores, rtol=SCORE_TOL)
    d.set_car(0.45, True)
    assert np.allclose(d.moe_layer(0, h)["scores"], [0.5, 0.15, 0.12], rtol=1e-4)  # dampened, not renormalised
    d.close()


def test_exact_ties_keep_lower_index(fb, oracle):
    """Identical router rows give identical logits: the CPU's top_k keeps the lower index first
    (src/tensor.c:226-252); near-identical rows exercise the exact-order arbiter."""
    n_experts, top_k, n_embd = 64, 6, 1024
    d = _mk(fb, 1, n_embd, n_experts, top_k, 5)
    w = H.router_weights(fb, 5, 0, n_experts, n_embd).copy()
    h = H.hidden(fb, 5, 0, n_embd)
    base = oracle.route(w, h, top_k)[0]
    # duplicate the best row into two other slots (exact three-way tie), and the 3rd-best into one more
    w[40] = w[base[0]]
    w[7] = w[base[0]]
    w[63] = w[base[2]]
    d.upload_router(0, w)
    got = d.moe_layer(0, h)
    want = oracle.route(w, h, top_k)[0]
    assert (got["ids"] == want).all(), (got["ids"], want)
    # near ties: perturb one element by one ulp-ish amount so the sums differ only in the last bits
    rng = np.random.default_rng(0)
    for trial in range(20):
        w2 = w.copy()
        j = int(rng.integers(0, n_embd))
        w2[40, j] = np.nextafter(w2[40, j], np.float32(1.0 if trial % 2 else -1.0))
        w2[7, (j + 1) % n_embd] = np.nextafter(w2[7, (j + 1) % n_embd], np.float32(-1.0 if trial % 2 else 1.0))
        d.upload_router(0, w2)
        got = d.moe_layer(0, h)
        want = oracle.route(w2, h, top_k)[0]
        assert (got["ids"] == want).all(), (trial, got["ids"], want)
    d.close()
