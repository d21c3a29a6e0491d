"""Pins the CPU oracle (oracle/fomoe_oracle.c) to the reference: against golden vectors produced by
the reference's own C code (tests/golden/golden.npz, made by tests/golden/make_golden.py) and, when
oracle/_ref/libfomoe_ref.so is present, against that library directly, bit for bit."""
import os

import numpy as np
import pytest

import helpers as H

GOLD = np.load(os.path.join(os.path.dirname(__file__), "golden", "golden.npz"))


def test_fp16_table(oracle):
    got = np.array([oracle.fp16_to_fp32(h) for h in range(65536)], dtype=np.float32).view(np.uint32)
    want = GOLD["fp16_all"]
    nan = ((want & 0x7F800000) == 0x7F800000) & ((want & 0x7FFFFF) != 0)
    assert (got[~nan] == want[~nan]).all()


def test_dequant_q8k_dots_golden(fb, oracle):
    seed = 1001
    q4 = fb.synth_matrix(seed, 0, 0, fb.M_GATE, H.Q4, 8, 4096)
    q6 = fb.synth_matrix(seed, 0, 0, fb.M_DOWN, H.Q6, 8, 1024)
    for r in range(8):
        assert (H.bits(oracle.dequantize(q4[r * 2304:(r + 1) * 2304], H.Q4, 4096)) == H.bits(GOLD["dq4"][r])).all()
        assert (H.bits(oracle.dequantize(q6[r * 840:(r + 1) * 840], H.Q6, 1024)) == H.bits(GOLD["dq6"][r])).all()
    x4, x1 = H.hidden(fb, seed, 0, 4096), H.hidden(fb, seed, 1, 1024)
    assert (oracle.quantize_q8k(x4) == GOLD["q8_4096"]).all()
    assert (oracle.quantize_q8k(x1) == GOLD["q8_1024"]).all()
    assert (H.bits(oracle.matvec_q8(q4, H.Q4, x4, 8, 4096)) == H.bits(GOLD["dot4"])).all()
    assert (H.bits(oracle.matvec_q8(q6, H.Q6, x1, 8, 1024)) == H.bits(GOLD["dot6"])).all()
    q5 = fb.synth_matrix(seed, 0, 1, fb.M_DOWN, H.Q5, 8, 1024)
    for r in range(8):
        assert (H.bits(oracle.dequantize(q5[r * 704:(r + 1) * 704], H.Q5, 1024)) == H.bits(GOLD["dq5"][r])).all()
    assert (H.bits(oracle.matvec_q8(q5, H.Q5, x1, 8, 1024)) == H.bits(GOLD["dot5"])).all()


def test_reference_matvec_pattern_dequant(oracle):
    p4 = GOLD["pat_q4_blocks"]
    got = oracle.dequantize(p4[:12].reshape(-1), H.Q4, 3072)
    assert (H.bits(got) == H.bits(GOLD["pat_q4_dequant_row0"])).all()


def test_car_known_answers(oracle):
    """src/test_v2.c:201-291: ids {0,5,6} with experts {0,1,2,3} cached and 4 in the second tier."""
    alls = np.array([0.5, 0.15, 0.12, 0.08, 0.05, 0.3, 0.2, 0.01], dtype=np.float32)
    mask = np.zeros(16, dtype=np.uint32)
    mask[0] = 0b11111  # both tiers count as resident; the second-tier expert 4 never wins here
    for name, damp in (("car_basic", False), ("car_basic_dampen", True)):
        ids, sc, subs = oracle.car([0, 5, 6], [0.5, 0.3, 0.2], alls, mask, 0.5, damp)
        assert (ids == GOLD[name + "_ids"]).all() and list(ids) == [0, 1, 2]
        assert (H.bits(sc) == H.bits(GOLD[name + "_scores"])).all()
        assert subs == GOLD[name + "_meta"][0] == 2
    assert np.allclose(GOLD["car_basic_scores"], [0.649350643, 0.194805205, 0.155844152], rtol=1e-7)
    assert np.allclose(GOLD["car_basic_dampen_scores"], [0.5, 0.150000006, 0.119999997], rtol=1e-7)
    m2 = np.zeros(16, dtype=np.uint32)
    m2[0] = 1
    ids, sc, subs = oracle.car([5], [0.8], np.array([0.1, 0, 0, 0, 0, 0.8, 0, 0], dtype=np.float32), m2, 0.9, False)
    assert subs == 0 and list(ids) == [5] and GOLD["car_reject_meta"][0] == 0 and GOLD["car_reject_meta"][1] == 1


def test_topk_tie_order(oracle):
    ids, _ = oracle.top_k(np.array([.1, .3, .3, .2, .3, .05, .2, 0], dtype=np.float32), 4)
    assert list(ids) == list(GOLD["topk_tie_ids"]) == [1, 2, 4, 3]


@pytest.mark.parametrize("tag,down_type", [("q6", H.Q6), ("q4", H.Q4), ("q5", H.Q5)])
def test_config0_layer_golden(fb, oracle, tag, down_type):
    seed = 2024
    h = H.hidden(fb, seed, 0, 4096)
    lay = H.oracle_layer(oracle, fb, seed, 0, h, 4096, 1024, 512, 10, down_type)
    assert (lay["ids"] == GOLD[f"cfg0_{tag}_ids"]).all()
    assert (H.bits(lay["scores"]) == H.bits(GOLD[f"cfg0_{tag}_scores"])).all()
    assert (H.bits(lay["out"]) == H.bits(GOLD[f"cfg0_{tag}_out"])).all()


def test_config3_car_golden(fb, oracle):
    seed = 2024
    h = H.hidden(fb, seed, 0, 4096)
    mask = H.zipf_resident_mask(seed, 0, 512)
    assert (mask == GOLD["cfg3_mask"]).all()
    lay = H.oracle_layer(oracle, fb, seed, 0, h, 4096, 1024, 512, 10, H.Q6, mask=mask, threshold=0.35, dampen=True)
    assert (lay["ids"] == GOLD["cfg3_ids"]).all() and lay["subs"] == GOLD["cfg3_subs"][0]
    assert (H.bits(lay["scores"]) == H.bits(GOLD["cfg3_scores"])).all()
    assert (H.bits(lay["out"]) == H.bits(GOLD["cfg3_out"])).all()


def test_stack_golden(fb, oracle):
    seed, n_embd, inter, n_experts, top_k = 4242, 1024, 512, 64, 4
    dts = [H.Q6, H.Q4, H.Q6]
    x = H.hidden(fb, seed, 0, n_embd)
    for l in range(3):
        r_, w_ = H.glue(fb, seed, l, n_embd)
        x = x + r_
        hh = oracle.rms_norm(x, w_, 1e-6)
        lay = H.oracle_layer(oracle, fb, seed, l, hh, n_embd, inter, n_experts, top_k, dts[l])
        x = x + lay["out"]
        assert (lay["ids"] == GOLD["stack_ids"][l]).all()
        assert (H.bits(x) == H.bits(GOLD["stack_x"][l])).all()


# ---- direct comparison with the compiled reference (skipped where it was not built) ----
def test_oracle_equals_compiled_reference(fb, oracle, ref):
    rng = np.random.default_rng(3)
    for qt, m, rows, cols in ((H.Q4, fb.M_GATE, 6, 4096), (H.Q6, fb.M_DOWN, 6, 1024), (H.Q4, fb.M_DOWN, 6, 1024),
                              (H.Q5, fb.M_DOWN, 6, 1024)):
        w = fb.synth_matrix(77, 1, 2, m, qt, rows, cols)
        rb = fb.matrix_bytes(qt, 1, cols)
        x = rng.normal(0, 2, cols).astype(np.float32)
        qa, qb = oracle.quantize_q8k(x), ref.quantize_q8k(x)
        assert (qa == qb).all()
        for r in range(rows):
            row = w[r * rb:(r + 1) * rb]
            assert (H.bits(oracle.dequantize(row, qt, cols)) == H.bits(ref.dequantize(row, qt, cols))).all()
            assert H.bits(oracle.vec_dot(row, qt, qa, cols // 256)) == H.bits(ref.vec_dot(row, qt, qa, cols // 256))
    W = H.router_weights(fb, 77, 0, 512, 4096)
    h = H.hidden(fb, 77, 0, 4096)
    assert (H.bits(oracle.router_logits(W, h)) == H.bits(ref.router_logits(W, h))).all()
    w_ = rng.normal(1, 0.1, 4096).astype(np.float32)
    assert (H.bits(oracle.rms_norm(h, w_, 1e-6)) == H.bits(ref.rms_norm(h, w_, 1e-6))).all()
    for layer in range(3):
        mask = H.zipf_resident_mask(77, layer, 512)
        for thr, damp in ((1.0, False), (0.35, True), (0.35, False), (0.7, False)):
            a = oracle.route(W, H.hidden(fb, 77, layer, 4096), 10, mask, thr, damp)
            b = ref.route(W, H.hidden(fb, 77, layer, 4096), 10, mask, thr, damp)
            assert (a[0] == b[0]).all() and a[3] == b[3]
            assert (H.bits(a[1]) == H.bits(b[1])).all() and (H.bits(a[2]) == H.bits(b[2])).all()
    lay_o = H.oracle_layer(oracle, fb, 78, 0, h, 4096, 1024, 512, 10, H.Q6)
    lay_r = H.oracle_layer(ref, fb, 78, 0, h, 4096, 1024, 512, 10, H.Q6)
    assert (H.bits(lay_o["out"]) == H.bits(lay_r["out"])).all()


@pytest.mark.parametrize("down_type", [H.Q4, H.Q5, H.Q6])
def test_fp32_activation_definition_equals_compiled_reference(fb, oracle, ref, down_type):
    """The reference's second definition of the expert FFN (fp32 activations: src/inference.c:556-596 over
    src/tensor.c and src/quant.c:109-143, 177-212, 249-262), restated and compared bit for bit."""
    n_embd, inter, seed = 1024, 512, 9
    ex = [H.expert_record(fb, seed, 0, e, down_type, n_embd, inter) for e in range(4)]
    sh = H.expert_record(fb, seed, 0, 7, down_type, n_embd, inter)
    h = H.hidden(fb, seed, 0, n_embd)
    sc = np.array([.4, .3, .2, .1], dtype=np.float32)
    gs = fb.matrix_bytes(H.Q4, inter, n_embd)
    a = oracle.moe_block(h, ex, sc, sh, H.Q4, H.Q4, down_type, gs, gs, n_embd, inter, act_f32=True)
    b = ref.moe_block(h, ex, sc, sh, H.Q4, H.Q4, down_type, gs, gs, n_embd, inter, act_f32=True)
    assert (H.bits(a) == H.bits(b)).all()
    q = ref.moe_block(h, ex, sc, sh, H.Q4, H.Q4, down_type, gs, gs, n_embd, inter)
    assert 1e-3 < H.rel_l2(q, b) < 0.2      # the two definitions are not interchangeable at the 1e-3 bar


def test_q8k_activation_path_differs_from_fp32_path(fb, ref):
    """The parity target is the Q8_K-activation path of src/cpu_expert.c; the fp32-activation matvec of
    src/tensor.c is a different definition (about 1e-2 apart), which is why the kernels quantise."""
    w = fb.synth_matrix(5, 0, 0, fb.M_GATE, H.Q4, 64, 4096)
    x = H.hidden(fb, 5, 0, 4096)
    a = ref.matvec_q8(w, H.Q4, x, 64, 4096)
    b = ref.mat_vec_mul_f32act(w, H.Q4, x, 64, 4096)
    assert 1e-4 < H.rel_l2(a, b) < 1e-1


@pytest.mark.parametrize("qtype", [H.Q8_0, H.MXFP4])
def test_blocks32_dequant_and_dot_pin(oracle, ref, qtype):
    """Q8_0 and MXFP4 (src/quant.c:266-337): dequantised rows and the fp32-activation matvec of the restatement equal
    the compiled reference bit for bit, special blocks included."""
    rows, cols = 48, 2048
    m = H.blocks32_matrix(qtype, rows, cols, 17 + qtype)
    rb = (cols // 32) * (34 if qtype == H.Q8_0 else 17)
    for r in (0, 1, rows - 1):
        a, b = oracle.dequantize32(m[r * rb:(r + 1) * rb], qtype, cols), ref.dequantize32(m[r * rb:(r + 1) * rb], qtype, cols)
        assert (H.bits(a) == H.bits(b)).all()
    x = np.random.default_rng(3).standard_normal(cols).astype(np.float32)
    got, want = oracle.mat_vec_mul_f32act(m, qtype, x, rows, cols), ref.mat_vec_mul_f32act(m, qtype, x, rows, cols)
    assert (H.bits(got) == H.bits(want)).all()
    assert np.isfinite(want).all() and np.abs(want).max() > 0


def test_shared_ffn_f32_pin(oracle, ref):
    """The shared expert on fp32 activations (src/inference.c:361-374) with MXFP4 gate/up and Q8_0 down, and the
    other way round: restatement == the reference's own mat_vec_mul / silu / vec_mul composition, bit for bit."""
    n_embd, inter = 1024, 512
    h = np.random.default_rng(9).standard_normal(n_embd).astype(np.float32)
    for gt, dt in ((H.MXFP4, H.Q8_0), (H.Q8_0, H.MXFP4)):
        g, u = H.blocks32_matrix(gt, inter, n_embd, 1), H.blocks32_matrix(gt, inter, n_embd, 2)
        d = H.blocks32_matrix(dt, n_embd, inter, 3)
        a = oracle.shared_ffn_f32(h, g, gt, u, gt, d, dt, n_embd, inter)
        b = ref.shared_ffn_f32(h, g, gt, u, gt, d, dt, n_embd, inter)
        assert (H.bits(a) == H.bits(b)).all() and np.abs(a).max() > 0

