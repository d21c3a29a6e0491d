"""The reference's operator surfaces: gpu_expert_ffn (include/gpu.h:70-83) and the CUDA twin of the
cpu_expert engine (include/cpu_expert.h:23-62), checked against the CPU oracle / compiled reference."""
import numpy as np
import pytest

import helpers as H

pytestmark = pytest.mark.gpu


def _experts(fb, seed, n, down_type, n_embd, inter):
    return [H.expert_record(fb, seed, 0, e, down_type, n_embd, inter) for e in range(n)]


@pytest.mark.parametrize("down_type,n", [(H.Q6, 10), (H.Q4, 8), (H.Q6, 1), (H.Q5, 6)])
def test_gpu_expert_ffn_matches_cpu_expert(fb, oracle, down_type, n):
    n_embd, inter, seed = 4096, 1024, 61
    op = fb.GpuOperator()
    ex = _experts(fb, seed, n, down_type, n_embd, inter)
    h = H.hidden(fb, seed, 0, n_embd)
    sc = np.random.default_rng(1).dirichlet(np.ones(n)).astype(np.float32)
    gs = fb.matrix_bytes(H.Q4, inter, n_embd)
    rc, out = op.expert_ffn(h, ex, sc, n_embd, inter, gs, gs, ex[0].size, H.Q4, H.Q4, down_type)
    assert rc == 0
    want = oracle.moe_block(h, ex, sc, None, H.Q4, H.Q4, down_type, gs, gs, n_embd, inter)
    assert H.rel_l2(out, want) < 3e-4
    op.close()


def test_gpu_expert_ffn_takes_records_in_device_memory(fb):
    """Expert pointers may be host memory (the reference's callers) or memory of the GPU: same bits either way."""
    import torch
    n_embd, inter, seed, n = 2048, 512, 67, 5
    op = fb.GpuOperator()
    ex = _experts(fb, seed, n, H.Q6, n_embd, inter)
    h = H.hidden(fb, seed, 0, n_embd)
    sc = np.random.default_rng(2).dirichlet(np.ones(n)).astype(np.float32)
    gs = fb.matrix_bytes(H.Q4, inter, n_embd)
    rc, host = op.expert_ffn(h, ex, sc, n_embd, inter, gs, gs, ex[0].size, H.Q4, H.Q4, H.Q6)
    assert rc == 0
    dev = [torch.from_numpy(e.copy()).cuda() for e in ex]
    mixed = [dev[i].data_ptr() if i % 2 == 0 else ex[i] for i in range(n)]   # device and host records in one call
    rc, got = op.expert_ffn(h, mixed, sc, n_embd, inter, gs, gs, ex[0].size, H.Q4, H.Q4, H.Q6)
    assert rc == 0 and (H.bits(got) == H.bits(host)).all()
    op.close()


def test_gpu_expert_ffn_fp32_activation_definition(fb, oracle, monkeypatch):
    """FOMOE_B200_ACT=f32 makes the operator compute the reference's fp32-activation definition (what its own GPU
    kernels and its CPU fallback loop, src/inference.c:556-575, compute)."""
    n_embd, inter, seed, n = 2048, 512, 73, 6
    monkeypatch.setenv("FOMOE_B200_ACT", "f32")
    op = fb.GpuOperator()
    ex = _experts(fb, seed, n, H.Q6, n_embd, inter)
    h = H.hidden(fb, seed, 0, n_embd)
    sc = np.random.default_rng(3).dirichlet(np.ones(n)).astype(np.float32)
    gs = fb.matrix_bytes(H.Q4, inter, n_embd)
    rc, out = op.expert_ffn(h, ex, sc, n_embd, inter, gs, gs, ex[0].size, H.Q4, H.Q4, H.Q6)
    assert rc == 0
    want = oracle.moe_block(h, ex, sc, None, H.Q4, H.Q4, H.Q6, gs, gs, n_embd, inter, act_f32=True)
    assert H.rel_l2(out, want) < 2e-5
    op.close()


def test_gpu_expert_ffn_rejects_like_the_reference(fb):
    """-1 = "fall back to CPU" for the reference's limits (src/gpu_kernels.hip:8393-8403)."""
    n_embd, inter, seed = 512, 256, 3
    op = fb.GpuOperator()
    ex = _experts(fb, seed, 11, H.Q6, n_embd, inter)
    h = H.hidden(fb, seed, 0, n_embd)
    gs = fb.matrix_bytes(H.Q4, inter, n_embd)
    sc = np.full(11, 1 / 11, dtype=np.float32)
    assert op.expert_ffn(h, ex, sc, n_embd, inter, gs, gs, ex[0].size, H.Q4, H.Q4, H.Q6)[0] == -1      # 11 experts
    assert op.expert_ffn(h, ex[:2], sc[:2], n_embd, inter, gs, gs, ex[0].size, H.Q4, H.Q4, 8)[0] == -1  # Q8_0 down
    assert op.expert_ffn(h, ex[:2], sc[:2], n_embd, inter, gs, gs, 13 << 20, H.Q4, H.Q4, H.Q6)[0] == -1  # stride
    assert op.expert_ffn(h, ex[:2], sc[:2], n_embd, inter, gs, gs, ex[0].size, H.Q4, H.Q4, H.Q6)[0] == 0
    l = fb.lib()
    assert l.gpu_upload_model(op._h, None) == -1
    assert l.gpu_forward(op._h, None, 0, 0) is None
    assert l.gpu_seed_vram_cache(op._h, None, None) == 0
    op.close()


def test_expert_engine_twin(fb, oracle):
    n_embd, inter, seed = 2048, 512, 71
    eng = fb.ExpertEngine(n_embd, inter)
    ex = _experts(fb, seed, 5, H.Q6, n_embd, inter)
    h = H.hidden(fb, seed, 0, n_embd)
    sc = np.array([0.3, 0.25, 0.2, 0.15, 0.1], dtype=np.float32)
    gs = fb.matrix_bytes(H.Q4, inter, n_embd)
    want = oracle.moe_block(h, ex, sc, None, H.Q4, H.Q4, H.Q6, gs, gs, n_embd, inter)
    # synchronous form: reset + one ffn per expert accumulates (src/cpu_expert.c:226-240)
    eng.reset()
    for e, s in zip(ex, sc):
        eng.ffn(e, h, float(s), H.Q4, H.Q4, H.Q6, gs, gs)
    assert H.rel_l2(eng.result(), want) < 3e-4
    # batch form (src/cpu_expert.c:242-279): starts from zero
    eng.submit_async(h, ex, sc, H.Q4, H.Q4, H.Q6, gs, gs)
    eng.wait()
    assert H.rel_l2(eng.result(), want) < 3e-4
    eng.reset()
    assert np.abs(eng.result()).max() == 0.0
    _, comp_us, n = eng.timing()
    assert n >= 2 and comp_us > 0
    eng.close()


def test_down_type_alternates_without_rebuilding(fb, oracle):
    """The 397B model alternates Q6_K and Q4_K down projections from layer to layer: one operator context and one
    expert engine take both (and Q5_K) call after call, and an engine keeps its accumulated sum and quantised input
    when the type changes between two b200_expert_ffn calls of the same layer."""
    n_embd, inter, seed = 2048, 512, 79
    gs = fb.matrix_bytes(H.Q4, inter, n_embd)
    h = H.hidden(fb, seed, 0, n_embd)
    op = fb.GpuOperator()
    for rnd in range(2):
        for dt in (H.Q6, H.Q4, H.Q5):
            ex = _experts(fb, seed + dt, 4, dt, n_embd, inter)
            sc = np.array([0.4, 0.3, 0.2, 0.1], dtype=np.float32)
            rc, out = op.expert_ffn(h, ex, sc, n_embd, inter, gs, gs, ex[0].size, H.Q4, H.Q4, dt)
            assert rc == 0
            want = oracle.moe_block(h, ex, sc, None, H.Q4, H.Q4, dt, gs, gs, n_embd, inter)
            assert H.rel_l2(out, want) < 3e-4, (rnd, dt)
    op.close()
    eng = fb.ExpertEngine(n_embd, inter)
    e6 = _experts(fb, seed, 2, H.Q6, n_embd, inter)
    e4 = _experts(fb, seed + 1, 2, H.Q4, n_embd, inter)
    eng.reset()
    eng.ffn(e6[0], h, 0.5, H.Q4, H.Q4, H.Q6, gs, gs)
    eng.ffn(e4[0], h, 0.3, H.Q4, H.Q4, H.Q4, gs, gs)       # another type inside the same layer
    eng.ffn(e6[1], h, 0.2, H.Q4, H.Q4, H.Q6, gs, gs)
    one = np.ones(1, dtype=np.float32)
    want = (0.5 * oracle.moe_block(h, [e6[0]], one, None, H.Q4, H.Q4, H.Q6, gs, gs, n_embd, inter)
            + 0.3 * oracle.moe_block(h, [e4[0]], one, None, H.Q4, H.Q4, H.Q4, gs, gs, n_embd, inter)
            + 0.2 * oracle.moe_block(h, [e6[1]], one, None, H.Q4, H.Q4, H.Q6, gs, gs, n_embd, inter))
    assert H.rel_l2(eng.result(), want) < 3e-4
    eng.close()


@pytest.mark.parametrize("down_type,n", [(H.Q6, 10), (H.Q4, 3)])
def test_gpu_expert_ffn_q6k_gate_up(fb, oracle, ref, down_type, n):
    """Q6_K gate and up projections (the reference's kernel for them: src/gpu_kernels.hip:1391) through the operator,
    against cpu_expert's definition (src/quant.c:478-607 for all three matrices when down is Q6_K too): the oracle
    and the compiled reference agree bit for bit, the device within the usual bound; mixed gate/up types are refused;
    a Q4_K call on the same context afterwards still works."""
    n_embd, inter, seed = 4096, 1024, 67
    op = fb.GpuOperator()
    ex = [H.expert_record(fb, seed, 0, e, down_type, n_embd, inter, H.Q6) for e in range(n)]
    h = H.hidden(fb, seed, 0, n_embd)
    sc = np.random.default_rng(2).dirichlet(np.ones(n)).astype(np.float32)
    gs = fb.matrix_bytes(H.Q6, inter, n_embd)
    assert ex[0].size == 2 * gs + fb.matrix_bytes(down_type, n_embd, inter)
    rc, out = op.expert_ffn(h, ex, sc, n_embd, inter, gs, gs, ex[0].size, H.Q6, H.Q6, down_type)
    assert rc == 0
    want = oracle.moe_block(h, ex, sc, None, H.Q6, H.Q6, down_type, gs, gs, n_embd, inter)
    assert (H.bits(want) == H.bits(ref.moe_block(h, ex, sc, None, H.Q6, H.Q6, down_type, gs, gs, n_embd, inter))).all()
    err = H.rel_l2(out, want)
    print(f"Q6_K gate/up, down type {down_type}, {n} experts: rel-L2 {err:.2e}")
    assert err < 3e-4
    rc, _ = op.expert_ffn(h, ex, sc, n_embd, inter, gs, gs, ex[0].size, H.Q6, H.Q4, down_type)
    assert rc == -1
    ex4 = _experts(fb, seed, 2, H.Q6, n_embd, inter)
    g4 = fb.matrix_bytes(H.Q4, inter, n_embd)
    rc, out4 = op.expert_ffn(h, ex4, sc[:2], n_embd, inter, g4, g4, ex4[0].size, H.Q4, H.Q4, H.Q6)
    assert rc == 0
    assert H.rel_l2(out4, oracle.moe_block(h, ex4, sc[:2], None, H.Q4, H.Q4, H.Q6, g4, g4, n_embd, inter)) < 3e-4
    op.close()


def test_expert_engine_twin_changes_gate_type_mid_accumulation(fb, oracle):
    """cpu_expert_ffn accumulates score * FFN(x) call by call (src/cpu_expert.c:114-115) whatever the experts' types:
    a Q4_K-gate expert, then a Q6_K-gate expert, then Q4_K again, on one context."""
    n_embd, inter, seed = 1024, 512, 71
    eng = fb.ExpertEngine(n_embd, inter)
    x = H.hidden(fb, seed, 0, n_embd)
    want = np.zeros(n_embd, dtype=np.float32)
    eng.reset()
    for i, (gt, dt, score) in enumerate([(H.Q4, H.Q6, 0.5), (H.Q6, H.Q6, 0.3), (H.Q4, H.Q4, 0.2)]):
        rec = H.expert_record(fb, seed, 0, i, dt, n_embd, inter, gt)
        gs = fb.matrix_bytes(gt, inter, n_embd)
        eng.ffn(rec, x, score, gt, gt, dt, gs, gs)
        one = oracle.moe_block(x, [rec], np.asarray([score], dtype=np.float32), None, gt, gt, dt, gs, gs, n_embd, inter)
        want = (want + one).astype(np.float32)
    got = eng.result()
    assert H.rel_l2(got, want) < 3e-4
    eng.close()

