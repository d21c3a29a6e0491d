"""Shared builders for the parity tests: seeded synthetic experts and comparison metrics."""
import numpy as np

Q4, Q5, Q6 = 12, 13, 14


def rel_l2(a, b):
    a = np.asarray(a, dtype=np.float64)
    b = np.asarray(b, dtype=np.float64)
    return float(np.linalg.norm(a - b) / max(np.linalg.norm(b), 1e-30))


def bits(a):
    return np.ascontiguousarray(a, dtype=np.float32).view(np.uint32)


def expert_record(fb, seed, layer, expert, down_type, n_embd, inter):
    """One expert in the reference's record order: gate | up | down, ggml bytes."""
    return fb.synth_expert_record(seed, layer, expert, down_type, n_embd, inter)


def router_weights(fb, seed, layer, n_experts, n_embd):
    return fb.synth_router(seed, layer, n_experts, n_embd)


def hidden(fb, seed, token, n_embd):
    return fb.synth_hidden(seed, token, n_embd)


def glue(fb, seed, layer, n_embd):
    return fb.synth_glue(seed, layer, n_embd)


def zipf_resident_mask(seed, layer, n_experts, frac=0.4, s=1.1):
    """Seeded residency mask: floor(frac*n) experts sampled without replacement with probability
    proportional to a Zipf(s) profile over a seeded permutation of the expert ids."""
    rng = np.random.default_rng([seed, layer, 0xCA5])
    perm = rng.permutation(n_experts)
    w = 1.0 / np.arange(1, n_experts + 1) ** s
    p = np.empty(n_experts)
    p[perm] = w / w.sum()
    chosen = rng.choice(n_experts, size=int(frac * n_experts), replace=False, p=p)
    mask = np.zeros(16, dtype=np.uint32)
    for e in chosen:
        mask[e >> 5] |= np.uint32(1 << (e & 31))
    return mask


def oracle_layer(orc, fb, seed, layer, h, n_embd, inter, n_experts, top_k, down_type, has_shared=True, mask=None,
                 threshold=1.0, dampen=False, router=None, shared_gate_w=None, act_f32=False):
    """Router -> top-k -> CAR -> experts (+shared) through a CPU checker (Oracle or Ref)."""
    w = router if router is not None else router_weights(fb, seed, layer, n_experts, n_embd)
    ids, scores, all_scores, subs = orc.route(w, h, top_k, mask, threshold, dampen)
    gs = fb.matrix_bytes(Q4, inter, n_embd)
    experts = [expert_record(fb, seed, layer, int(e), down_type, n_embd, inter) for e in ids]
    shared = expert_record(fb, seed, layer, n_experts, down_type, n_embd, inter) if has_shared else None
    if shared_gate_w is None:
        out = orc.moe_block(h, experts, scores, shared, Q4, Q4, down_type, gs, gs, n_embd, inter, act_f32=act_f32)
        return dict(ids=ids, scores=scores, all_scores=all_scores, subs=subs, out=out)
    # gated shared expert (the reference's src/inference.c:582-596): buf_down *= sigmoid(h . w); ffn += buf_down
    routed = orc.moe_block(h, experts, scores, None, Q4, Q4, down_type, gs, gs, n_embd, inter)
    one = np.ones(1, dtype=np.float32)
    sh = orc.moe_block(h, [shared], one, None, Q4, Q4, down_type, gs, gs, n_embd, inter)
    gate = orc.shared_gate(h, shared_gate_w)
    out = (routed + (sh * np.float32(gate)).astype(np.float32)).astype(np.float32)
    return dict(ids=ids, scores=scores, all_scores=all_scores, subs=subs, out=out, gate=gate)
