"""Shared builders for the parity tests: seeded synthetic experts and comparison metrics."""
import numpy as np

Q4, Q5, Q6 = 12, 13, 14


def rel_l2(a, b):
    a = np.asarray(a, dtype=np.float64)
    b = np.asarray(b, dtype=np.float64)
    return float(np.linalg.norm(a - b) / max(np.linalg.norm(b), 1e-30))


def bits(a):
    return np.ascontiguousarray(a, dtype=np.float32).view(np.uint32)


def expert_record(fb, seed, layer, expert, down_type, n_embd, inter, gate_type=12):
    """One expert in the reference's record order: gate | up | down, ggml bytes."""
    return fb.synth_expert_record(seed, layer, expert, down_type, n_embd, inter, gate_type)


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
                 threshold=1.0, dampen=False, router=None, shared_gate_w=None, act_f32=False, gate_type=None):
    """Router -> top-k -> CAR -> experts (+shared) through a CPU checker (Oracle or Ref)."""
    w = router if router is not None else router_weights(fb, seed, layer, n_experts, n_embd)
    ids, scores, all_scores, subs = orc.route(w, h, top_k, mask, threshold, dampen)
    gt = Q4 if gate_type is None else gate_type
    gs = fb.matrix_bytes(gt, inter, n_embd)
    experts = [expert_record(fb, seed, layer, int(e), down_type, n_embd, inter, gt) for e in ids]
    shared = expert_record(fb, seed, layer, n_experts, down_type, n_embd, inter, gt) if has_shared else None
    if shared_gate_w is None:
        out = orc.moe_block(h, experts, scores, shared, gt, gt, down_type, gs, gs, n_embd, inter, act_f32=act_f32)
        return dict(ids=ids, scores=scores, all_scores=all_scores, subs=subs, out=out)
    # gated shared expert (the reference's src/inference.c:582-596): buf_down *= sigmoid(h . w); ffn += buf_down
    routed = orc.moe_block(h, experts, scores, None, Q4, Q4, down_type, gs, gs, n_embd, inter)
    one = np.ones(1, dtype=np.float32)
    sh = orc.moe_block(h, [shared], one, None, Q4, Q4, down_type, gs, gs, n_embd, inter)
    gate = orc.shared_gate(h, shared_gate_w)
    out = (routed + (sh * np.float32(gate)).astype(np.float32)).astype(np.float32)
    return dict(ids=ids, scores=scores, all_scores=all_scores, subs=subs, out=out, gate=gate)


def parse_trace(path):
    """The reader's view of a routing trace (the format tools/read_trace.py of the reference parses)."""
    import struct
    data = open(path, "rb").read()
    magic, version, n_layers, n_experts, top_k, _, _, _ = struct.unpack("<IIHHHHQQ", data[:32])
    assert magic == 0x54524345 and version == 1
    fmt = f"<IHBB{top_k}h{top_k}f{top_k}h{top_k}f{top_k}B"
    pad = (8 - struct.calcsize(fmt) % 8) % 8
    fmt += f"{pad}x" if pad else ""
    size = struct.calcsize(fmt)
    assert (len(data) - 32) % size == 0
    recs = []
    for off in range(32, len(data), size):
        f = struct.unpack_from(fmt, data, off)
        k = top_k
        recs.append(dict(token=f[0], layer=f[1], n_used=f[2], n_subs=f[3], orig_ids=list(f[4:4 + k]),
                         orig_scores=list(f[4 + k:4 + 2 * k]), final_ids=list(f[4 + 2 * k:4 + 3 * k]),
                         final_scores=list(f[4 + 3 * k:4 + 4 * k]), source=list(f[4 + 4 * k:4 + 5 * k])))
    return dict(n_layers=n_layers, n_experts=n_experts, top_k=top_k, rec_size=size, records=recs)


Q8_0, MXFP4 = 8, 39


def blocks32_matrix(qtype, rows, cols, seed, special=True):
    """A seeded matrix in 32-value blocks, ggml byte order: Q8_0 {fp16 d, int8 qs[32]} with d = |N(0, 1e-2)|, or
    MXFP4 {e8m0 s, 16 nibble bytes} with exponents 2^-17 .. 2^7; a few special blocks when asked: the NaN exponent
    0xFF (read as scale 0), the smallest exponent 0 (2^-127, a subnormal), d = 0 and the extreme quants."""
    rng = np.random.default_rng(seed)
    nb = cols // 32
    if qtype == Q8_0:
        m = np.zeros((rows, nb, 34), dtype=np.uint8)
        d = (np.abs(rng.standard_normal((rows, nb))) * 1e-2).astype(np.float16)
        if special:
            d[0, 0] = 0.0
        m[:, :, 0:2] = d.view(np.uint8).reshape(rows, nb, 2)
        m[:, :, 2:] = rng.integers(0, 256, (rows, nb, 32), dtype=np.uint8)
        if special:
            m[rows - 1, nb - 1, 2:] = 0x80          # all -128
            m[rows - 1, 0, 2:] = 0x7F               # all +127
    else:
        m = rng.integers(0, 256, (rows, nb, 17), dtype=np.uint8)
        m[:, :, 0] = rng.integers(110, 135, (rows, nb), dtype=np.uint8)
        if special:
            m[0, 0, 0] = 255
            m[1 % rows, 1 % nb, 0] = 0
    return m.reshape(-1)

