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


def write_gguf(path, kvs, tensors, alignment=32, version=3):
    """A GGUF file (the container of include/gguf.h:6-145 of the reference, format version 3): kvs = [(key, type id,
    value)] with type ids 4 u32, 5 i32, 6 f32, 8 string, 9 (element type id, list); tensors = [(name, dims fastest
    first, ggml type id, bytes)].  general.alignment is written when it differs from 32."""
    import struct

    def gstr(s):
        b = s.encode()
        return struct.pack("<Q", len(b)) + b

    def scalar(t, v):
        return {4: lambda: struct.pack("<I", v), 5: lambda: struct.pack("<i", v), 6: lambda: struct.pack("<f", v),
                10: lambda: struct.pack("<Q", v), 7: lambda: struct.pack("<B", int(v)), 8: lambda: gstr(v)}[t]()

    kvs = list(kvs)
    if alignment != 32:
        kvs.append(("general.alignment", 4, alignment))
    out = struct.pack("<IIQQ", 0x46554747, version, len(tensors), len(kvs))
    for key, t, v in kvs:
        out += gstr(key) + struct.pack("<I", t)
        if t == 9:
            et, items = v
            out += struct.pack("<IQ", et, len(items)) + b"".join(scalar(et, x) for x in items)
        else:
            out += scalar(t, v)
    offs, off = [], 0
    for _, _, _, data in tensors:
        offs.append(off)
        off = (off + len(data) + alignment - 1) // alignment * alignment
    for (name, dims, ttype, _), o in zip(tensors, offs):
        out += gstr(name) + struct.pack("<I", len(dims)) + b"".join(struct.pack("<Q", d) for d in dims)
        out += struct.pack("<IQ", ttype, o)
    out += b"\0" * ((len(out) + alignment - 1) // alignment * alignment - len(out))
    with open(path, "wb") as f:
        f.write(out)
        for (_, _, _, data), o in zip(tensors, offs):
            f.write(bytes(data))
            pad = (len(data) + alignment - 1) // alignment * alignment - len(data)
            f.write(b"\0" * pad)


def moe_gguf(fb, path, seed, n_layers, n_embd, inter, n_experts, down_types, shared=True, first_block=0, gate_type=12,
             router_type=0, alignment=32):
    """A model file holding the MoE tensors of `n_layers` blocks, generated from `seed` like the library's table."""
    tensors = []
    for l in range(n_layers):
        b = first_block + l
        recs = [expert_record(fb, seed, l, e, down_types[l], n_embd, inter, gate_type) for e in range(n_experts + (1 if shared else 0))]
        gs = fb.matrix_bytes(gate_type, inter, n_embd)
        w = router_weights(fb, seed, l, n_experts, n_embd)
        if router_type == 1:
            wb = w.astype(np.float16).tobytes()
        elif router_type == 30:
            wb = (w.view(np.uint32) >> 16).astype(np.uint16).tobytes()
        else:
            wb = w.tobytes()
        tensors.append((f"blk.{b}.ffn_gate_inp.weight", [n_embd, n_experts], router_type, wb))
        tensors.append((f"blk.{b}.ffn_gate_exps.weight", [n_embd, inter, n_experts], gate_type,
                        b"".join(r[:gs].tobytes() for r in recs[:n_experts])))
        tensors.append((f"blk.{b}.ffn_up_exps.weight", [n_embd, inter, n_experts], gate_type,
                        b"".join(r[gs:2 * gs].tobytes() for r in recs[:n_experts])))
        tensors.append((f"blk.{b}.ffn_down_exps.weight", [inter, n_embd, n_experts], down_types[l],
                        b"".join(r[2 * gs:].tobytes() for r in recs[:n_experts])))
        if shared:
            r = recs[n_experts]
            tensors.append((f"blk.{b}.ffn_gate_shexp.weight", [n_embd, inter], gate_type, r[:gs].tobytes()))
            tensors.append((f"blk.{b}.ffn_up_shexp.weight", [n_embd, inter], gate_type, r[gs:2 * gs].tobytes()))
            tensors.append((f"blk.{b}.ffn_down_shexp.weight", [inter, n_embd], down_types[l], r[2 * gs:].tobytes()))
        _, normw = glue(fb, seed, l, n_embd)
        tensors.append((f"blk.{b}.post_attention_norm.weight" if l % 2 == 0 else f"blk.{b}.ffn_norm.weight", [n_embd], 0,
                        normw.tobytes()))
        tensors.append((f"blk.{b}.attn_q.weight", [n_embd, 64], 1, np.zeros(n_embd * 64, dtype=np.float16).tobytes()))
    kvs = [("general.architecture", 8, "qwen3moe"), ("qwen3moe.block_count", 4, n_layers + first_block),
           ("qwen3moe.expert_count", 4, n_experts), ("qwen3moe.attention.layer_norm_rms_epsilon", 6, 1e-6),
           ("tokenizer.ggml.tokens", 9, (8, ["<s>", "</s>", "a", "b"])), ("tokenizer.ggml.token_type", 9, (5, [1, 1, 0, 0])),
           ("general.file_type", 4, 15), ("some.flag", 7, True), ("some.big", 10, 1 << 40)]
    write_gguf(path, kvs, tensors, alignment=alignment)
    return tensors

