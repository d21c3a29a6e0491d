"""GGUF ingestion.  CPU part: a model file written by the test (format version 3) is read by the library's own GGUF
reader and by the reference's (src/gguf.c, compiled unmodified into the reference checker): same directory, same
bytes.  GPU part: the MoE tensors of the file land in the table, router and norm weights in their places, and a layer
computed from the loaded context equals the oracle on the original tensors."""
import ctypes as C

import numpy as np
import pytest

import helpers as H


def _ref_read(ref, path, name, nbytes):
    lib = ref.lib
    lib.gguf_open.argtypes = [C.c_char_p]
    lib.gguf_open.restype = C.c_void_p
    lib.gguf_close.argtypes = [C.c_void_p]
    lib.gguf_find_tensor.argtypes = [C.c_void_p, C.c_char_p]
    lib.gguf_find_tensor.restype = C.c_int64
    lib.gguf_read_tensor.argtypes = [C.c_void_p, C.c_int64, C.c_void_p, C.c_size_t]
    lib.gguf_read_tensor.restype = C.c_size_t
    g = lib.gguf_open(str(path).encode())
    assert g, "the reference's reader rejects the file"
    try:
        tid = lib.gguf_find_tensor(g, name.encode())
        if tid < 0:
            return None
        buf = np.empty(nbytes, dtype=np.uint8)
        got = lib.gguf_read_tensor(g, tid, buf.ctypes.data, nbytes)
        assert got == nbytes, (name, got, nbytes)
        return buf
    finally:
        lib.gguf_close(g)


@pytest.mark.parametrize("alignment", [32, 64])
def test_reader_agrees_with_the_reference_reader(fb, ref, tmp_path, alignment):
    path = tmp_path / "model.gguf"
    tensors = H.moe_gguf(fb, path, 11, 2, 256, 256, 4, [H.Q6, H.Q4], first_block=3, alignment=alignment)
    for name, dims, ttype, data in tensors:
        got = fb.gguf_tensor(path, name)
        assert got is not None, name
        t, d, raw = got
        assert t == ttype and d[:len(dims)] == list(dims) and all(x == 1 for x in d[len(dims):])
        assert raw.tobytes() == bytes(data)
        assert _ref_read(ref, path, name, len(data)).tobytes() == bytes(data)
    assert fb.gguf_tensor(path, "blk.9.ffn_gate_inp.weight") is None
    assert _ref_read(ref, path, "blk.9.ffn_gate_inp.weight", 4) is None


def test_reader_rejects_what_is_not_gguf(fb, tmp_path):
    p = tmp_path / "junk.gguf"
    p.write_bytes(b"GGUF" + bytes(60))                     # right magic, version 0
    assert fb.gguf_tensor(p, "x") is None
    p.write_bytes(b"QMOE" + bytes(60))
    assert fb.gguf_tensor(p, "x") is None
    assert fb.gguf_tensor(tmp_path / "absent.gguf", "x") is None
    H.write_gguf(p, [("k", 8, "v")], [("t", [32], 0, np.arange(32, dtype=np.float32).tobytes())])
    data = p.read_bytes()
    p.write_bytes(data[:-64])                               # directory intact, tensor data cut short
    t = fb.gguf_tensor(p, "t", read=False)
    assert t is not None and t[0] == 0 and t[1][0] == 32
    assert fb.gguf_tensor(p, "t") is None


@pytest.mark.gpu
@pytest.mark.parametrize("router_type,gate_type", [(0, H.Q4), (1, H.Q4), (30, H.Q6)])
def test_load_gguf_into_the_table(fb, oracle, tmp_path, router_type, gate_type):
    n_layers, n_embd, inter, n_experts, top_k, seed, first = 2, 512, 256, 8, 2, 23, 5
    dts = [H.Q6, H.Q4]
    path = tmp_path / "moe.gguf"
    H.moe_gguf(fb, path, seed, n_layers, n_embd, inter, n_experts, dts, first_block=first, gate_type=gate_type,
               router_type=router_type)
    d = fb.MoeDecoder(n_layers, n_embd, inter, n_experts, top_k, True, dts, gate_type=gate_type)
    d.generate(seed + 1)                                    # something else first: every byte must be replaced
    assert d.load_gguf(path, first) == n_layers
    gs = fb.matrix_bytes(gate_type, inter, n_embd)
    for l in range(n_layers):
        for e in (0, n_experts - 1, n_experts):             # two routed experts and the shared one
            rec = H.expert_record(fb, seed, l, e, dts[l], n_embd, inter, gate_type)
            assert (d.export_shard(l, e, fb.M_GATE) == rec[:gs]).all()
            assert (d.export_shard(l, e, fb.M_UP) == rec[gs:2 * gs]).all()
            assert (d.export_shard(l, e, fb.M_DOWN) == rec[2 * gs:]).all()
    h = H.hidden(fb, seed, 0, n_embd)
    w = H.router_weights(fb, seed, 0, n_experts, n_embd)
    if router_type == 1:
        w = w.astype(np.float16).astype(np.float32)
    elif router_type == 30:
        w = ((w.view(np.uint32) >> 16) << 16).view(np.float32)
    got = d.moe_layer(0, h)
    want = H.oracle_layer(oracle, fb, seed, 0, h, n_embd, inter, n_experts, top_k, dts[0], router=w, gate_type=gate_type)
    assert (got["ids"] == want["ids"]).all()
    assert H.rel_l2(got["out"], want["out"]) < 3e-4
    # the norm weight arrived too: a stack step with the file's norm equals the oracle's
    d.upload_glue(0, resid=H.glue(fb, seed, 0, n_embd)[0])   # the residual stand-in is not part of a model file
    x = d.stack_run(h, 0, 1)
    d2 = fb.MoeDecoder(n_layers, n_embd, inter, n_experts, top_k, True, dts, gate_type=gate_type)
    d2.generate(seed)
    d2.upload_router(0, w)
    assert (H.bits(d2.stack_run(h, 0, 1)) == H.bits(x)).all()
    # a file of another shape is refused as a whole
    H.moe_gguf(fb, tmp_path / "other.gguf", seed, 1, n_embd, inter, n_experts + 1, dts, first_block=0, gate_type=gate_type)
    with pytest.raises(RuntimeError):
        d.load_gguf(tmp_path / "other.gguf", 0)
    d.close()
    d2.close()
