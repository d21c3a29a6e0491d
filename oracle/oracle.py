"""ctypes loaders for the two CPU checkers (TEST INFRASTRUCTURE ONLY).

``Oracle``  wraps oracle/libfomoe_oracle.so, this repo's scalar C restatement of
            fomoe's routed-expert FFN decode arithmetic (oracle/fomoe_oracle.c).
``Ref``     wraps oracle/_ref/libfomoe_ref.so, the reference's own C files compiled
            unmodified plus the glue in oracle/ref_driver.c.  ``Ref.available()`` is
            False when that library was not built.

Only tests, the smoke check and the benchmark's CPU-baseline leg import this module;
the product package never does.
"""
import ctypes as C
import os
import subprocess

import numpy as np

_HERE = os.path.dirname(os.path.abspath(__file__))
ORACLE_SO = os.path.join(_HERE, "libfomoe_oracle.so")
REF_SO = os.path.join(_HERE, "_ref", "libfomoe_ref.so")

TYPE_F32, TYPE_Q4_K, TYPE_Q5_K, TYPE_Q6_K = 0, 12, 13, 14
TYPE_Q8_0, TYPE_MXFP4 = 8, 39
QK_K = 256
Q4K_BLOCK, Q5K_BLOCK, Q6K_BLOCK, Q8K_BLOCK = 144, 176, 210, 292

_f32p = C.POINTER(C.c_float)
_i32p = C.POINTER(C.c_int)
_u32p = C.POINTER(C.c_uint32)


def build(force=False):
    """Compile the oracle (and the reference library when its sources are present)."""
    if force or not os.path.exists(ORACLE_SO) or (
        os.path.getmtime(ORACLE_SO) < os.path.getmtime(os.path.join(_HERE, "fomoe_oracle.c"))
    ) or (not os.path.exists(REF_SO) and os.path.isdir(os.environ.get("FOMOE_REF", "/root/reference"))):
        subprocess.run(["make", "-s", "-C", _HERE], check=True)


def row_bytes(qtype, k):
    if qtype in (TYPE_Q8_0, TYPE_MXFP4):
        return (k // 32) * (34 if qtype == TYPE_Q8_0 else 17)
    return (k // QK_K) * {TYPE_Q4_K: Q4K_BLOCK, TYPE_Q5_K: Q5K_BLOCK, TYPE_Q6_K: Q6K_BLOCK}[qtype]


def _fp(a):
    return a.ctypes.data_as(_f32p)


def _vp(a):
    return a.ctypes.data_as(C.c_void_p)


def _f32(a):
    return np.ascontiguousarray(a, dtype=np.float32)


def _u8(a):
    a = np.ascontiguousarray(a)
    return a.view(np.uint8).reshape(-1)


class _Common:
    """Operations both libraries offer, under a per-library symbol prefix map."""

    def __init__(self, lib, names):
        self.lib = lib
        self.n = names
        g = lambda k: getattr(lib, names[k])
        g("dq4").argtypes = [C.c_void_p, _f32p, C.c_int64]
        g("dq4").restype = None
        g("dq6").argtypes = [C.c_void_p, _f32p, C.c_int64]
        g("dq6").restype = None
        g("dq5").argtypes = [C.c_void_p, _f32p, C.c_int64]
        g("dq5").restype = None
        g("dot5").argtypes = [C.c_void_p, C.c_void_p, C.c_int]
        g("dot5").restype = C.c_float
        g("q8").argtypes = [_f32p, C.c_void_p, C.c_int64]
        g("q8").restype = None
        g("dot4").argtypes = [C.c_void_p, C.c_void_p, C.c_int]
        g("dot4").restype = C.c_float
        g("dot6").argtypes = [C.c_void_p, C.c_void_p, C.c_int]
        g("dot6").restype = C.c_float
        g("fp16").argtypes = [C.c_uint16]
        g("fp16").restype = C.c_float
        g("softmax").argtypes = [_f32p, C.c_int64]
        g("softmax").restype = None
        g("topk").argtypes = [_f32p, C.c_int64, C.c_int, _i32p, _f32p]
        g("topk").restype = None
        g("rms").argtypes = [_f32p, _f32p, _f32p, C.c_int64, C.c_float]
        g("rms").restype = None
        g("route").argtypes = [_f32p, _f32p, C.c_int, C.c_int, C.c_int, C.c_void_p, C.c_float, C.c_int,
                               _f32p, _i32p, _f32p]
        g("route").restype = C.c_int
        g("moe").argtypes = [_f32p, _f32p, C.POINTER(C.c_void_p), _f32p, C.c_int, C.c_void_p, C.c_int,
                             C.c_int, C.c_int, C.c_uint64, C.c_uint64, C.c_int, C.c_int]
        g("moe").restype = None
        g("moe_f32").argtypes = g("moe").argtypes
        g("moe_f32").restype = None

    def _f(self, k):
        return getattr(self.lib, self.n[k])

    def fp16_to_fp32(self, h):
        return np.float32(self._f("fp16")(int(h)))

    def dequantize(self, blocks, qtype, k):
        """blocks: bytes of k/256 blocks -> float32[k]."""
        b = _u8(blocks)
        assert b.size == row_bytes(qtype, k)
        y = np.empty(k, dtype=np.float32)
        self._f({TYPE_Q4_K: "dq4", TYPE_Q5_K: "dq5", TYPE_Q6_K: "dq6"}[qtype])(_vp(b), _fp(y), k)
        return y

    def quantize_q8k(self, x):
        """float32[k] -> uint8[(k/256)*292] holding block_q8_K records."""
        x = _f32(x)
        out = np.zeros((x.size // QK_K) * Q8K_BLOCK, dtype=np.uint8)
        self._f("q8")(_fp(x), _vp(out), x.size)
        return out

    def vec_dot(self, row_blocks, qtype, q8, nb):
        b = _u8(row_blocks)
        q = _u8(q8)
        return np.float32(self._f({TYPE_Q4_K: "dot4", TYPE_Q5_K: "dot5", TYPE_Q6_K: "dot6"}[qtype])(_vp(b), _vp(q), nb))

    def matvec_q8(self, mat, qtype, x, M, K):
        """out[M] = mat[M x K] (quantised rows) . Q8_K(x)."""
        q8 = self.quantize_q8k(x)
        m = _u8(mat)
        rb = row_bytes(qtype, K)
        out = np.empty(M, dtype=np.float32)
        for i in range(M):
            out[i] = self.vec_dot(m[i * rb:(i + 1) * rb], qtype, q8, K // QK_K)
        return out

    def softmax(self, x):
        x = _f32(x).copy()
        self._f("softmax")(_fp(x), x.size)
        return x

    def top_k(self, x, k):
        x = _f32(x)
        ids = np.empty(k, dtype=np.int32)
        vals = np.empty(k, dtype=np.float32)
        self._f("topk")(_fp(x), x.size, k, ids.ctypes.data_as(_i32p), _fp(vals))
        return ids, vals

    def rms_norm(self, x, w, eps):
        x, w = _f32(x), _f32(w)
        out = np.empty_like(x)
        self._f("rms")(_fp(out), _fp(x), _fp(w), x.size, C.c_float(eps))
        return out

    def route(self, router_w, h, k, mask=None, threshold=1.0, dampen=False):
        """-> (ids int32[k], scores float32[k], all_scores float32[n_experts], n_subs)."""
        w, h = _f32(router_w), _f32(h)
        n_experts, n_embd = w.shape
        all_scores = np.empty(n_experts, dtype=np.float32)
        ids = np.empty(k, dtype=np.int32)
        scores = np.empty(k, dtype=np.float32)
        mp = None
        if mask is not None:
            mask = np.ascontiguousarray(mask, dtype=np.uint32)
            mp = _vp(mask)
        subs = self._f("route")(_fp(w), _fp(h), n_experts, n_embd, k, mp, C.c_float(threshold),
                                int(bool(dampen)), _fp(all_scores), ids.ctypes.data_as(_i32p), _fp(scores))
        return ids, scores, all_scores, subs

    def moe_block(self, h, experts, scores, shared, gate_type, up_type, down_type, gate_size, up_size,
                  n_embd, inter, act_f32=False):
        """experts: list of uint8 arrays (gate|up|down records); shared: uint8 array or None.
        act_f32: the reference's fp32-activation definition instead of the Q8_K one of cpu_expert.c."""
        h, scores = _f32(h), _f32(scores)
        keep = [_u8(e) for e in experts]
        ptrs = (C.c_void_p * len(keep))(*[e.ctypes.data for e in keep])
        sh = _u8(shared) if shared is not None else None
        out = np.empty(n_embd, dtype=np.float32)
        self._f("moe_f32" if act_f32 else "moe")(_fp(out), _fp(h), ptrs, _fp(scores), len(keep), _vp(sh) if sh is not None else None,
                       gate_type, up_type, down_type, gate_size, up_size, n_embd, inter)
        return out


class Oracle(_Common):
    def __init__(self):
        build()
        lib = C.CDLL(ORACLE_SO)
        super().__init__(lib, dict(dq4="orc_dequantize_row_q4_K", dq6="orc_dequantize_row_q6_K",
                                   dq5="orc_dequantize_row_q5_K", dot5="orc_vec_dot_q5_K_q8_K",
                                   q8="orc_quantize_row_q8_K", dot4="orc_vec_dot_q4_K_q8_K",
                                   dot6="orc_vec_dot_q6_K_q8_K", fp16="orc_fp16_to_fp32",
                                   softmax="orc_softmax", topk="orc_top_k", rms="orc_rms_norm",
                                   route="orc_route", moe="orc_moe_block", moe_f32="orc_moe_block_f32"))
        lib.orc_car.argtypes = [_i32p, _f32p, C.c_int, _f32p, C.c_int, C.c_void_p, C.c_float, C.c_int]
        lib.orc_car.restype = C.c_int
        lib.orc_router_logits.argtypes = [_f32p, _f32p, _f32p, C.c_int, C.c_int]
        lib.orc_router_logits.restype = None
        lib.orc_shared_gate.argtypes = [_f32p, _f32p, C.c_int]
        lib.orc_shared_gate.restype = C.c_float
        lib.orc_expert_ffn.argtypes = [_f32p, C.c_void_p, C.c_void_p, C.c_float, C.c_int, C.c_int, C.c_int,
                                       C.c_uint64, C.c_uint64, C.c_int, C.c_int, _f32p]
        lib.orc_expert_ffn.restype = None
        lib.orc_mat_vec_mul_f32act.argtypes = [_f32p, C.c_void_p, C.c_int, _f32p, C.c_int, C.c_int]
        lib.orc_mat_vec_mul_f32act.restype = None
        lib.orc_shared_ffn_f32.argtypes = [_f32p, _f32p, C.c_void_p, C.c_int, C.c_void_p, C.c_int, C.c_void_p, C.c_int,
                                           C.c_int, C.c_int]
        lib.orc_shared_ffn_f32.restype = None
        for nm in ("orc_dequantize_row_q8_0", "orc_dequantize_row_mxfp4"):
            getattr(lib, nm).argtypes = [C.c_void_p, _f32p, C.c_int64]
            getattr(lib, nm).restype = None

    def mat_vec_mul_f32act(self, mat, qtype, x, M, K):
        """The fp32-activation matvec of src/tensor.c:102-171 for every quantised type, Q8_0 and MXFP4 included."""
        m, x = _u8(mat), _f32(x)
        out = np.empty(M, dtype=np.float32)
        self.lib.orc_mat_vec_mul_f32act(_fp(out), _vp(m), qtype, _fp(x), M, K)
        return out

    def dequantize32(self, blocks, qtype, k):
        b = _u8(blocks)
        y = np.empty(k, dtype=np.float32)
        getattr(self.lib, "orc_dequantize_row_q8_0" if qtype == TYPE_Q8_0 else "orc_dequantize_row_mxfp4")(_vp(b), _fp(y), k)
        return y

    def shared_ffn_f32(self, h, gate, gate_type, up, up_type, down, down_type, n_embd, inter):
        """src/inference.c:361-374 on fp32 activations."""
        g, u, d = _u8(gate), _u8(up), _u8(down)
        out = np.empty(n_embd, dtype=np.float32)
        self.lib.orc_shared_ffn_f32(_fp(out), _fp(_f32(h)), _vp(g), gate_type, _vp(u), up_type, _vp(d), down_type, n_embd, inter)
        return out

    def shared_gate(self, h, w):
        h, w = _f32(h), _f32(w)
        return np.float32(self.lib.orc_shared_gate(_fp(h), _fp(w), h.size))

    def router_logits(self, w, h):
        w, h = _f32(w), _f32(h)
        out = np.empty(w.shape[0], dtype=np.float32)
        self.lib.orc_router_logits(_fp(out), _fp(w), _fp(h), w.shape[0], w.shape[1])
        return out

    def car(self, ids, scores, all_scores, mask, threshold, dampen):
        ids = np.ascontiguousarray(ids, dtype=np.int32).copy()
        scores = _f32(scores).copy()
        a = _f32(all_scores)
        m = np.ascontiguousarray(mask, dtype=np.uint32)
        subs = self.lib.orc_car(ids.ctypes.data_as(_i32p), _fp(scores), ids.size, _fp(a), a.size, _vp(m),
                                C.c_float(threshold), int(bool(dampen)))
        return ids, scores, subs

    def expert_act(self, expert, h, gate_type, up_type, down_type, gate_size, up_size, n_embd, inter):
        """silu(gate.h)*up.h for one expert (the down-projection input), float32[inter]."""
        q8 = self.quantize_q8k(h)
        e = _u8(expert)
        partial = np.zeros(n_embd, dtype=np.float32)
        act = np.empty(inter, dtype=np.float32)
        self.lib.orc_expert_ffn(_fp(partial), _vp(e), _vp(q8), C.c_float(1.0), gate_type, up_type, down_type,
                                gate_size, up_size, n_embd, inter, _fp(act))
        return act, partial


class Ref(_Common):
    @staticmethod
    def available():
        build()
        return os.path.exists(REF_SO)

    def __init__(self):
        build()
        lib = C.CDLL(REF_SO)
        super().__init__(lib, dict(dq4="dequantize_row_q4_K", dq6="dequantize_row_q6_K",
                                   dq5="dequantize_row_q5_K", dot5="vec_dot_q5_K_q8_K",
                                   q8="quantize_row_q8_K", dot4="vec_dot_q4_K_q8_K",
                                   dot6="vec_dot_q6_K_q8_K", fp16="fp16_to_fp32", softmax="softmax",
                                   topk="top_k", rms="rms_norm", route="refdrv_route",
                                   moe="refdrv_moe_block", moe_f32="refdrv_moe_block_f32"))
        lib.mat_vec_mul.argtypes = [_f32p, C.c_void_p, C.c_int, _f32p, C.c_int64, C.c_int64]
        lib.mat_vec_mul.restype = None
        lib.refdrv_car_case.argtypes = [C.c_float, C.c_int, _i32p, _f32p, C.c_int, _f32p, C.c_int, _i32p,
                                        C.c_int, _i32p, C.c_int, _i32p, _i32p, _i32p]
        lib.refdrv_car_case.restype = C.c_int
        lib.refdrv_max_threads.restype = C.c_int
        lib.refdrv_set_threads.argtypes = [C.c_int]
        lib.fp32_to_fp16.argtypes = [C.c_float]
        lib.fp32_to_fp16.restype = C.c_uint16
        for nm in ("dequantize_row_q8_0", "dequantize_row_mxfp4"):
            getattr(lib, nm).argtypes = [C.c_void_p, _f32p, C.c_int64]
            getattr(lib, nm).restype = None

    def dequantize32(self, blocks, qtype, k):
        b = _u8(blocks)
        y = np.empty(k, dtype=np.float32)
        getattr(self.lib, "dequantize_row_q8_0" if qtype == TYPE_Q8_0 else "dequantize_row_mxfp4")(_vp(b), _fp(y), k)
        return y

    def shared_ffn_f32(self, h, gate, gate_type, up, up_type, down, down_type, n_embd, inter):
        """The reference's shared_expert_ffn (src/inference.c:361-374) composed from its own mat_vec_mul: silu, multiply."""
        g = self.mat_vec_mul_f32act(gate, gate_type, h, inter, n_embd)
        self.lib.silu.argtypes = [_f32p, C.c_int64]
        self.lib.silu.restype = None
        self.lib.vec_mul.argtypes = [_f32p, _f32p, _f32p, C.c_int64]
        self.lib.vec_mul.restype = None
        self.lib.silu(_fp(g), inter)
        u = self.mat_vec_mul_f32act(up, up_type, h, inter, n_embd)
        self.lib.vec_mul(_fp(g), _fp(g), _fp(u), inter)
        return self.mat_vec_mul_f32act(down, down_type, g, n_embd, inter)

    def write_store(self, path, layers):
        """Write an expert store (.qmoe) with the reference's own writer.  layers: list of (down_type, records),
        records = list of uint8 arrays gate | up | down, gate and up of equal size."""
        n_layers, n_experts = len(layers), len(layers[0][1])
        keep = [_u8(r) for _, recs in layers for r in recs]
        ptrs = (C.c_void_p * len(keep))(*[k.ctypes.data for k in keep])
        down_types = (C.c_uint32 * n_layers)(*[int(t) for t, _ in layers])
        gate = None
        downs = []
        for t, recs in layers:
            blk = {TYPE_Q4_K: Q4K_BLOCK, TYPE_Q5_K: Q5K_BLOCK, TYPE_Q6_K: Q6K_BLOCK}[t]
            # gate/up are Q4_K [inter x n_embd], down is [n_embd x inter]: same element count, other block size
            n = _u8(recs[0]).size
            g = n * Q4K_BLOCK // (2 * Q4K_BLOCK + blk)
            gate = g
            downs.append(n - 2 * g)
        down_sizes = (C.c_uint64 * n_layers)(*downs)
        self.lib.refdrv_write_store.argtypes = [C.c_char_p, C.c_int, C.c_int, C.c_uint64, C.c_uint64, C.c_void_p,
                                                C.c_void_p, C.c_void_p]
        self.lib.refdrv_write_store.restype = C.c_int
        rc = self.lib.refdrv_write_store(path.encode(), n_layers, n_experts, gate, gate, down_sizes, down_types, ptrs)
        if rc != 0:
            raise RuntimeError("reference expert_store writer failed")

    def max_threads(self):
        return int(self.lib.refdrv_max_threads())

    def set_threads(self, n):
        self.lib.refdrv_set_threads(int(n))

    def fp32_to_fp16(self, f):
        return int(self.lib.fp32_to_fp16(C.c_float(f)))

    def router_logits(self, w, h):
        w, h = _f32(w), _f32(h)
        out = np.empty(w.shape[0], dtype=np.float32)
        self.lib.mat_vec_mul(_fp(out), _vp(w), TYPE_F32, _fp(h), w.shape[0], w.shape[1])
        return out

    def mat_vec_mul_f32act(self, mat, qtype, x, M, K):
        """The reference's fp32-activation matvec (src/tensor.c:102-127)."""
        m, x = _u8(mat), _f32(x)
        out = np.empty(M, dtype=np.float32)
        self.lib.mat_vec_mul(_fp(out), _vp(m), qtype, _fp(x), M, K)
        return out

    def car_case(self, threshold, dampen, ids, scores, all_scores, vram_ids, ram_ids):
        ids = np.ascontiguousarray(ids, dtype=np.int32).copy()
        scores = _f32(scores).copy()
        a = _f32(all_scores)
        v = np.ascontiguousarray(vram_ids, dtype=np.int32)
        r = np.ascontiguousarray(ram_ids, dtype=np.int32)
        n_unc = C.c_int(0)
        nv = C.c_int(0)
        vsi = np.zeros(16, dtype=np.int32)
        ip = lambda z: z.ctypes.data_as(_i32p)
        subs = self.lib.refdrv_car_case(C.c_float(threshold), int(bool(dampen)), ip(ids), _fp(scores), ids.size,
                                        _fp(a), a.size, ip(v), v.size, ip(r), r.size, C.byref(n_unc), ip(vsi),
                                        C.byref(nv))
        return dict(subs=subs, ids=ids, scores=scores, n_uncached=n_unc.value,
                    vram_sub_indices=vsi[:nv.value].copy())
