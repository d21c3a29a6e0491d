"""fomoe_b200 -- fomoe's routed-expert FFN decode path, native on B200.

This package is a thin ctypes mirror of ``include/fomoe_b200.h``; all work happens in
``libfomoe_b200.so`` (hand-written CUDA for sm_100a behind a C host library).  There is no
Python or CPU implementation of the path: if the shared library is missing or no CUDA
device is present, construction fails loudly.

The three classes follow the three groups of the C ABI:

* :class:`GpuOperator`   -- the reference's ``gpu.h`` surface (``gpu_init`` / ``gpu_expert_ffn``)
* :class:`ExpertEngine`  -- CUDA twin of the reference's ``cpu_expert.h`` engine
* :class:`MoeDecoder`    -- resident expert table + on-device routing + decode stack
"""
import ctypes as C
import os

import numpy as np

_HERE = os.path.dirname(os.path.abspath(__file__))
LIB_PATH = os.environ.get("FOMOE_B200_LIB") or os.path.join(_HERE, "libfomoe_b200.so")  # override: a differently built library

TYPE_Q4_K, TYPE_Q5_K, TYPE_Q6_K = 12, 13, 14
STREAM_ROUTER, STREAM_RESID, STREAM_NORMW, STREAM_HIDDEN = 3, 4, 5, 6
M_GATE, M_UP, M_DOWN = 0, 1, 2
TYPE_Q8_0, TYPE_MXFP4 = 8, 39
ROUTER_STD, RESID_STD, NORMW_MEAN, NORMW_STD = 0.02, 1.0, 1.0, 0.1
BLOCK_BYTES = {TYPE_Q4_K: 144, TYPE_Q5_K: 176, TYPE_Q6_K: 210}

_f32p = C.POINTER(C.c_float)
_i32p = C.POINTER(C.c_int)


class Config(C.Structure):
    _fields_ = [("device", C.c_int), ("n_layers", C.c_int), ("n_embd", C.c_int), ("n_inter", C.c_int),
                ("n_experts", C.c_int), ("top_k", C.c_int), ("has_shared", C.c_int), ("gate_type", C.c_int),
                ("down_types", _i32p), ("tp_rank", C.c_int), ("tp_size", C.c_int), ("rms_eps", C.c_float),
                ("car_threshold", C.c_float), ("car_dampen", C.c_int), ("max_tokens", C.c_int)]


class BatchConfig(C.Structure):
    _fields_ = [("device", C.c_int), ("n_layers", C.c_int), ("n_embd", C.c_int), ("n_inter", C.c_int),
                ("n_experts", C.c_int), ("top_k", C.c_int), ("has_shared", C.c_int), ("max_tokens", C.c_int),
                ("rms_eps", C.c_float), ("tp_rank", C.c_int), ("tp_size", C.c_int)]


class Work(C.Structure):
    _fields_ = [("expert_data", C.c_void_p), ("score", C.c_float), ("gate_type", C.c_int), ("up_type", C.c_int),
                ("down_type", C.c_int), ("expert_gate_size", C.c_uint64), ("expert_up_size", C.c_uint64)]


# name -> (restype, argtypes); every symbol include/fomoe_b200.h declares
_SIGS = {
    "gpu_init": (C.c_void_p, []),
    "gpu_free": (None, [C.c_void_p]),
    "gpu_register_buffers": (None, [C.c_void_p, C.POINTER(C.c_void_p), C.c_int, C.c_uint64]),
    "gpu_unregister_buffers": (None, [C.c_void_p, C.POINTER(C.c_void_p), C.c_int]),
    "gpu_upload_model": (C.c_int, [C.c_void_p, C.c_void_p]),
    "gpu_set_ram_cache_mb": (None, [C.c_void_p, C.c_int]),
    "gpu_set_vram_cache_mb": (None, [C.c_void_p, C.c_int]),
    "gpu_forward": (C.c_void_p, [C.c_void_p, C.c_void_p, C.c_int, C.c_int]),
    "gpu_reset_state": (None, [C.c_void_p]),
    "gpu_seed_vram_cache": (C.c_int, [C.c_void_p, C.c_void_p, C.c_char_p]),
    "gpu_enable_expert_freq": (None, [C.c_void_p]),
    "gpu_get_expert_freq": (C.c_void_p, [C.c_void_p]),
    "gpu_get_expert_dims": (None, [C.c_void_p, _i32p, _i32p]),
    "gpu_get_pingpong_relay_stats": (None, [C.c_void_p] + [C.POINTER(C.c_uint64)] * 5),
    "gpu_expert_ffn": (C.c_int, [C.c_void_p, _f32p, C.POINTER(C.c_void_p), _f32p, C.c_int, C.c_int, C.c_int,
                                 C.c_uint64, C.c_uint64, C.c_uint64, C.c_int, C.c_int, C.c_int, _f32p]),
    "b200_expert_create": (C.c_void_p, [C.c_int, C.c_int]),
    "b200_expert_free": (None, [C.c_void_p]),
    "b200_expert_reset": (None, [C.c_void_p]),
    "b200_expert_ffn": (None, [C.c_void_p, C.c_void_p, _f32p, C.c_float, C.c_int, C.c_int, C.c_int, C.c_uint64,
                               C.c_uint64]),
    "b200_expert_submit_async": (None, [C.c_void_p, _f32p, C.POINTER(Work), C.c_int]),
    "b200_expert_wait": (None, [C.c_void_p]),
    "b200_expert_result": (_f32p, [C.c_void_p]),
    "b200_expert_get_timing": (None, [C.c_void_p, C.POINTER(C.c_double), C.POINTER(C.c_double), _i32p]),
    "fomoe_b200_create": (C.c_void_p, [C.POINTER(Config)]),
    "fomoe_b200_destroy": (None, [C.c_void_p]),
    "fomoe_b200_last_error": (C.c_char_p, [C.c_void_p]),
    "fomoe_b200_status": (C.c_int, [C.c_void_p]),
    "fomoe_b200_proj_matvec_f32": (C.c_int, [C.c_void_p, C.c_int, C.c_void_p, C.c_int, C.c_int, _f32p, _f32p]),
    "fomoe_b200_shared_ffn_f32": (C.c_int, [C.c_void_p, C.c_void_p, C.c_int, C.c_void_p, C.c_int, C.c_void_p, C.c_int,
                                            C.c_int, C.c_int, _f32p, _f32p]),
    "fomoe_b200_get_config": (C.c_void_p, [C.c_void_p]),
    "fomoe_b200_load_gguf": (C.c_int, [C.c_void_p, C.c_char_p, C.c_int]),
    "fomoe_b200_gguf_tensor": (C.c_int, [C.c_char_p, C.c_char_p, _i32p, C.POINTER(C.c_int64), C.POINTER(C.c_uint64),
                                         C.c_void_p, C.c_uint64]),
    "fomoe_b200_batch_set_allreduce": (C.c_int, [C.c_void_p, C.c_void_p, C.c_void_p]),
    "fomoe_b200_record_bytes": (C.c_uint64, [C.c_void_p, C.c_int]),
    "fomoe_b200_table_bytes": (C.c_uint64, [C.c_void_p]),
    "fomoe_b200_table_generate": (C.c_int, [C.c_void_p, C.c_uint64]),
    "fomoe_b200_table_upload": (C.c_int, [C.c_void_p, C.c_int, C.c_int, C.c_void_p]),
    "fomoe_b200_table_export": (C.c_int, [C.c_void_p, C.c_int, C.c_int, C.c_int, C.c_void_p]),
    "fomoe_b200_table_dequant": (C.c_int, [C.c_void_p, C.c_int, C.c_int, C.c_int, _f32p]),
    "fomoe_b200_router_upload": (C.c_int, [C.c_void_p, C.c_int, _f32p]),
    "fomoe_b200_glue_upload": (C.c_int, [C.c_void_p, C.c_int, _f32p, _f32p]),
    "fomoe_b200_set_resident_mask": (C.c_int, [C.c_void_p, C.c_int, C.c_void_p]),
    "fomoe_b200_shared_gate_upload": (C.c_int, [C.c_void_p, C.c_int, C.c_void_p]),
    "fomoe_b200_table_load_qmoe": (C.c_int, [C.c_void_p, C.c_char_p, C.c_int]),
    "fomoe_b200_set_allreduce": (C.c_int, [C.c_void_p, C.c_void_p, C.c_void_p]),
    "fomoe_b200_tp_recv_ptr": (C.c_void_p, [C.c_void_p]),
    "fomoe_b200_tp_connect_ptrs": (C.c_int, [C.c_void_p, C.c_void_p]),
    "fomoe_b200_set_wait_limit": (C.c_int, [C.c_void_p, C.c_uint]),
    "fomoe_b200_tp_enable_peer": (C.c_int, [C.c_void_p, C.c_int]),
    "fomoe_b200_tp_inject": (C.c_int, [C.c_void_p, C.c_int, C.c_void_p, C.c_uint]),
    "fomoe_b200_routing_trace_open": (C.c_int, [C.c_void_p, C.c_char_p]),
    "fomoe_b200_routing_trace_close": (C.c_int, [C.c_void_p]),
    "fomoe_b200_enable_expert_freq": (C.c_int, [C.c_void_p]),
    "fomoe_b200_get_expert_freq": (C.c_int, [C.c_void_p, C.POINTER(C.c_uint32)]),
    "fomoe_b200_gpu_attach": (C.c_int, [C.c_void_p, C.c_void_p]),
    "fomoe_b200_set_act_mode": (C.c_int, [C.c_void_p, C.c_int]),
    "fomoe_b200_stream": (C.c_void_p, [C.c_void_p]),
    "fomoe_b200_set_car": (C.c_int, [C.c_void_p, C.c_float, C.c_int]),
    "fomoe_b200_moe_layer": (C.c_int, [C.c_void_p, C.c_int, _f32p, _f32p, _i32p, _f32p, _i32p, _f32p]),
    "fomoe_b200_moe_layer_routed": (C.c_int, [C.c_void_p, C.c_int, _f32p, _i32p, _f32p, C.c_int, _f32p]),
    "fomoe_b200_stack_run": (C.c_int, [C.c_void_p, _f32p, C.c_int, C.c_int, _f32p]),
    "fomoe_b200_tokens_upload": (C.c_int, [C.c_void_p, C.c_int, C.c_int, _f32p]),
    "fomoe_b200_tokens_run": (C.c_int, [C.c_void_p, C.c_int, C.c_int, _f32p]),
    "fomoe_b200_tokens_download": (C.c_int, [C.c_void_p, C.c_int, C.c_int, _f32p]),
    "fomoe_b200_decode_token": (C.c_int, [C.c_void_p, _f32p, _f32p]),
    "fomoe_b200_tokens_profile": (C.c_int, [C.c_void_p, C.c_int, C.c_int, _f32p, _i32p]),
    "fomoe_b200_get_routing": (C.c_int, [C.c_void_p, C.c_int, _i32p, _f32p, _i32p]),
    "fomoe_b200_substitutions": (C.c_uint64, [C.c_void_p]),
    "fomoe_b200_kernel_launches": (C.c_uint64, [C.c_void_p]),
    "fomoe_b200_set_graphs": (C.c_int, [C.c_void_p, C.c_int]),
    "fomoe_b200_set_variant": (C.c_int, [C.c_void_p, C.c_int]),
    "fomoe_b200_tp_export": (C.c_int, [C.c_void_p, C.c_void_p]),
    "fomoe_b200_tp_connect": (C.c_int, [C.c_void_p, C.c_void_p]),
    "fomoe_b200_trace_enable": (C.c_int, [C.c_void_p, C.c_int, C.c_int]),
    "fomoe_b200_trace_read": (C.c_int, [C.c_void_p, C.POINTER(C.c_uint64), C.c_int]),
    "fomoe_b200_peek": (C.c_int, [C.c_void_p, C.c_int, C.c_void_p, C.c_uint64]),
    "fomoe_b200_matvec": (C.c_int, [C.c_void_p, C.c_int, C.c_void_p, C.c_int, C.c_int, _f32p, _f32p]),
    "fomoe_b200_matvec_noalloc": (C.c_int, [C.c_int, C.c_void_p, C.c_int, C.c_int, C.c_void_p, C.c_void_p, C.c_void_p]),
    "fomoe_b200_quantize_q8k": (C.c_int, [C.c_void_p, _f32p, C.c_int, C.c_void_p]),
    "fomoe_b200_batch_create": (C.c_void_p, [C.POINTER(BatchConfig)]),
    "fomoe_b200_batch_destroy": (None, [C.c_void_p]),
    "fomoe_b200_batch_last_error": (C.c_char_p, [C.c_void_p]),
    "fomoe_b200_batch_status": (C.c_int, [C.c_void_p]),
    "fomoe_b200_batch_table_bytes": (C.c_uint64, [C.c_void_p]),
    "fomoe_b200_batch_kernel_launches": (C.c_uint64, [C.c_void_p]),
    "fomoe_b200_batch_generate": (C.c_int, [C.c_void_p, C.c_uint64, C.c_int]),
    "fomoe_b200_batch_upload": (C.c_int, [C.c_void_p, C.c_int, C.c_int, C.c_void_p]),
    "fomoe_b200_batch_export": (C.c_int, [C.c_void_p, C.c_int, C.c_int, C.c_void_p]),
    "fomoe_b200_batch_moe_layer": (C.c_int, [C.c_void_p, C.c_int, C.c_int, _f32p, _f32p, _f32p, _i32p, _f32p]),
    "fomoe_b200_batch_tokens_upload": (C.c_int, [C.c_void_p, C.c_int, _f32p]),
    "fomoe_b200_batch_stack_run": (C.c_int, [C.c_void_p, C.c_int, C.c_int, C.c_int, _f32p]),
    "fomoe_b200_batch_tokens_download": (C.c_int, [C.c_void_p, C.c_int, _f32p]),
    "fomoe_b200_batch_get_routing": (C.c_int, [C.c_void_p, C.c_int, _i32p, _f32p, _i32p]),
    "fomoe_b200_batch_wait_profile": (C.c_int, [C.c_void_p, C.c_int, C.POINTER(C.c_uint64)]),
    "fomoe_b200_batch_synth_logits": (None, [C.c_uint64, C.c_int, C.c_int, C.c_int, C.c_int, _f32p]),
    "fomoe_b200_synth_matrix": (None, [C.c_uint64, C.c_int, C.c_int, C.c_int, C.c_int, C.c_int, C.c_int, C.c_void_p]),
    "fomoe_b200_synth_f32": (None, [C.c_uint64, C.c_int, C.c_int, C.c_float, C.c_float, C.c_uint64, _f32p]),
}

_lib = None


def lib():
    """Load libfomoe_b200.so (built by ``__graft_entry__.build()`` / ``make -C fomoe_b200/csrc``)."""
    global _lib
    if _lib is None:
        if not os.path.exists(LIB_PATH):
            raise ImportError(f"{LIB_PATH} is missing: build it with `make -C fomoe_b200/csrc` "
                              "(there is no fallback implementation)")
        l = C.CDLL(LIB_PATH)
        for name, (res, args) in _SIGS.items():
            f = getattr(l, name)
            f.restype = res
            f.argtypes = args
        _lib = l
    return _lib


def exported_symbols():
    return sorted(_SIGS)


def _f32(a):
    return np.ascontiguousarray(a, dtype=np.float32)


def _fp(a):
    return a.ctypes.data_as(_f32p)


def _ip(a):
    return a.ctypes.data_as(_i32p)


def matrix_bytes(qtype, rows, cols):
    return rows * (cols // 256) * BLOCK_BYTES[qtype]


def synth_matrix(seed, layer, expert, matrix, qtype, rows, cols):
    """Host-side synthetic generator: ggml-ordered bytes of one expert matrix."""
    out = np.empty(matrix_bytes(qtype, rows, cols), dtype=np.uint8)
    lib().fomoe_b200_synth_matrix(seed, layer, expert, matrix, qtype, rows, cols, out.ctypes.data)
    return out


def synth_f32(seed, layer, stream_id, mean, std, n):
    out = np.empty(n, dtype=np.float32)
    lib().fomoe_b200_synth_f32(seed, layer, stream_id, mean, std, n, _fp(out))
    return out


# ---- the seeded synthetic inputs of the benchmark configurations, as the table generator on the device makes them
def synth_hidden(seed, token, n_embd):
    """Input hidden state of token `token`: N(0, 1)."""
    return synth_f32(seed, token, STREAM_HIDDEN, 0.0, 1.0, n_embd)


def synth_router(seed, layer, n_experts, n_embd):
    """fp32 router of a layer: N(0, 0.02), [n_experts, n_embd]."""
    return synth_f32(seed, layer, STREAM_ROUTER, 0.0, ROUTER_STD, n_experts * n_embd).reshape(n_experts, n_embd)


def synth_glue(seed, layer, n_embd):
    """(residual vector, RMSNorm weight) of a layer of the decode stack."""
    return (synth_f32(seed, layer, STREAM_RESID, 0.0, RESID_STD, n_embd),
            synth_f32(seed, layer, STREAM_NORMW, NORMW_MEAN, NORMW_STD, n_embd))


def synth_expert_record(seed, layer, expert, down_type, n_embd, inter, gate_type=TYPE_Q4_K):
    """One expert in the reference's record order (include/expert_store.h:9-40): gate | up | down, ggml bytes."""
    return np.concatenate([synth_matrix(seed, layer, expert, M_GATE, gate_type, inter, n_embd),
                           synth_matrix(seed, layer, expert, M_UP, gate_type, inter, n_embd),
                           synth_matrix(seed, layer, expert, M_DOWN, down_type, n_embd, inter)])


def gguf_tensor(path, name, read=True):
    """(ggml type, dims fastest-first, bytes or None) of one tensor of a GGUF file, by the library's own reader; None
    when the tensor is not there."""
    t, nb = C.c_int(0), C.c_uint64(0)
    dims = (C.c_int64 * 4)()
    if lib().fomoe_b200_gguf_tensor(str(path).encode(), name.encode(), C.byref(t), dims, C.byref(nb), None, 0):
        return None
    data = None
    if read and nb.value:
        data = np.empty(nb.value, dtype=np.uint8)
        if lib().fomoe_b200_gguf_tensor(str(path).encode(), name.encode(), None, None, None, data.ctypes.data, nb.value):
            return None
    return t.value, [int(d) for d in dims], data


class MoeDecoder:
    """Resident expert table + router/CAR + SwiGLU experts + decode stack on one GPU (one TP rank)."""

    def __init__(self, n_layers, n_embd=4096, n_inter=1024, n_experts=512, top_k=10, has_shared=True,
                 down_types=None, device=0, tp_rank=0, tp_size=1, rms_eps=1e-6, car_threshold=1.0,
                 car_dampen=False, max_tokens=1, gate_type=TYPE_Q4_K):
        self._l = lib()
        self.n_layers, self.n_embd, self.n_inter = n_layers, n_embd, n_inter
        self.gate_type = gate_type
        self.n_experts, self.top_k, self.has_shared = n_experts, top_k, bool(has_shared)
        self.tp_rank, self.tp_size, self.device = tp_rank, tp_size, device
        self.down_types = list(down_types) if down_types is not None else [TYPE_Q6_K] * n_layers
        self._dt = (C.c_int * n_layers)(*self.down_types)
        cfg = Config(device, n_layers, n_embd, n_inter, n_experts, top_k, int(bool(has_shared)), gate_type,
                     C.cast(self._dt, _i32p), tp_rank, tp_size, rms_eps, car_threshold, int(bool(car_dampen)),
                     max_tokens)
        self._h = self._l.fomoe_b200_create(C.byref(cfg))
        if not self._h:
            raise RuntimeError("fomoe_b200_create failed (no CUDA device, unsupported shape or out of memory)")

    def close(self):
        if getattr(self, "_h", None):
            self._l.fomoe_b200_destroy(self._h)
            self._h = None

    __del__ = close

    def _ck(self, rc, what):
        if rc != 0:
            raise RuntimeError(f"{what}: {self._l.fomoe_b200_last_error(self._h).decode()}")

    # ---- table
    def record_bytes(self, layer):
        return int(self._l.fomoe_b200_record_bytes(self._h, layer))

    def table_bytes(self):
        return int(self._l.fomoe_b200_table_bytes(self._h))

    def generate(self, seed):
        self._ck(self._l.fomoe_b200_table_generate(self._h, seed), "table_generate")

    def upload_expert(self, layer, expert, record):
        r = np.ascontiguousarray(record).view(np.uint8).reshape(-1)
        assert r.size == self.record_bytes(layer), (r.size, self.record_bytes(layer))
        self._ck(self._l.fomoe_b200_table_upload(self._h, layer, expert, r.ctypes.data), "table_upload")

    def load_gguf(self, path, first_block=0):
        """Router, experts, shared expert and norm weight of every layer from a GGUF model file; layers loaded."""
        n = self._l.fomoe_b200_load_gguf(self._h, str(path).encode(), first_block)
        if n < 0:
            raise RuntimeError("load_gguf failed (see stderr)")
        return n

    def proj_matvec_f32(self, qtype, w, rows, cols, x):
        """y = W x on fp32 activations, W in 32-value blocks (TYPE_Q8_0 / TYPE_MXFP4), ggml order."""
        w = np.ascontiguousarray(w).view(np.uint8).reshape(-1)
        y = np.empty(rows, dtype=np.float32)
        self._ck(self._l.fomoe_b200_proj_matvec_f32(self._h, qtype, w.ctypes.data, rows, cols, _fp(_f32(x)), _fp(y)),
                 "proj_matvec_f32")
        return y

    def shared_ffn_f32(self, h, gate, gate_type, up, up_type, down, down_type, n_embd, inter):
        """The reference's shared_expert_ffn (src/inference.c:361-374) for Q8_0 / MXFP4 projections."""
        g, u, d = (np.ascontiguousarray(a).view(np.uint8).reshape(-1) for a in (gate, up, down))
        out = np.empty(n_embd, dtype=np.float32)
        self._ck(self._l.fomoe_b200_shared_ffn_f32(self._h, g.ctypes.data, gate_type, u.ctypes.data, up_type, d.ctypes.data,
                                                   down_type, n_embd, inter, _fp(_f32(h)), _fp(out)), "shared_ffn_f32")
        return out

    @property
    def half_mode(self):
        """Twice as many ranks as 256-wide windows: two ranks share a window (see the C header)."""
        return self.tp_size == 2 * (self.n_inter // 256)

    def _shard_shape(self, layer, matrix):
        il = 256 if self.half_mode else self.n_inter // self.tp_size
        if matrix == M_DOWN:
            return self.down_types[layer], self.n_embd, 128 if self.half_mode else il
        return self.gate_type, il, self.n_embd

    def export_shard(self, layer, expert, matrix):
        """This rank's shard of one matrix, ggml block order, row-major over (rows, column blocks)."""
        t, rows, cols = self._shard_shape(layer, matrix)
        out = np.empty(matrix_bytes(t, rows, cols), dtype=np.uint8)
        self._ck(self._l.fomoe_b200_table_export(self._h, layer, expert, matrix, out.ctypes.data), "table_export")
        return out

    def dequant_shard(self, layer, expert, matrix):
        t, rows, cols = self._shard_shape(layer, matrix)
        out = np.empty((rows, cols), dtype=np.float32)
        self._ck(self._l.fomoe_b200_table_dequant(self._h, layer, expert, matrix, _fp(out)), "table_dequant")
        return out

    def upload_router(self, layer, w):
        w = _f32(w)
        assert w.shape == (self.n_experts, self.n_embd)
        self._ck(self._l.fomoe_b200_router_upload(self._h, layer, _fp(w)), "router_upload")

    def upload_glue(self, layer, resid=None, normw=None):
        r = _f32(resid) if resid is not None else None
        w = _f32(normw) if normw is not None else None
        self._ck(self._l.fomoe_b200_glue_upload(self._h, layer, _fp(r) if r is not None else None,
                                                _fp(w) if w is not None else None), "glue_upload")

    def load_qmoe(self, path, first_store_layer=0):
        """Fill the routed experts from an expert store file of the reference; returns the number loaded."""
        n = self._l.fomoe_b200_table_load_qmoe(self._h, path.encode(), first_store_layer)
        self._ck(0 if n >= 0 else -1, "table_load_qmoe")
        return n

    def set_act_mode(self, f32):
        """False: Q8_K int8 activations (src/cpu_expert.c, default); True: fp32 activations (the reference's
        forward pass without cpu_expert)."""
        self._ck(self._l.fomoe_b200_set_act_mode(self._h, 1 if f32 else 0), "set_act_mode")

    def set_shared_gate(self, layer, w):
        """w: float32[n_embd] (the shared expert's output is scaled by sigmoid(h . w)) or None (no gate)."""
        if w is None:
            self._ck(self._l.fomoe_b200_shared_gate_upload(self._h, layer, None), "shared_gate_upload")
            return
        w = _f32(w)
        assert w.size == self.n_embd
        self._ck(self._l.fomoe_b200_shared_gate_upload(self._h, layer, w.ctypes.data), "shared_gate_upload")

    def set_resident_mask(self, layer, mask):
        if mask is None:
            self._ck(self._l.fomoe_b200_set_resident_mask(self._h, layer, None), "set_resident_mask")
            return
        m = np.zeros(16, dtype=np.uint32)
        mm = np.ascontiguousarray(mask, dtype=np.uint32)
        m[:mm.size] = mm
        self._ck(self._l.fomoe_b200_set_resident_mask(self._h, layer, m.ctypes.data), "set_resident_mask")

    def set_car(self, threshold, dampen):
        self._ck(self._l.fomoe_b200_set_car(self._h, threshold, int(bool(dampen))), "set_car")

    # ---- compute
    def moe_layer(self, layer, h):
        """-> dict(out, ids, scores, ids_orig, all_scores)."""
        h = _f32(h)
        out = np.empty(self.n_embd, dtype=np.float32)
        ids = np.empty(self.top_k, dtype=np.int32)
        ids0 = np.empty(self.top_k, dtype=np.int32)
        sc = np.empty(self.top_k, dtype=np.float32)
        alls = np.empty(self.n_experts, dtype=np.float32)
        self._ck(self._l.fomoe_b200_moe_layer(self._h, layer, _fp(h), _fp(out), _ip(ids), _fp(sc), _ip(ids0),
                                              _fp(alls)), "moe_layer")
        return dict(out=out, ids=ids, scores=sc, ids_orig=ids0, all_scores=alls)

    def moe_layer_routed(self, layer, h, ids, scores):
        h, scores = _f32(h), _f32(scores)
        ids = np.ascontiguousarray(ids, dtype=np.int32)
        out = np.empty(self.n_embd, dtype=np.float32)
        self._ck(self._l.fomoe_b200_moe_layer_routed(self._h, layer, _fp(h), _ip(ids), _fp(scores), ids.size,
                                                     _fp(out)), "moe_layer_routed")
        return out

    def stack_run(self, x, l0=0, l1=None):
        x = _f32(x)
        out = np.empty_like(x)
        self._ck(self._l.fomoe_b200_stack_run(self._h, _fp(x), l0, self.n_layers if l1 is None else l1, _fp(out)),
                 "stack_run")
        return out

    def tokens_upload(self, first, x):
        x = _f32(x).reshape(-1, self.n_embd)
        self._ck(self._l.fomoe_b200_tokens_upload(self._h, first, x.shape[0], _fp(x)), "tokens_upload")

    def tokens_run(self, first, count):
        """Runs `count` resident tokens through every layer; returns CUDA-event milliseconds."""
        ms = C.c_float(0.0)
        self._ck(self._l.fomoe_b200_tokens_run(self._h, first, count, C.byref(ms)), "tokens_run")
        return float(ms.value)

    def decode_token(self, x):
        """One token host -> host through every layer: one pinned copy in, one launch of the stack kernel (which
        writes the result into pinned host memory), one synchronise."""
        x = _f32(x)
        out = np.empty_like(x)
        self._ck(self._l.fomoe_b200_decode_token(self._h, _fp(x), _fp(out)), "decode_token")
        return out

    def tokens_profile(self, first, count):
        """Plain launches with CUDA events around every kernel -> (ms, launches) per phase."""
        ms = np.zeros(5, dtype=np.float32)
        n = np.zeros(4, dtype=np.int32)
        self._ck(self._l.fomoe_b200_tokens_profile(self._h, first, count, _fp(ms), _ip(n)), "tokens_profile")
        names = ("prologue", "router", "gate_up", "down")
        return {k: (float(ms[i]), int(n[i])) for i, k in enumerate(names)}, float(ms[4])

    def tokens_download(self, first, count):
        out = np.empty((count, self.n_embd), dtype=np.float32)
        self._ck(self._l.fomoe_b200_tokens_download(self._h, first, count, _fp(out)), "tokens_download")
        return out

    def get_routing(self, layer):
        ids = np.empty(self.top_k, dtype=np.int32)
        ids0 = np.empty(self.top_k, dtype=np.int32)
        sc = np.empty(self.top_k, dtype=np.float32)
        self._ck(self._l.fomoe_b200_get_routing(self._h, layer, _ip(ids), _fp(sc), _ip(ids0)), "get_routing")
        return ids, sc, ids0

    def status(self):
        return int(self._l.fomoe_b200_status(self._h))

    def substitutions(self):
        return int(self._l.fomoe_b200_substitutions(self._h))

    def kernel_launches(self):
        return int(self._l.fomoe_b200_kernel_launches(self._h))

    def trace(self, first, count, cta=0):
        """Run `count` resident tokens with phase stamps of block `cta`; returns (index, ns) arrays."""
        cap = 9 * self.n_layers * count
        self._ck(self._l.fomoe_b200_trace_enable(self._h, cap, cta), "trace_enable")
        self.tokens_run(first, count)
        buf = np.zeros(cap * (self.n_blocks() if cta < 0 else 1), dtype=np.uint64)
        self._ck(self._l.fomoe_b200_trace_read(self._h, buf.ctypes.data_as(C.POINTER(C.c_uint64)), buf.size),
                 "trace_read")
        self._ck(self._l.fomoe_b200_trace_enable(self._h, 0, 0), "trace_enable")
        return (buf >> np.uint64(56)).astype(np.int64), (buf & np.uint64((1 << 56) - 1)).astype(np.int64)

    def n_blocks(self):
        import torch
        return torch.cuda.get_device_properties(self.device).multi_processor_count

    def tp_recv_ptr(self):
        return int(self._l.fomoe_b200_tp_recv_ptr(self._h) or 0)

    def tp_connect_ptrs(self, ptrs):
        """ptrs: the receive buffers (device addresses) of all tp_size ranks of this process, rank order."""
        arr = (C.c_void_p * len(ptrs))(*ptrs)
        self._ck(self._l.fomoe_b200_tp_connect_ptrs(self._h, arr), "tp_connect_ptrs")

    def tp_enable_peer(self, peer_device):
        self._ck(self._l.fomoe_b200_tp_enable_peer(self._h, int(peer_device)), "tp_enable_peer")

    def tp_inject(self, src_rank, partial=None, ahead=1):
        """Host-side stand-in for rank `src_rank`: its partial (zeros if None) for the layer-token `ahead` after the
        last one launched."""
        p = None if partial is None else _f32(partial)
        self._ck(self._l.fomoe_b200_tp_inject(self._h, src_rank, None if p is None else p.ctypes.data, ahead), "tp_inject")

    def trace_open(self, path):
        """Append a routing-trace record (the reference's format, tools/read_trace.py) per layer and token from now on."""
        self._ck(self._l.fomoe_b200_routing_trace_open(self._h, path.encode()), "routing_trace_open")

    def trace_close(self):
        self._ck(self._l.fomoe_b200_routing_trace_close(self._h), "routing_trace_close")

    def enable_expert_freq(self):
        self._ck(self._l.fomoe_b200_enable_expert_freq(self._h), "enable_expert_freq")

    def expert_freq(self):
        out = np.zeros((self.n_layers, self.n_experts), dtype=np.uint32)
        self._ck(self._l.fomoe_b200_get_expert_freq(self._h, out.ctypes.data_as(C.POINTER(C.c_uint32))), "get_expert_freq")
        return out

    def set_wait_limit(self, polls):
        self._ck(self._l.fomoe_b200_set_wait_limit(self._h, int(polls)), "set_wait_limit")

    def set_allreduce(self, fn):
        """fn(device_pointer, n_floats, cuda_stream_handle) -> 0: the caller's in-place sum over the tensor-parallel
        ranks, enqueued on that stream; used by the per-phase kernels (set_variant(0)).  None removes it."""
        if fn is None:
            self._allreduce_cb = None
            self._ck(self._l.fomoe_b200_set_allreduce(self._h, None, None), "set_allreduce")
            return
        proto = C.CFUNCTYPE(C.c_int, C.c_void_p, C.c_void_p, C.c_int, C.c_void_p)
        self._allreduce_cb = proto(lambda user, ptr, n, stream: int(fn(ptr, n, stream) or 0))
        self._ck(self._l.fomoe_b200_set_allreduce(self._h, C.cast(self._allreduce_cb, C.c_void_p), None),
                 "set_allreduce")

    def stream_handle(self):
        return int(self._l.fomoe_b200_stream(self._h) or 0)

    def tp_export(self):
        """64-byte handle of this rank's receive buffer (bytes)."""
        buf = C.create_string_buffer(64)
        self._ck(self._l.fomoe_b200_tp_export(self._h, buf), "tp_export")
        return buf.raw

    def tp_connect(self, handles):
        """handles: list of tp_size 64-byte handles in rank order."""
        blob = b"".join(handles)
        assert len(blob) == 64 * self.tp_size
        self._ck(self._l.fomoe_b200_tp_connect(self._h, blob), "tp_connect")

    def set_variant(self, variant):
        """2: persistent stack kernel for whole tokens (default); 0 / 1: per-phase kernels (plain / ring)."""
        self._ck(self._l.fomoe_b200_set_variant(self._h, variant), "set_variant")

    def set_graphs(self, enable):
        self._ck(self._l.fomoe_b200_set_graphs(self._h, int(bool(enable))), "set_graphs")

    def peek(self, what, n_slots=None):
        """Intermediates of the most recent layer call: 'act', 'q8a', 'q8h', 'dots', 'h'."""
        ns = self.top_k + int(self.has_shared) if n_slots is None else n_slots
        il = 256 if self.half_mode else self.n_inter // self.tp_size
        sel, dtype, shape = {"act": (0, np.float32, (ns, il)), "q8a": (1, np.uint8, (ns, il // 256, 304)),
                             "q8h": (2, np.uint8, (self.n_embd // 256, 304)),
                             "dots": (3, np.float32, (ns, self.n_embd)), "h": (4, np.float32, (self.n_embd,))}[what]
        out = np.empty(shape, dtype=dtype)
        self._ck(self._l.fomoe_b200_peek(self._h, sel, out.ctypes.data, out.nbytes), "peek")
        return out

    # ---- micro helpers
    def matvec(self, qtype, w_ggml, rows, cols, x):
        w = np.ascontiguousarray(w_ggml).view(np.uint8).reshape(-1)
        assert w.size == matrix_bytes(qtype, rows, cols)
        x = _f32(x)
        y = np.empty(rows, dtype=np.float32)
        self._ck(self._l.fomoe_b200_matvec(self._h, qtype, w.ctypes.data, rows, cols, _fp(x), _fp(y)), "matvec")
        return y

    def quantize_q8k(self, x):
        x = _f32(x)
        out = np.empty((x.size // 256) * 292, dtype=np.uint8)
        self._ck(self._l.fomoe_b200_quantize_q8k(self._h, _fp(x), x.size, out.ctypes.data), "quantize_q8k")
        return out


class GpuOperator:
    """The reference's gpu.h operator surface (gpu_init / gpu_expert_ffn / gpu_free)."""

    def __init__(self):
        self._l = lib()
        self._h = self._l.gpu_init()
        if not self._h:
            raise RuntimeError("gpu_init failed: no CUDA device")

    def close(self):
        if getattr(self, "_h", None):
            self._l.gpu_free(self._h)
            self._h = None

    __del__ = close

    def attach(self, decoder):
        """The statistics calls of this surface (expert histogram, dims) report `decoder` (a MoeDecoder) from now on."""
        if self._l.fomoe_b200_gpu_attach(self._h, decoder._h if decoder is not None else None) != 0:
            raise RuntimeError("fomoe_b200_gpu_attach failed")

    def enable_expert_freq(self):
        self._l.gpu_enable_expert_freq(self._h)

    def expert_dims(self):
        a, b = C.c_int(0), C.c_int(0)
        self._l.gpu_get_expert_dims(self._h, C.byref(a), C.byref(b))
        return a.value, b.value

    def expert_freq(self):
        """uint32[n_layers, n_experts] or None (not enabled / nothing attached)."""
        p = self._l.gpu_get_expert_freq(self._h)
        if not p:
            return None
        nl, ne = self.expert_dims()
        return np.ctypeslib.as_array(C.cast(p, C.POINTER(C.c_uint32)), shape=(nl, ne)).copy()

    def expert_ffn(self, h, expert_buffers, scores, n_embd, inter, gate_size, up_size, stride, gate_type, up_type,
                   down_type):
        """Returns (rc, ffn_out); rc == -1 means "fall back to the CPU path" as in the reference."""
        h, scores = _f32(h), _f32(scores)
        # an int is taken as a raw address (e.g. a record already in device memory), anything else as host bytes
        keep = [e if isinstance(e, int) else np.ascontiguousarray(e).view(np.uint8).reshape(-1) for e in expert_buffers]
        ptrs = (C.c_void_p * len(keep))(*[e if isinstance(e, int) else e.ctypes.data for e in keep])
        out = np.zeros(n_embd, dtype=np.float32)
        rc = self._l.gpu_expert_ffn(self._h, _fp(h), ptrs, _fp(scores), len(keep), n_embd, inter, gate_size, up_size,
                                    stride, gate_type, up_type, down_type, _fp(out))
        return rc, out


class ExpertEngine:
    """CUDA twin of the reference's cpu_expert.h engine (create/reset/ffn/submit_async/wait/result)."""

    def __init__(self, n_embd, inter):
        self._l = lib()
        self.n_embd, self.inter = n_embd, inter
        self._h = self._l.b200_expert_create(n_embd, inter)
        if not self._h:
            raise RuntimeError("b200_expert_create failed: no CUDA device or unsupported shape")
        self._keep = []

    def close(self):
        if getattr(self, "_h", None):
            self._l.b200_expert_free(self._h)
            self._h = None

    __del__ = close

    def reset(self):
        self._l.b200_expert_reset(self._h)

    def ffn(self, expert, x, score, gate_type, up_type, down_type, gate_size, up_size):
        e = np.ascontiguousarray(expert).view(np.uint8).reshape(-1)
        x = _f32(x)
        self._l.b200_expert_ffn(self._h, e.ctypes.data, _fp(x), score, gate_type, up_type, down_type, gate_size,
                                up_size)

    def submit_async(self, x, experts, scores, gate_type, up_type, down_type, gate_size, up_size):
        self._keep = [np.ascontiguousarray(e).view(np.uint8).reshape(-1) for e in experts] + [_f32(x)]
        w = (Work * len(experts))()
        for i, e in enumerate(self._keep[:-1]):
            w[i] = Work(e.ctypes.data, float(scores[i]), gate_type, up_type, down_type, gate_size, up_size)
        self._l.b200_expert_submit_async(self._h, _fp(self._keep[-1]), w, len(experts))

    def wait(self):
        self._l.b200_expert_wait(self._h)

    def result(self):
        p = self._l.b200_expert_result(self._h)
        return np.ctypeslib.as_array(p, shape=(self.n_embd,)).copy()

    def timing(self):
        a, b, n = C.c_double(0), C.c_double(0), C.c_int(0)
        self._l.b200_expert_get_timing(self._h, C.byref(a), C.byref(b), C.byref(n))
        return a.value, b.value, n.value


class BatchedMoe:
    """Many tokens per call (prefill / batched decode): routed-expert FFN on the tensor cores, Q4_K experts."""

    def __init__(self, n_layers, n_embd, n_inter, n_experts, top_k, has_shared=True, max_tokens=512, device=0,
                 rms_eps=1e-6, tp_rank=0, tp_size=1):
        self._l = lib()
        self.n_layers, self.n_embd, self.n_inter = n_layers, n_embd, n_inter
        self.n_experts, self.top_k, self.has_shared, self.max_tokens = n_experts, top_k, bool(has_shared), max_tokens
        self.tp_rank, self.tp_size, self._hook = tp_rank, tp_size, None
        cfg = BatchConfig(device, n_layers, n_embd, n_inter, n_experts, top_k, int(bool(has_shared)), max_tokens, rms_eps,
                          tp_rank, tp_size)
        self._h = self._l.fomoe_b200_batch_create(C.byref(cfg))
        if not self._h:
            raise RuntimeError("fomoe_b200_batch_create failed (no CUDA device, unsupported shape or out of memory)")

    def close(self):
        if getattr(self, "_h", None):
            self._l.fomoe_b200_batch_destroy(self._h)
            self._h = None

    __del__ = close

    def _ck(self, rc, what):
        if rc != 0:
            raise RuntimeError(f"{what}: {self._l.fomoe_b200_batch_last_error(self._h).decode()}")

    def record_bytes(self):
        """Bytes of a whole expert record in ggml order (what upload_expert takes)."""
        return 2 * matrix_bytes(TYPE_Q4_K, self.n_inter, self.n_embd) + matrix_bytes(TYPE_Q4_K, self.n_embd, self.n_inter)

    def shard_bytes(self):
        """Bytes of this rank's shard of a record (what export_expert returns: gate rows | up rows | down columns)."""
        return self.record_bytes() // self.tp_size

    def set_allreduce(self, fn):
        """fn(ptr, n, stream) -> 0: sums the n floats at device pointer ptr over the ranks, in place, on that stream."""
        if fn is None:
            self._hook = None
            self._ck(self._l.fomoe_b200_batch_set_allreduce(self._h, None, None), "set_allreduce")
            return
        proto = C.CFUNCTYPE(C.c_int, C.c_void_p, C.c_void_p, C.c_int, C.c_void_p)
        self._hook = proto(lambda user, ptr, n, stream: int(fn(ptr, n, stream) or 0))
        self._ck(self._l.fomoe_b200_batch_set_allreduce(self._h, self._hook, None), "set_allreduce")

    def table_bytes(self):
        return int(self._l.fomoe_b200_batch_table_bytes(self._h))

    def kernel_launches(self):
        return int(self._l.fomoe_b200_batch_kernel_launches(self._h))

    def status(self):
        return int(self._l.fomoe_b200_batch_status(self._h))

    def generate(self, seed, with_logits=False):
        self._ck(self._l.fomoe_b200_batch_generate(self._h, seed, int(bool(with_logits))), "batch_generate")

    def upload_expert(self, layer, expert, record):
        r = np.ascontiguousarray(record).view(np.uint8).reshape(-1)
        assert r.size == self.record_bytes()
        self._ck(self._l.fomoe_b200_batch_upload(self._h, layer, expert, r.ctypes.data), "batch_upload")

    def export_expert(self, layer, expert):
        out = np.empty(self.shard_bytes(), dtype=np.uint8)
        self._ck(self._l.fomoe_b200_batch_export(self._h, layer, expert, out.ctypes.data), "batch_export")
        return out

    def moe_layer(self, layer, h, logits):
        """h [T, n_embd], logits [T, n_experts] -> dict(out [T, n_embd], ids [T, k], scores [T, k])."""
        h = _f32(h).reshape(-1, self.n_embd)
        lg = _f32(logits).reshape(-1, self.n_experts)
        T = h.shape[0]
        assert lg.shape[0] == T
        out = np.empty_like(h)
        ids = np.empty((T, self.top_k), dtype=np.int32)
        sc = np.empty((T, self.top_k), dtype=np.float32)
        self._ck(self._l.fomoe_b200_batch_moe_layer(self._h, layer, T, _fp(h), _fp(lg), _fp(out), _ip(ids), _fp(sc)),
                 "batch_moe_layer")
        return dict(out=out, ids=ids, scores=sc)

    def tokens_upload(self, x):
        x = _f32(x).reshape(-1, self.n_embd)
        self._ck(self._l.fomoe_b200_batch_tokens_upload(self._h, x.shape[0], _fp(x)), "batch_tokens_upload")

    def stack_run(self, n_tokens, l0=0, l1=None):
        """Layers [l0, l1) on the resident tokens; returns CUDA-event milliseconds."""
        ms = C.c_float(0.0)
        self._ck(self._l.fomoe_b200_batch_stack_run(self._h, n_tokens, l0, self.n_layers if l1 is None else l1, C.byref(ms)),
                 "batch_stack_run")
        return float(ms.value)

    def tokens_download(self, n_tokens):
        out = np.empty((n_tokens, self.n_embd), dtype=np.float32)
        self._ck(self._l.fomoe_b200_batch_tokens_download(self._h, n_tokens, _fp(out)), "batch_tokens_download")
        return out

    def wait_profile(self, on):
        """on=True: start counting block 0's wait cycles per role; on=False: -> uint64[16] (see the C header)."""
        out = np.zeros(16, dtype=np.uint64)
        self._ck(self._l.fomoe_b200_batch_wait_profile(self._h, int(bool(on)), out.ctypes.data_as(C.POINTER(C.c_uint64))),
                 "batch_wait_profile")
        return out

    def get_routing(self, n_tokens):
        ids = np.empty((n_tokens, self.top_k), dtype=np.int32)
        sc = np.empty((n_tokens, self.top_k), dtype=np.float32)
        cnt = np.empty(self.n_experts + int(self.has_shared), dtype=np.int32)
        self._ck(self._l.fomoe_b200_batch_get_routing(self._h, n_tokens, _ip(ids), _fp(sc), _ip(cnt)), "batch_get_routing")
        return ids, sc, cnt


def synth_logits(seed, layer, n_tokens, n_experts):
    """Seeded router logits N(0, 1) of a layer as the batched benchmark configuration draws them: [n_tokens, n_experts]."""
    out = np.empty((n_tokens, n_experts), dtype=np.float32)
    lib().fomoe_b200_batch_synth_logits(seed, layer, n_tokens, n_experts, n_tokens, _fp(out))
    return out
