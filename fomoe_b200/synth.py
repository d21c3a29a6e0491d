"""Seeded synthetic inputs (hidden states, routers, expert records) from the host-only generator library
``libfomoe_synth.so``: the same bytes the device generator puts into the expert table, without loading the CUDA
library.  The CPU arm of the benchmark takes its inputs from here."""
import ctypes as C
import os

import numpy as np

_HERE = os.path.dirname(os.path.abspath(__file__))
LIB_PATH = os.path.join(_HERE, "libfomoe_synth.so")
TYPE_Q4_K, TYPE_Q5_K, TYPE_Q6_K = 12, 13, 14
M_GATE, M_UP, M_DOWN = 0, 1, 2
STREAM_ROUTER, STREAM_RESID, STREAM_NORMW, STREAM_HIDDEN = 3, 4, 5, 6
BLOCK_BYTES = {TYPE_Q4_K: 144, TYPE_Q5_K: 176, TYPE_Q6_K: 210}
_lib = None


def _l():
    global _lib
    if _lib is None:
        if not os.path.exists(LIB_PATH):
            raise ImportError(f"{LIB_PATH} is missing: build it with `make -C fomoe_b200/csrc`")
        _lib = C.CDLL(LIB_PATH)
        _lib.fomoe_synth_matrix.argtypes = [C.c_uint64] + [C.c_int] * 6 + [C.c_void_p]
        _lib.fomoe_synth_matrix.restype = None
        _lib.fomoe_synth_f32.argtypes = [C.c_uint64, C.c_int, C.c_int, C.c_float, C.c_float, C.c_uint64, C.c_void_p]
        _lib.fomoe_synth_f32.restype = None
    return _lib


def matrix_bytes(qtype, rows, cols):
    return rows * (cols // 256) * BLOCK_BYTES[qtype]


def matrix(seed, layer, expert, m, qtype, rows, cols):
    out = np.empty(matrix_bytes(qtype, rows, cols), dtype=np.uint8)
    _l().fomoe_synth_matrix(seed, layer, expert, m, qtype, rows, cols, out.ctypes.data)
    return out


def f32(seed, layer, stream_id, mean, std, n):
    out = np.empty(n, dtype=np.float32)
    _l().fomoe_synth_f32(seed, layer, stream_id, mean, std, n, out.ctypes.data)
    return out


def hidden(seed, token, n_embd):
    return f32(seed, token, STREAM_HIDDEN, 0.0, 1.0, n_embd)


def router(seed, layer, n_experts, n_embd):
    return f32(seed, layer, STREAM_ROUTER, 0.0, 0.02, n_experts * n_embd).reshape(n_experts, n_embd)


def glue(seed, layer, n_embd):
    return f32(seed, layer, STREAM_RESID, 0.0, 1.0, n_embd), f32(seed, layer, STREAM_NORMW, 1.0, 0.1, n_embd)


def expert_record(seed, layer, expert, down_type, n_embd, inter):
    """gate | up | down in ggml byte order, the reference's record layout (include/expert_store.h:9-40)."""
    return np.concatenate([matrix(seed, layer, expert, M_GATE, TYPE_Q4_K, inter, n_embd),
                           matrix(seed, layer, expert, M_UP, TYPE_Q4_K, inter, n_embd),
                           matrix(seed, layer, expert, M_DOWN, down_type, n_embd, inter)])
