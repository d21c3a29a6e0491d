"""The C-ABI library loads without a GPU and exports every function include/fomoe_b200.h declares;
the host-side generator is deterministic; constructors fail cleanly without CUDA."""
import ctypes
import os
import re

import numpy as np
import pytest

import helpers as H

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def _declared_functions():
    src = open(os.path.join(ROOT, "include", "fomoe_b200.h")).read()
    src = re.sub(r"/\*.*?\*/", "", src, flags=re.S)
    src = re.sub(r"typedef struct \{.*?\} \w+;", "", src, flags=re.S)
    names = re.findall(r"\b(\w+)\s*\([^;{]*\)\s*;", src)
    return sorted(set(n for n in names if n.startswith(("gpu_", "b200_expert_", "fomoe_b200_"))))


def test_header_symbols_exported(fb):
    declared = _declared_functions()
    assert len(declared) >= 50
    raw = ctypes.CDLL(fb.LIB_PATH)
    missing = [n for n in declared if not hasattr(raw, n)]
    assert not missing, missing
    assert sorted(fb.exported_symbols()) == declared


def test_no_gpu_means_null_not_fallback(fb):
    import torch
    if torch.cuda.is_available():
        pytest.skip("a GPU is present")
    with pytest.raises(RuntimeError):
        fb.MoeDecoder(1, 256, 256, 4, 1)
    with pytest.raises(RuntimeError):
        fb.GpuOperator()
    with pytest.raises(RuntimeError):
        fb.ExpertEngine(256, 256)


def test_product_does_not_import_oracle():
    for dirpath, _, files in os.walk(os.path.join(ROOT, "fomoe_b200")):
        for f in files:
            if f.endswith((".py", ".c", ".cu", ".h", ".cuh")) or f == "Makefile":
                txt = open(os.path.join(dirpath, f)).read()
                assert "oracle" not in txt.lower() or f == "__never__", os.path.join(dirpath, f)


def test_host_generator_deterministic_and_distributed(fb):
    a = fb.synth_matrix(1, 2, 3, fb.M_GATE, H.Q4, 64, 4096)
    b = fb.synth_matrix(1, 2, 3, fb.M_GATE, H.Q4, 64, 4096)
    assert (a == b).all()
    assert not (a == fb.synth_matrix(2, 2, 3, fb.M_GATE, H.Q4, 64, 4096)).all()
    blk = a.reshape(-1, 144)
    d = blk[:, 0:4].copy().view(np.float16).astype(np.float64)
    assert 6e-4 < d.mean() < 1e-3 and d.min() >= 0  # E|N(0,1e-3)| = 7.98e-4
    nib = np.concatenate([blk[:, 16:] & 15, blk[:, 16:] >> 4], axis=None)
    assert abs(nib.mean() - 7.5) < 0.05
    q6 = fb.synth_matrix(1, 2, 3, fb.M_DOWN, H.Q6, 256, 1024).reshape(-1, 210)
    sc = q6[:, 192:208].copy().view(np.int8)
    assert sc.min() == -32 and sc.max() == 31
    r = fb.synth_f32(1, 0, fb.STREAM_ROUTER, 0.0, 0.02, 1 << 18)
    assert abs(r.std() - 0.02) < 2e-4 and abs(r.mean()) < 2e-4
    # pinned values: the generator is part of the parity contract (golden outputs depend on it)
    assert a[:8].tolist() == fb.synth_matrix(1, 2, 3, fb.M_GATE, H.Q4, 1, 256)[:8].tolist()
