"""The allocation-free matvec entry point (fomoe_b200_matvec_noalloc).

It exists for callers that may not allocate device memory while running (all memory handed out at start-up,
or no tolerance for cudaMalloc's device-wide synchronisation): its temporaries sit in a fixed array inside the
library.  The caller brings device buffers; here torch provides them.  The result must equal the allocating
entry point's (same kernels, same arithmetic: bit for bit) on two calls in a row, the second with different
data so stale scratch contents would show, and oversize requests must be refused.

This file sorts last on purpose: a run that stops at the first failure has then already run everything else.
"""
import ctypes as C

import numpy as np
import pytest

import helpers as H

pytestmark = pytest.mark.gpu


def _dev(t):
    return C.c_void_p(t.data_ptr())


@pytest.mark.parametrize("qtype,rows,cols", [(H.Q4, 1024, 4096), (H.Q6, 4096, 1024), (H.Q6, 24, 512)])
def test_noalloc_matches_allocating_entry_point(fb, oracle, qtype, rows, cols):
    import torch
    lib = fb.lib()
    dec = fb.MoeDecoder(1, 256, 256, 2, 1, False, [H.Q6])   # only for the allocating reference call
    torch.cuda.set_device(0)
    y_dev = torch.empty(rows, dtype=torch.float32, device="cuda")
    for call in range(2):
        w = fb.synth_matrix(50 + call, 0, call, fb.M_GATE, qtype, rows, cols)
        x = H.hidden(fb, 50 + call, call, cols)
        w_dev = torch.from_numpy(w).cuda()
        x_dev = torch.from_numpy(x).cuda()
        y_dev.fill_(float("nan"))
        torch.cuda.synchronize()
        rc = lib.fomoe_b200_matvec_noalloc(qtype, _dev(w_dev), rows, cols, _dev(x_dev), _dev(y_dev), None)
        assert rc == 0
        torch.cuda.synchronize()
        got = y_dev.cpu().numpy()
        want = dec.matvec(qtype, w, rows, cols, x)
        assert (H.bits(got) == H.bits(want)).all(), call
        assert H.rel_l2(got, oracle.matvec_q8(w, qtype, x, rows, cols)) < 2e-6
    dec.close()


def test_noalloc_refuses_what_does_not_fit(fb):
    import torch
    lib = fb.lib()
    torch.cuda.set_device(0)
    d = torch.zeros(16, dtype=torch.float32, device="cuda")
    # 4096 x 4096 Q4_K = 9.4 MB of weights: beyond the 4 MiB array
    assert lib.fomoe_b200_matvec_noalloc(H.Q4, _dev(d), 4096, 4096, _dev(d), _dev(d), None) == -1
    assert lib.fomoe_b200_matvec_noalloc(H.Q4, _dev(d), 4, 16384, _dev(d), _dev(d), None) == -1   # > 8192 columns
    assert lib.fomoe_b200_matvec_noalloc(8, _dev(d), 4, 256, _dev(d), _dev(d), None) == -1        # Q8_0: not a type it takes
    assert lib.fomoe_b200_matvec_noalloc(H.Q4, None, 4, 256, _dev(d), _dev(d), None) == -1


def test_noalloc_second_device_after_the_first(fb, oracle):
    """The array's device address is looked up per device: a call on device 1 after calls on device 0 must use
    device 1's copy (needs two GPUs)."""
    import torch
    if torch.cuda.device_count() < 2:
        pytest.skip("needs 2 GPUs")
    lib = fb.lib()
    qtype, rows, cols = H.Q4, 512, 1024
    w = fb.synth_matrix(77, 0, 0, fb.M_GATE, qtype, rows, cols)
    x = H.hidden(fb, 77, 0, cols)
    want = oracle.matvec_q8(w, qtype, x, rows, cols)
    outs = []
    for dev in (0, 1, 0):
        torch.cuda.set_device(dev)
        w_dev, x_dev = torch.from_numpy(w).cuda(dev), torch.from_numpy(x).cuda(dev)
        y_dev = torch.full((rows,), float("nan"), dtype=torch.float32, device=f"cuda:{dev}")
        torch.cuda.synchronize(dev)
        assert lib.fomoe_b200_matvec_noalloc(qtype, _dev(w_dev), rows, cols, _dev(x_dev), _dev(y_dev), None) == 0
        torch.cuda.synchronize(dev)
        outs.append(y_dev.cpu().numpy())
        assert H.rel_l2(outs[-1], want) < 2e-6
    assert (H.bits(outs[0]) == H.bits(outs[1])).all() and (H.bits(outs[0]) == H.bits(outs[2])).all()
    torch.cuda.set_device(0)
