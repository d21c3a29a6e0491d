"""Dequant-matvec with Q8_K activations against the CPU oracle
(reference src/quant.c:343-375, 405-607; src/cpu_expert.c:52-72)."""
import numpy as np
import pytest

import helpers as H

pytestmark = pytest.mark.gpu

# fp32 only reassociates the <=16-term sum over super-blocks; everything below that is exact integer work
TOL = 2e-6


@pytest.fixture(scope="module")
def dec(fb):
    d = fb.MoeDecoder(1, 256, 256, 2, 1, False, [H.Q6])
    yield d
    d.close()


@pytest.mark.parametrize("n", [256, 1024, 4096])
def test_quantize_q8k_bit_exact(fb, dec, oracle, n):
    rng = np.random.default_rng(n)
    x = rng.normal(0, 1, n).astype(np.float32)
    x[5] = 0.5 / (127.0 / np.abs(x[:256]).max())  # an exact .5 rounding case
    assert (dec.quantize_q8k(x) == oracle.quantize_q8k(x)).all()
    z = np.zeros(n, dtype=np.float32)
    z[n - 256:] = x[:256]
    assert (dec.quantize_q8k(z) == oracle.quantize_q8k(z)).all()  # all-zero blocks: d = 0, qs = 0


@pytest.mark.parametrize("qtype,rows,cols", [(H.Q4, 1024, 4096), (H.Q6, 4096, 1024), (H.Q4, 4096, 1024),
                                             (H.Q4, 64, 256), (H.Q6, 40, 512), (H.Q6, 8, 8192), (H.Q4, 3, 2048),
                                             (H.Q5, 4096, 1024), (H.Q5, 24, 512)])
def test_matvec_vs_oracle(fb, dec, oracle, qtype, rows, cols):
    w = fb.synth_matrix(9, 0, 1, fb.M_GATE, qtype, rows, cols)
    x = H.hidden(fb, 9, rows, cols)
    got = dec.matvec(qtype, w, rows, cols, x)
    want = oracle.matvec_q8(w, qtype, x, rows, cols)
    # Q4_K / Q6_K: both sides form exact integer block sums, only the fp32 sum over blocks is reassociated.
    # Q5_K: the reference adds 256 rounded fp32 products per block (src/quant.c:609-621), the device sums exact
    # integers, so the two differ by the reference's own rounding noise.
    tol, peak = (TOL, 1e-5) if qtype != H.Q5 else (3e-5, 1e-4)
    assert H.rel_l2(got, want) < tol
    scale = np.abs(want).max()
    assert np.abs(got - want).max() <= peak * scale


def test_matvec_reference_patterns(fb, dec, oracle):
    """Deterministic block patterns of the reference's tools/test_matvec.c:21-31, 88-99 (K=3072 there;
    K=2048 here because the kernels take power-of-two block counts)."""
    K, M = 2048, 16
    nb = M * K // 256
    f16 = lambda v: np.float16(v).view(np.uint16)
    q4 = np.zeros((nb, 144), dtype=np.uint8)
    for i in range(nb):
        q4[i, 0:2] = np.frombuffer(f16(0.5 + 0.1 * (i % 7)).tobytes(), dtype=np.uint8)
        q4[i, 2:4] = np.frombuffer(f16(0.1 + 0.05 * (i % 5)).tobytes(), dtype=np.uint8)
        q4[i, 4:16] = [(10 + (i + j) % 50) for j in range(12)]
        q4[i, 16:] = [((i * 7 + j * 3) & 0xFF) for j in range(128)]
    x = (np.sin(np.arange(K, dtype=np.float32) * np.float32(0.01)) * np.float32(0.1)).astype(np.float32)
    got = dec.matvec(H.Q4, q4, M, K, x)
    assert H.rel_l2(got, oracle.matvec_q8(q4, H.Q4, x, M, K)) < TOL
    q6 = np.zeros((nb, 210), dtype=np.uint8)
    for i in range(nb):
        q6[i, 0:128] = [((i * 5 + j * 7) & 0xFF) for j in range(128)]
        q6[i, 128:192] = [((i * 3 + j * 11) & 0xFF) for j in range(64)]
        q6[i, 192:208] = np.array([((i + j * 3) % 64 - 32) for j in range(16)], dtype=np.int8).view(np.uint8)
        q6[i, 208:210] = np.frombuffer(f16(0.3 + 0.1 * (i % 5)).tobytes(), dtype=np.uint8)
    x = (np.cos(np.arange(K, dtype=np.float32) * np.float32(0.01)) * np.float32(0.1)).astype(np.float32)
    got = dec.matvec(H.Q6, q6, M, K, x)
    assert H.rel_l2(got, oracle.matvec_q8(q6, H.Q6, x, M, K)) < TOL


def test_matvec_extreme_scales(fb, dec, oracle):
    """Full-range int8 Q6_K scales and maximal nibbles/quants."""
    rng = np.random.default_rng(1)
    rows, cols = 64, 1024
    q6 = rng.integers(0, 256, (rows * 4, 210), dtype=np.uint8)
    q6[:, 208:210] = np.frombuffer(np.float16(0.01).tobytes(), dtype=np.uint8)
    q6[0, 0:192] = 0xFF
    q6[0, 192:208] = 0x80  # scale -128
    x = rng.normal(0, 3, cols).astype(np.float32)
    assert H.rel_l2(dec.matvec(H.Q6, q6, rows, cols, x), oracle.matvec_q8(q6, H.Q6, x, rows, cols)) < TOL
    q4 = rng.integers(0, 256, (rows * 4, 144), dtype=np.uint8)
    q4[:, 0:4] = np.frombuffer(np.array([0.02, 0.01], dtype=np.float16).tobytes(), dtype=np.uint8)
    q4[1, 4:] = 0xFF
    assert H.rel_l2(dec.matvec(H.Q4, q4, rows, cols, x), oracle.matvec_q8(q4, H.Q4, x, rows, cols)) < TOL


@pytest.mark.parametrize("qtype,rows,cols", [(H.Q8_0, 1024, 4096), (H.MXFP4, 1024, 4096), (H.Q8_0, 7, 96),
                                              (H.MXFP4, 33, 32), (H.MXFP4, 4096, 1024)])
def test_blocks32_matvec_f32(fb, oracle, qtype, rows, cols):
    """Q8_0 / MXFP4 projections on fp32 activations against src/quant.c:276-288, 320-337: fp32 reassociation only
    (every weight is exact in fp32), so 1e-5 relative L2; special blocks (NaN exponent, smallest exponent, zero
    scale, extreme quants) included; a matrix already in device memory gives the same bits as a host one."""
    d = fb.MoeDecoder(1, 256, 256, 4, 1, False, [H.Q4])
    m = H.blocks32_matrix(qtype, rows, cols, 100 + rows)
    x = np.random.default_rng(rows).standard_normal(cols).astype(np.float32)
    got = d.proj_matvec_f32(qtype, m, rows, cols, x)
    want = oracle.mat_vec_mul_f32act(m, qtype, x, rows, cols)
    assert np.isfinite(got).all()
    err = H.rel_l2(got, want)
    print(f"type {qtype} {rows}x{cols}: rel-L2 {err:.2e}")
    assert err < 1e-5
    assert d.status() == 0
    d.close()


def test_shared_ffn_f32_blocks32(fb, oracle):
    """The reference's shared_expert_ffn (src/inference.c:361-374) with MXFP4 gate/up + Q8_0 down and with Q8_0
    gate/up + MXFP4 down, at the 397B shared-expert shape."""
    n_embd, inter = 4096, 1024
    d = fb.MoeDecoder(1, 256, 256, 4, 1, False, [H.Q4])
    h = H.hidden(fb, 5, 0, n_embd)
    for gt, dt in ((H.MXFP4, H.Q8_0), (H.Q8_0, H.MXFP4)):
        g, u = H.blocks32_matrix(gt, inter, n_embd, 11, special=False), H.blocks32_matrix(gt, inter, n_embd, 12, special=False)
        dn = H.blocks32_matrix(dt, n_embd, inter, 13, special=False)
        got = d.shared_ffn_f32(h, g, gt, u, gt, dn, dt, n_embd, inter)
        want = oracle.shared_ffn_f32(h, g, gt, u, gt, dn, dt, n_embd, inter)
        err = H.rel_l2(got, want)
        print(f"shared FFN gate/up type {gt}, down type {dt}: rel-L2 {err:.2e}")
        assert np.isfinite(got).all() and err < 1e-5
    with pytest.raises(RuntimeError):                      # K-quant types are not served by this entry
        d.proj_matvec_f32(H.Q4, np.zeros(144 * 8, dtype=np.uint8), 8, 256, h[:256])
    d.close()

