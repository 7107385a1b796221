"""CPU checks of the q8_1 quantiser, the integer block dots and the two GEMV restatements."""
import numpy as np
import pytest

from bonsai_vk_b200 import ptq


def _unpack_q81(xq):
    blk = xq.reshape(-1, 36)
    d = (blk[:, :4] & 0xFFFF).astype(np.uint16).view(np.float16).astype(np.float32)
    s = (blk[:, :4] >> 16).astype(np.uint16).view(np.float16).astype(np.float32)
    q = blk[:, 4:].copy().view(np.int8).reshape(-1, 4, 32)
    return d, s, q


def test_q81_recipe(oracle):
    rng = np.random.default_rng(3)
    x = rng.standard_normal(1024).astype(np.float32)
    x[128:160] = 0.0                      # dead block: d = 0, codes 0
    x[200] = 1e-36                        # below the 1e-35 floor is still "dead" territory for amax
    d, s, q = _unpack_q81(oracle.quantize_q8_1(x))
    xb = x.reshape(-1, 4, 32)
    amax = np.abs(xb).max(axis=2)
    d32 = np.where(amax > 1e-35, amax / np.float32(127.0), np.float32(0)).astype(np.float32)
    assert np.array_equal(d, d32.astype(np.float16).astype(np.float32))
    inv = np.where(d32 != 0, np.float32(1.0) / np.where(d32 != 0, d32, 1), 0).astype(np.float32)
    prod = (xb * inv[:, :, None]).astype(np.float32)
    want = np.clip(np.sign(prod) * np.floor(np.abs(prod) + np.float32(0.5)), -127, 127).astype(np.int8)
    assert np.array_equal(q, want)
    assert np.array_equal(s, (d32 * q.sum(axis=2).astype(np.float32)).astype(np.float16).astype(np.float32))
    assert np.all(q[1, 0] == 0) and d[1, 0] == 0.0
    assert np.abs(q).max() <= 127


def test_q81_ties_round_away_from_zero(oracle):
    x = np.zeros(128, dtype=np.float32)
    x[0] = 127.0            # d = 1 exactly
    x[1], x[2], x[3], x[4] = 0.5, -0.5, 1.5, -2.5
    _, _, q = _unpack_q81(oracle.quantize_q8_1(x))
    assert list(q[0, 0, :5]) == [127, 1, -1, 2, -3]


def test_block_dots_definition_vs_shader_lanes(oracle):
    """The lane-level restatement of _mul_mat_vecq_ptq1_0.comp (16-bit-lane multiply, residue cancelled
    by masked activations, packed dot products) gives the same four sub-block sums as sum(trit*q)."""
    rng = np.random.default_rng(11)
    x = (rng.standard_normal(128 * 64) * 3).astype(np.float32)
    xq = oracle.quantize_q8_1(x).reshape(-1, 36)
    blocks = rng.integers(0, 256, size=(64, 28), dtype=np.uint8)     # raw bytes incl. 243..255
    legal = ptq.synth_matrix(rng, 1, 128 * 64)[0]
    for i in range(64):
        for blk in (blocks[i], legal[i]):
            a = oracle.block_dots(blk, xq[i])
            b = oracle.block_dots(blk, xq[i], shader=True)
            assert np.array_equal(a, b)
            sym = oracle.ptq_trits(blk)[0].astype(np.int64)
            q = xq[i, 4:].copy().view(np.int8).astype(np.int64)
            assert np.array_equal(a, (sym * q).reshape(4, 32).sum(axis=1))


@pytest.mark.parametrize("K", [128, 512, 640, 4096])
def test_gemv_q81_float_close_to_exact(oracle, K):
    rng = np.random.default_rng(K)
    M = 96
    W = ptq.synth_matrix(rng, M, K)
    x = rng.standard_normal(K).astype(np.float32)
    xq = oracle.quantize_q8_1(x)
    out, exact, dots = oracle.gemv_q81(W, M, K, xq, want_dots=True)
    assert dots.shape == (M, K // 128, 4)
    scale = np.sqrt(np.mean(exact ** 2))
    assert np.max(np.abs(out - exact)) <= 2e-6 * scale
    # and the q8_1 result tracks the unquantised product to quantisation accuracy
    truth = oracle.gemv_dequant_f64(W, M, K, x)
    assert np.max(np.abs(exact - truth)) <= 0.05 * scale


def test_gemv_f32act_engine_form(oracle):
    """gemv_ternary.comp form d*(sum c*x - xsum) agrees with dequantise+dot to the reference's own
    gate (rel < 1e-5, bonsai_weights.h:769-782) and is split-count stable."""
    rng = np.random.default_rng(5)
    M, K = 128, 4096
    W = ptq.synth_matrix(rng, M, K)
    x = rng.standard_normal(K).astype(np.float32)
    truth = oracle.gemv_dequant_f64(W, M, K, x)
    scale = np.sqrt(np.mean(truth ** 2))
    for S in (1, 4, 8):
        out, exact = oracle.gemv_f32act(W, M, K, x, n_splits=S)
        assert np.max(np.abs(exact - truth)) <= 1e-9 * scale
        assert np.max(np.abs(out - truth)) <= 1e-5 * scale


def test_kernel_lab_case_scale_one(oracle):
    """Reference kernel-lab input (bonsai_vk.cpp:414-429): xorshift32 bytes, every scale 1.0,
    x in [-1, 1); its CPU truth d*(cs - xs) (bonsai_vk.cpp:752-772) equals dequantise+dot."""
    M, K = 16, 256
    nbytes = M * (K // 128) * 28
    raw, st = ptq.xorshift32_bytes(nbytes)
    W = raw.reshape(M, K // 128, 28).copy()
    W[:, :, 26] = 0x00
    W[:, :, 27] = 0x3C
    x = np.empty(K, dtype=np.float32)
    for i in range(K):
        st ^= (st << 13) & 0xFFFFFFFF
        st ^= st >> 17
        st ^= (st << 5) & 0xFFFFFFFF
        x[i] = np.float32((st & 0xFFFF) / 32768.0) - np.float32(1.0)
    truth = oracle.gemv_dequant_f64(W, M, K, x)
    sym = oracle.ptq_trits(W).astype(np.float64).reshape(M, K)
    want = sym @ x.astype(np.float64) - x.astype(np.float64).sum()
    assert np.allclose(truth, want, rtol=0, atol=1e-9)
    out, _ = oracle.gemv_f32act(W, M, K, x)
    assert np.max(np.abs(out - truth)) < 1e-4      # the lab expects rel ~1e-6 on values of order 10


def test_table_driven_block_dots_equal_the_definition(oracle):
    """The whole-token checker evaluates the integer block dots through a 256-entry trit table; it must give the very
    numbers of the per-element definition (sum trit_e * q_e with trit_of_byte, ptq_decode.h:34-45) on raw random bytes
    (243..255 included), on every byte value in every position, and with extreme activation codes."""
    rng = np.random.default_rng(11)
    for _ in range(300):
        blk = rng.integers(0, 256, size=28, dtype=np.uint8)
        xq = np.zeros(36, dtype=np.uint32)
        xq[4:] = rng.integers(-127, 128, size=128).astype(np.int8).view(np.uint32)
        assert np.array_equal(oracle.block_dots(blk, xq), oracle.block_dots(blk, xq, fast=True))
    xq = np.zeros(36, dtype=np.uint32)
    xq[4:] = np.full(128, 127, dtype=np.int8).view(np.uint32)
    for v in range(256):
        blk = np.full(28, v, dtype=np.uint8)
        assert np.array_equal(oracle.block_dots(blk, xq), oracle.block_dots(blk, xq, fast=True))
