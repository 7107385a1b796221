"""Pins the CPU oracle for the PTQ1_0 format and the fp16 conversions against the reference's own
known-answer tests and, where the reference shim is built, against the reference's real CPU code.

Reference tests mirrored here:
  runtime_vk/align_27b.cpp:56-111   recurrence == closed form over 256 x 5; element map bijection
  runtime_vk/align_dequant.cpp:91-99,235-248  15 fp16 scale patterns x 256 byte patterns, 3-way equal
  runtime_vk/align_dequant.cpp:491-515        d*(cs - xs) == sum(w*x) with LCG activations
  runtime_vk/align_f16.cpp:1-22               all 65 536 fp16 patterns vs the IEEE definition
"""
import ctypes as C

import numpy as np
import pytest

from bonsai_vk_b200 import ptq


def _p(a):
    return a.ctypes.data_as(C.c_void_p)


def test_trit_recurrence_equals_closed_form(oracle):
    for b in range(256):
        for t in range(5):
            assert oracle.lib.bo_trit_of_byte(b, t) == oracle.lib.bo_trit_closed_form(b, t)
            assert 0 <= oracle.lib.bo_trit_of_byte(b, t) <= 2


def test_trit_matches_reference_code(oracle, ref):
    for b in range(256):
        for t in range(5):
            assert oracle.lib.bo_trit_of_byte(b, t) == ref.ref_trit_of_byte(b, t)


def test_element_map_bijection_80_40_8(oracle):
    seen = {}
    by, tr = C.c_int(), C.c_int()
    for e in range(128):
        oracle.lib.bo_elem_to_byte_trit(e, C.byref(by), C.byref(tr))
        seen[(by.value, tr.value)] = e
    assert len(seen) == 128
    assert sum(1 for (b, t) in seen if b < 16) == 80
    assert sum(1 for (b, t) in seen if 16 <= b < 24) == 40
    assert sum(1 for (b, t) in seen if b >= 24) == 8
    assert all(t <= 3 for (b, t) in seen if b >= 24)


def test_element_map_matches_reference_code(oracle, ref):
    a, b, c, d = C.c_int(), C.c_int(), C.c_int(), C.c_int()
    for e in range(128):
        oracle.lib.bo_elem_to_byte_trit(e, C.byref(a), C.byref(b))
        ref.ref_elem_to_byte_trit(e, C.byref(c), C.byref(d))
        assert (a.value, b.value) == (c.value, d.value)


def test_f16_to_f32_all_patterns_vs_ieee(oracle):
    bits = np.arange(65536, dtype=np.uint16)
    got = oracle.f16_to_f32(bits)
    want = bits.view(np.float16).astype(np.float32)
    nan = np.isnan(want)
    assert np.array_equal(got[~nan].view(np.uint32), want[~nan].view(np.uint32))
    assert np.all(np.isnan(got[nan]))
    # NaN payload is carried, not canonicalised (runtime_vk/ptq_decode.h:62-72): 0x7C10 -> 0x7F820000
    assert got.view(np.uint32)[0x7C10] == 0x7F820000
    # subnormals are man * 2^-24 exactly (runtime_vk/ptq_decode.h:51-60)
    assert got[0x0001] == np.float32(2.0 ** -24)
    assert got[0x0123] == np.float32(0x123 * 2.0 ** -24)


def test_f16_to_f32_all_patterns_vs_reference_code(oracle, ref):
    bits = np.arange(65536, dtype=np.uint16)
    got = oracle.f16_to_f32(bits)
    want = np.empty(65536, dtype=np.float32)
    ref.ref_f16_to_f32(_p(bits), 65536, _p(want))
    assert np.array_equal(got.view(np.uint32), want.view(np.uint32))


def _f32_probe_values():
    rng = np.random.default_rng(7)
    vals = [rng.standard_normal(20000).astype(np.float32) * s for s in (1e-8, 1e-5, 1e-3, 1.0, 100.0, 7e4)]
    # every fp16 value, the midpoints between neighbours, and one ulp either side of the midpoints
    h = np.arange(0x7C00, dtype=np.uint16).view(np.float16).astype(np.float64)
    mid = ((h[:-1] + h[1:]) / 2).astype(np.float32)
    vals += [h.astype(np.float32), mid, np.nextafter(mid, np.float32(np.inf)), np.nextafter(mid, np.float32(-np.inf))]
    vals.append(np.array([0.0, -0.0, np.inf, -np.inf, np.nan, 65504.0, 65519.99, 65520.0, 1e-45, 2.0 ** -25,
                          2.0 ** -24, 3e-8], dtype=np.float32))
    v = np.concatenate(vals)
    return np.concatenate([v, -v])


def test_f32_to_f16_rne_vs_numpy(oracle):
    v = _f32_probe_values()
    got = oracle.f32_to_f16(v)
    with np.errstate(over="ignore"):
        want = v.astype(np.float16).view(np.uint16)
    nan = np.isnan(v)
    # binary32 subnormal inputs flush to signed zero in the reference packer (f16_rne_host.h:41)
    tiny = np.abs(v) < np.float32(2.0 ** -126)
    ok = ~nan & ~tiny
    assert np.array_equal(got[ok], want[ok])
    assert np.all((got[nan] & 0x7FFF) == 0x7E00)
    assert np.all((got[tiny & ~nan] & 0x7FFF) == 0)


def test_f32_to_f16_vs_reference_code(oracle, ref):
    v = np.ascontiguousarray(_f32_probe_values())
    want = np.empty(v.size, dtype=np.uint16)
    ref.ref_f32_to_f16(_p(v), v.size, _p(want))
    assert np.array_equal(oracle.f32_to_f16(v), want)


def _bits_equal_nan_aware(a, b):
    na, nb = np.isnan(a), np.isnan(b)
    return np.array_equal(na, nb) and np.array_equal(a[~na].view(np.uint32), b[~nb].view(np.uint32))


def test_align_dequant_synth_matrix_census(oracle):
    """The reference's synthetic decode matrix: 3 840 blocks / 491 520 weights; class counts quoted
    by the reference for it: 10 880 NaN + 21 888 Inf per +-Inf scale class (FAITHFUL_REPRO.md:96-107)."""
    blocks = ptq.align_dequant_synth()
    assert blocks.shape == (3840, 28)
    w = oracle.ptq_dequant(blocks)
    assert w.size == 491520
    per = w.reshape(15, 256 * 128)
    for e, bits in enumerate(ptq.EDGE_SCALE_BITS):
        if bits in (0x7C00, 0xFC00):       # Inf scale: 0*Inf = NaN for the zero symbol, +-Inf otherwise
            assert int(np.isnan(per[e]).sum()) == 10880
            assert int(np.isinf(per[e]).sum()) == 21888
    # numpy decode of the same blocks agrees symbol for symbol
    sym = ptq.decode_symbols(blocks)
    assert np.array_equal(sym, oracle.ptq_trits(blocks))


def test_align_dequant_synth_three_way(oracle, ref):
    """oracle == reference ptq_dequant_ours == reference transcription of the official shader."""
    blocks = np.ascontiguousarray(ptq.align_dequant_synth())
    mine = oracle.ptq_dequant(blocks)
    ours = np.empty_like(mine)
    off = np.empty_like(mine)
    ref.ref_ptq_dequant_ours(_p(blocks), C.c_long(blocks.shape[0]), _p(ours))
    ref.ref_ptq_dequant_official(_p(blocks), C.c_long(blocks.shape[0]), _p(off))
    assert _bits_equal_nan_aware(mine.ravel(), ours.ravel())
    assert _bits_equal_nan_aware(mine.ravel(), off.ravel())
    # NaN bit patterns too (payload and sign), not only the class
    assert np.array_equal(mine.view(np.uint32), ours.view(np.uint32))


def test_encoder_inverts_decoder_exhaustively(oracle):
    # every 5-trit and 4-trit code, placed in every byte slot
    sym = np.zeros((243, 128), dtype=np.int8)
    for n in range(243):
        digits = [(n // 3 ** (4 - t)) % 3 for t in range(5)]
        for e in range(128):
            by, tr = C.c_int(), C.c_int()
            oracle.lib.bo_elem_to_byte_trit(e, C.byref(by), C.byref(tr))
            sym[n, e] = digits[tr.value] if by.value < 24 else digits[tr.value + 1]
    enc = oracle.ptq_encode(sym, np.full(243, 0x3C00, dtype=np.uint16))
    assert np.array_equal(oracle.ptq_trits(enc), sym)
    assert np.array_equal(ptq.encode(sym, np.full(243, 0x3C00, dtype=np.uint16)), enc)
    assert int(enc[:, :24].max()) <= 255


def test_out_of_range_bytes_still_decode(oracle):
    """Bytes 243..255 are outside the legal pack space but decode to {0,1,2} (align_27b.cpp:71)."""
    blocks = np.zeros((13, 28), dtype=np.uint8)
    for i, b in enumerate(range(243, 256)):
        blocks[i, :26] = b
    t = oracle.ptq_trits(blocks)
    assert t.min() >= 0 and t.max() <= 2


def test_dot_form_identity(oracle):
    """d*(cs - xs) == sum(w*x) on the synthetic matrix with the reference's LCG activations
    (runtime_vk/align_dequant.cpp:491-515)."""
    blocks = ptq.align_dequant_synth()
    w = oracle.ptq_dequant(blocks).astype(np.float64)
    sym = oracle.ptq_trits(blocks).astype(np.float64)
    d = ptq.scales_f32(blocks).astype(np.float64)
    lcg = 12345
    worst = 0.0
    for p in range(blocks.shape[0]):
        x = np.empty(128)
        for e in range(128):
            lcg = (lcg * 6364136223846793005 + 1442695040888963407) & 0xFFFFFFFFFFFFFFFF
            x[e] = np.float32(((lcg >> 33) % 2000) / 1000.0 - 1.0)
        if not np.isfinite(d[p]):
            continue
        a = d[p] * (float(sym[p] @ x) - float(x.sum()))
        b = float(w[p] @ x)
        worst = max(worst, abs(a - b) / (abs(a) + 1e-30) if a != 0 else abs(b))
    assert worst < 1e-9


def test_kernel_lab_generator_first_bytes():
    """xorshift32 seeded 0x2545F491 (runtime_vk/bonsai_vk.cpp:414-416)."""
    by, st = ptq.xorshift32_bytes(4)
    s = 0x2545F491
    exp = []
    for _ in range(4):
        s ^= (s << 13) & 0xFFFFFFFF
        s ^= s >> 17
        s ^= (s << 5) & 0xFFFFFFFF
        exp.append(s & 0xFF)
    assert list(by) == exp and st == s


@pytest.mark.parametrize("seed", [0, 1])
def test_gemv_truth_matches_reference_code(oracle, ref, seed):
    """The dequantise + float64 dot used as GEMV truth (bonsai_weights.h:751-768) - oracle port vs
    the loop over the reference's own dequantiser."""
    rng = np.random.default_rng(seed)
    M, K = 64, 512
    W = np.ascontiguousarray(ptq.synth_matrix(rng, M, K))
    x = rng.standard_normal(K).astype(np.float32)
    mine = oracle.gemv_dequant_f64(W, M, K, x)
    want = np.empty(M, dtype=np.float64)
    ref.ref_gemv_dequant_f64(_p(W), M, K, _p(x), _p(want), 1)
    assert np.array_equal(mine, want)
