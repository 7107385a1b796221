"""The CPU checker against vectors produced by the reference's own CPU code (tests/golden/reference_vectors.npz,
written by tests/golden/make_golden.py from oracle/_ref/libref.so). Needs neither the reference tree nor the shim,
so the pin also holds on a machine that has only this repository."""
import os

import numpy as np
import pytest

from bonsai_vk_b200 import ptq

GOLD = os.path.join(os.path.dirname(os.path.abspath(__file__)), "golden", "reference_vectors.npz")


@pytest.fixture(scope="module")
def gold():
    return np.load(GOLD)


def test_trit_recurrence_and_element_map(oracle, gold):
    got = np.array([[oracle.lib.bo_trit_of_byte(b, t) for t in range(5)] for b in range(256)], dtype=np.int8)
    assert np.array_equal(got, gold["trits"])
    # the python packer follows the same map: element e lives in byte em[e,0] at level em[e,1]
    em = gold["elem_map"]
    sym = np.zeros((128, 128), dtype=np.int8)
    for e in range(128):
        sym[e, e] = 1                                   # block e: only element e is +1
    blocks = oracle.ptq_encode(sym, np.full(128, 0x3C00, dtype=np.uint16))
    trits = oracle.ptq_trits(blocks)
    assert np.array_equal(trits, sym)
    for e in range(128):
        by, tr = int(em[e, 0]), int(em[e, 1])
        assert int(gold["trits"][blocks[e, by], tr]) == 1


def test_half_conversions(oracle, gold):
    f = oracle.f16_to_f32(gold["h2f_bits"])
    assert np.array_equal(f.view(np.uint32), gold["h2f_out_bits"])
    h = oracle.f32_to_f16(gold["f2h_in_bits"].view(np.float32))
    want = gold["f2h_out"]
    nan = (want & 0x7C00) == 0x7C00
    nan &= (want & 0x03FF) != 0
    assert np.array_equal(h[~nan], want[~nan])
    assert np.all((h[nan] & 0x7C00) == 0x7C00) and np.all((h[nan] & 0x03FF) != 0)


def test_dequantisers(oracle, gold):
    got = oracle.ptq_dequant(gold["dq_blocks"]).view(np.uint32)
    for key in ("dq_ours_bits", "dq_official_bits"):
        want = gold[key]
        wf, gf = want.view(np.float32), got.view(np.float32)
        both_nan = np.isnan(wf) & np.isnan(gf)
        assert np.array_equal(np.isnan(wf), np.isnan(gf)), key
        assert np.array_equal(got[~both_nan], want[~both_nan]), key


def test_projection_truth(oracle, gold):
    W, x, y = gold["gemv_W"], gold["gemv_x"], gold["gemv_y"]
    got = oracle.gemv_dequant_f64(W, W.shape[0], x.size, x)
    assert np.array_equal(got, y)
    # and the packer's own dequantiser agrees with it
    assert np.allclose(ptq.dequant(W.reshape(W.shape[0], -1, 28)).astype(np.float64) @ x.astype(np.float64), y, rtol=1e-12, atol=1e-12)
