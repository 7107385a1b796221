"""Writes tests/golden/reference_vectors.npz from the reference's OWN CPU code (oracle/_ref/libref.so, compiled by
oracle/Makefile from the reference headers ptq_decode.h, f16_rne_host.h and attn_vk.h where they lie).

    make -C oracle && python tests/golden/make_golden.py

The vectors travel with the repository, so the CPU checker can be pinned against the reference's outputs on a machine
that has neither the reference tree nor the shim (tests/test_golden.py). All inputs are generated from fixed seeds
and stored next to the outputs.
"""
import ctypes as C
import os
import sys

import numpy as np

ROOT = os.path.dirname(os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
sys.path.insert(0, ROOT)

from bonsai_vk_b200 import ptq  # noqa: E402
from tests import _oracle  # noqa: E402


def _p(a):
    return a.ctypes.data_as(C.c_void_p)


def main():
    ref = _oracle.load_ref()
    if ref is None:
        raise SystemExit("oracle/_ref/libref.so is missing: run `make -C oracle` where the reference tree is mounted")
    rng = np.random.default_rng(20250101)
    out = {}
    # trit recurrence and element map
    out["trits"] = np.array([[ref.ref_trit_of_byte(b, t) for t in range(5)] for b in range(256)], dtype=np.int8)
    em = np.empty((128, 2), dtype=np.int32)
    for e in range(128):
        by, tr = C.c_int(), C.c_int()
        ref.ref_elem_to_byte_trit(e, C.byref(by), C.byref(tr))
        em[e] = (by.value, tr.value)
    out["elem_map"] = em
    # fp16 <-> fp32: every exponent class, specials, ties
    bits = np.concatenate([np.arange(0, 65536, 97, dtype=np.uint32), np.array([0, 1, 0x3FF, 0x400, 0x7BFF, 0x7C00, 0x7C01, 0x7E00, 0x8000,
                           0x8001, 0xFBFF, 0xFC00, 0xFE00], dtype=np.uint32)]).astype(np.uint16)
    f = np.empty(bits.size, dtype=np.float32)
    ref.ref_f16_to_f32(_p(bits), bits.size, _p(f))
    out["h2f_bits"], out["h2f_out_bits"] = bits, f.view(np.uint32)
    probes = np.concatenate([rng.standard_normal(300).astype(np.float32) * np.float32(10.0) ** rng.integers(-8, 5, 300).astype(np.float32),
                             np.array([0.0, -0.0, 65504.0, 65520.0, 65519.99, 1e-8, 5.96e-8, 2.98e-8, 2.9802322e-8, 6.1e-5, np.inf, -np.inf,
                                       np.nan, 1.0009765625, 1.00048828125, 1.000732421875], dtype=np.float32)]).astype(np.float32)
    h = np.empty(probes.size, dtype=np.uint16)
    ref.ref_f32_to_f16(_p(probes), probes.size, _p(h))
    out["f2h_in_bits"], out["f2h_out"] = probes.view(np.uint32), h
    # both reference dequantisers on random bytes (243..255 included) with edge scales
    blocks = rng.integers(0, 256, size=(24, 28), dtype=np.uint8)
    edge = np.array(ptq.EDGE_SCALE_BITS, dtype=np.uint16)
    sc = np.concatenate([edge, rng.integers(0, 0x7BFF, size=24 - len(edge)).astype(np.uint16)])[:24] if len(edge) < 24 else edge[:24]
    blocks[:, 26] = (sc & 0xFF).astype(np.uint8)
    blocks[:, 27] = (sc >> 8).astype(np.uint8)
    ours = np.empty((24, 128), dtype=np.float32)
    off = np.empty((24, 128), dtype=np.float32)
    ref.ref_ptq_dequant_ours(_p(blocks), C.c_long(24), _p(ours))
    ref.ref_ptq_dequant_official(_p(blocks), C.c_long(24), _p(off))
    out["dq_blocks"], out["dq_ours_bits"], out["dq_official_bits"] = blocks, ours.view(np.uint32), off.view(np.uint32)
    # dequantise + fp64 dot (the reference's CPU truth for a projection)
    M, K = 12, 512
    W = np.ascontiguousarray(ptq.synth_matrix(np.random.default_rng(5), M, K))
    x = np.random.default_rng(6).standard_normal(K).astype(np.float32)
    y = np.empty(M, dtype=np.float64)
    ref.ref_gemv_dequant_f64(_p(W), M, K, _p(x), _p(y), 1)
    out["gemv_W"], out["gemv_x"], out["gemv_y"] = W, x, y
    path = os.path.join(ROOT, "tests", "golden", "reference_vectors.npz")
    np.savez_compressed(path, **out)
    print("wrote", path, os.path.getsize(path), "bytes")


if __name__ == "__main__":
    main()
