"""PTQ1_0 host-side data format helpers (numpy): packing, unpacking and seeded synthetic tensors.

PTQ1_0 block (reference: runtime_vk/ptq_decode.h:8-19): 28 bytes = 128 ternary weights + fp16 scale.
  bytes  0..15  byte j, trit t (0..4) -> element 16*t + j
  bytes 16..23  byte j, trit t (0..4) -> element 80 + 8*t + (j-16)
  bytes 24..25  byte h, trit t (0..3) -> element 120 + 2*t + h
  bytes 26..27  fp16 block scale
A byte holds its trits as a base-3 fixed-point fraction: trit_t = floor(b * 3^(t+1) / 256) mod 3
(runtime_vk/align_27b.cpp:56-75). The reference has no encoder; `encode` is the inverse map
b = ceil(n * 256 / 3^T), n = sum_t trit_t * 3^(T-1-t), T = 5 (qs bytes) or 4 (qh bytes).

These helpers only prepare inputs (synthetic weights, GGUF tensors). They do not compute any part
of the decode path.
"""
from __future__ import annotations

import numpy as np

BLOCK_BYTES = 28
BLOCK_ELEMS = 128

# element index of (byte, trit level); -1 where a byte has no such level (qh bytes, level 4)
_ELEM = np.full((26, 5), -1, dtype=np.int64)
for _j in range(16):
    for _t in range(5):
        _ELEM[_j, _t] = 16 * _t + _j
for _j in range(8):
    for _t in range(5):
        _ELEM[16 + _j, _t] = 80 + 8 * _t + _j
for _h in range(2):
    for _t in range(4):
        _ELEM[24 + _h, _t] = 120 + 2 * _t + _h


def encode(sym: np.ndarray, scale_bits: np.ndarray) -> np.ndarray:
    """sym: [..., nblk, 128] values in {0,1,2}; scale_bits: [..., nblk] uint16 -> [..., nblk, 28] uint8."""
    sym = np.asarray(sym)
    lead = sym.shape[:-1]
    s = sym.reshape(-1, BLOCK_ELEMS).astype(np.uint32)
    out = np.empty((s.shape[0], BLOCK_BYTES), dtype=np.uint8)
    # qs bytes: 5 trits
    n = np.zeros((s.shape[0], 24), dtype=np.uint32)
    for t in range(5):
        n = n * 3 + s[:, _ELEM[:24, t]]
    out[:, :24] = ((n * 256 + 242) // 243).astype(np.uint8)
    n = np.zeros((s.shape[0], 2), dtype=np.uint32)
    for t in range(4):
        n = n * 3 + s[:, _ELEM[24:, t]]
    out[:, 24:26] = ((n * 256 + 80) // 81).astype(np.uint8)
    sb = np.asarray(scale_bits, dtype=np.uint16).reshape(-1)
    out[:, 26] = (sb & 0xFF).astype(np.uint8)
    out[:, 27] = (sb >> 8).astype(np.uint8)
    return out.reshape(*lead, BLOCK_BYTES)


def decode_symbols(blocks: np.ndarray) -> np.ndarray:
    """[..., 28] uint8 -> [..., 128] int8 raw symbols {0,1,2} (weight = (symbol-1)*scale)."""
    b = np.asarray(blocks, dtype=np.uint8)
    lead = b.shape[:-1]
    flat = b.reshape(-1, BLOCK_BYTES).astype(np.uint32)
    out = np.zeros((flat.shape[0], BLOCK_ELEMS), dtype=np.int8)
    for t in range(5):
        p = 3 ** (t + 1)
        tr = ((flat[:, :26] * p) >> 8) % 3
        nb = 26 if t < 4 else 24
        out[:, _ELEM[:nb, t]] = tr[:, :nb].astype(np.int8)
    return out.reshape(*lead, BLOCK_ELEMS)


def scales_f32(blocks: np.ndarray) -> np.ndarray:
    b = np.asarray(blocks, dtype=np.uint8)
    bits = b[..., 26].astype(np.uint16) | (b[..., 27].astype(np.uint16) << 8)
    return bits.view(np.float16).astype(np.float32)


def dequant(blocks: np.ndarray) -> np.ndarray:
    """[..., nblk, 28] -> [..., nblk*128] float32 weights."""
    sym = decode_symbols(blocks).astype(np.float32) - 1.0
    w = sym * scales_f32(blocks)[..., None]
    return w.reshape(*w.shape[:-2], -1)


def synth_matrix(rng: np.random.Generator, M: int, K: int, p_neg: float = 0.3, p_zero: float = 0.4,
                 scale_sigma: float = 0.02) -> np.ndarray:
    """Seeded synthetic PTQ1_0 matrix [M, K/128, 28]: trits i.i.d. P(-1)=p_neg, P(0)=p_zero,
    P(+1)=1-p_neg-p_zero; one fp16 scale per block drawn from |N(0, scale_sigma)|."""
    assert K % BLOCK_ELEMS == 0
    nb = K // BLOCK_ELEMS
    u = rng.random((M, nb, BLOCK_ELEMS), dtype=np.float32)
    sym = (u >= p_neg).astype(np.int8) + (u >= p_neg + p_zero).astype(np.int8)
    sc = np.abs(rng.normal(0.0, scale_sigma, size=(M, nb))).astype(np.float16)
    return encode(sym, sc.view(np.uint16))


# fp16 scale bit patterns the reference's decode test crosses with every byte value
# (runtime_vk/align_dequant.cpp:91-99): zeros, subnormals, extremes, +-Inf, NaN.
EDGE_SCALE_BITS = (0x0000, 0x8000, 0x0001, 0x0123, 0x03FF, 0x83FF, 0x0400, 0x8400, 0x3C00,
                   0x7BFF, 0xFBFF, 0x7C00, 0xFC00, 0x7E00, 0xFE00)


def align_dequant_synth() -> np.ndarray:
    """The reference's synthetic decode matrix (runtime_vk/align_dequant.cpp:235-248): 15 scale
    patterns x 256 blocks, byte slot j of block q = (q + 7*j) & 0xFF. Returns [3840, 28] uint8."""
    out = np.empty((len(EDGE_SCALE_BITS), 256, BLOCK_BYTES), dtype=np.uint8)
    q = np.arange(256)[:, None]
    j = np.arange(26)[None, :]
    body = ((q + 7 * j) & 0xFF).astype(np.uint8)
    for e, bits in enumerate(EDGE_SCALE_BITS):
        out[e, :, :26] = body
        out[e, :, 26] = bits & 0xFF
        out[e, :, 27] = bits >> 8
    return out.reshape(-1, BLOCK_BYTES)


def xorshift32_bytes(n: int, seed: int = 0x2545F491):
    """The reference kernel lab's generator (runtime_vk/bonsai_vk.cpp:414-416): xorshift32, one
    byte (low 8 bits) per step. Returns (bytes[n], final state)."""
    out = np.empty(n, dtype=np.uint8)
    st = seed
    for i in range(n):
        st ^= (st << 13) & 0xFFFFFFFF
        st ^= st >> 17
        st ^= (st << 5) & 0xFFFFFFFF
        out[i] = st & 0xFF
    return out, st
