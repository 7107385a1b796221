"""GPU parity of the multi-column tensor-core projection (tcgen05, through the C ABI).

The reference has no integer-dot GEMM beyond 8 columns (it falls back to dequantise + f16 matmul), so the pin is
column-wise: every column must equal the single-column projection of the same vector - the CPU oracle's
same-order restatement, bit for bit, and with it the q8_1 codes and scales the activation image was built from.
Edge scales (zero, subnormal, negative, Inf, NaN) must land in the same class as the oracle's.
"""
import numpy as np
import pytest

from bonsai_vk_b200 import ptq

pytestmark = pytest.mark.gpu


def _gemm(ctx, W, M, K, X, signs=None, hat_block=0, out_stride=0, tiled=False):
    ncol = X.shape[0]
    xb, wb = ctx.from_numpy(np.ascontiguousarray(X)), ctx.from_numpy(W)
    image = ctx.alloc(ctx.gemm_image_bytes(K, ncol))
    sb = ctx.from_numpy(signs) if signs is not None else None
    ctx.gemm_act_quant(xb, K, ncol, image, signs=sb, hat_block=hat_block)
    stride = out_stride or M
    out = ctx.alloc(ncol * stride * 4)
    wt = ctx.gemm_repack(wb, M, K) if tiled else None
    ctx.gemm_q81(wt if tiled else wb, M, K, image, ncol, out, out_stride=stride, tiled=tiled)
    ctx.sync()
    if wt is not None:
        wt.free()
    res = out.download(np.float32, ncol * stride).reshape(ncol, stride)[:, :M].copy()
    img = image.download(np.uint8, ctx.gemm_image_bytes(K, ncol))
    for b in (xb, wb, image, out) + ((sb,) if sb is not None else ()):
        b.free()
    return res, img


def _image_column(img, K, ncol, c):
    """q8_1 record of column c rebuilt from the image: (codes [K] int8, d [K/32] f32, s [K/32] f32)."""
    nb = K // 128
    ncp = 8 if ncol <= 8 else (16 if ncol <= 16 else 32)
    blocks = img[:nb * ncp * 160].reshape(nb, ncp * 160)
    codes = np.empty((nb, 4, 2, 16), dtype=np.int8)
    for sb in range(4):
        for kh in range(2):
            off = (c // 8) * 1024 + (sb * 2 + kh) * 128 + (c % 8) * 16
            codes[:, sb, kh, :] = blocks[:, off:off + 16].view(np.int8)
    # scales: per group of 8 columns 256 bytes; entry (sb, pair) = fp32 (d, d', -s, -s')
    grp = np.ascontiguousarray(blocks[:, ncp * 128 + (c // 8) * 256: ncp * 128 + (c // 8) * 256 + 256]).view(np.float32).reshape(nb, 4, 4, 4)
    d = np.ascontiguousarray(grp[:, :, (c % 8) // 2, c % 2]).reshape(-1)
    s = -np.ascontiguousarray(grp[:, :, (c % 8) // 2, 2 + c % 2]).reshape(-1)
    return codes.reshape(K), d, s + np.float32(0.0)


def _oracle_record(xq, K):
    nb = K // 128
    rec = xq.reshape(nb, 36)
    d = (rec[:, :4] & 0xFFFF).astype(np.uint16).view(np.float16).astype(np.float32).reshape(-1)
    s = (rec[:, :4] >> 16).astype(np.uint16).view(np.float16).astype(np.float32).reshape(-1)
    codes = np.ascontiguousarray(rec[:, 4:]).view(np.int8).reshape(K)
    return codes, d, s


@pytest.mark.parametrize("M,K,ncol", [(512, 1024, 3), (4096, 4096, 8), (300, 2048, 16), (1024, 12288, 16), (256, 1024, 32),
                                      (128, 4096, 1), (2048, 4096, 20)])
@pytest.mark.parametrize("tiled", [False, True])
def test_gemm_columns_equal_the_single_column_projection(ctx, oracle, M, K, ncol, tiled):
    rng = np.random.default_rng(M * 7 + K + ncol)
    W = ptq.synth_matrix(rng, M, K)
    X = rng.standard_normal((ncol, K)).astype(np.float32) * rng.uniform(0.1, 4.0, size=(ncol, 1)).astype(np.float32)
    got, img = _gemm(ctx, W, M, K, X, out_stride=M + 64 if ncol == 3 else 0, tiled=tiled)
    for c in range(ncol):
        xq = oracle.quantize_q8_1(X[c])
        codes, d, s = _image_column(img, K, ncol, c)
        oc, od, os_ = _oracle_record(xq, K)
        assert np.array_equal(codes, oc), f"column {c}: int8 codes differ"
        assert np.array_equal(d.view(np.uint32), od.view(np.uint32)) and np.array_equal(s.view(np.uint32), os_.view(np.uint32))
        out, exact, _ = oracle.gemv_q81(W, M, K, xq, want_dots=True)
        assert np.array_equal(got[c].view(np.uint32), out.view(np.uint32)), f"column {c} is not bit-identical to the GEMV restatement"
        rms = float(np.sqrt(np.mean(exact ** 2)))
        rel = np.abs(got[c].astype(np.float64) - exact) / np.maximum(np.abs(exact), 0.05 * rms)
        assert rel.max() <= 1e-5


@pytest.mark.parametrize("hb", [1024, 256, 64, 32, 16])
def test_gemm_with_rotation(ctx, oracle, hb):
    """Rotation per Hadamard block in front of the multi-column projection, down to the smallest block the reference
    accepts (16, runtime_vk/bonsai_model.h:853-858: smaller than a q8_1 sub-block)."""
    M, K, ncol = 1024, 3072, 5
    rng = np.random.default_rng(11)
    W = ptq.synth_matrix(rng, M, K)
    X = rng.standard_normal((ncol, K)).astype(np.float32)
    signs = (rng.integers(0, 2, size=K, dtype=np.int32) * 2 - 1).astype(np.int32)
    got, _ = _gemm(ctx, W, M, K, X, signs=signs, hat_block=hb, tiled=True)
    for c in range(ncol):
        y = oracle.rotate_fwd(X[c], signs, hb)
        out, _, _ = oracle.gemv_q81(W, M, K, oracle.quantize_q8_1(y), want_dots=True)
        assert np.array_equal(got[c].view(np.uint32), out.view(np.uint32))


def test_gemm_edge_scales_and_raw_bytes(ctx, oracle):
    """Raw random weight bytes (243..255 included) and the edge scale patterns: same values / same NaN-Inf class."""
    M, K, ncol = 256, 1024, 8
    rng = np.random.default_rng(5)
    W = rng.integers(0, 256, size=(M, K // 128, 28), dtype=np.uint8)
    edge = np.array(ptq.EDGE_SCALE_BITS, dtype=np.uint16)
    sc = edge[rng.integers(0, len(edge), size=(M, K // 128))]
    W[:, :, 26] = (sc & 0xFF).astype(np.uint8)
    W[:, :, 27] = (sc >> 8).astype(np.uint8)
    W = np.ascontiguousarray(W.reshape(M, -1))
    X = rng.standard_normal((ncol, K)).astype(np.float32)
    X[2] = 0.0                                        # an all-zero column: d = 0, every code 0
    got, _ = _gemm(ctx, W, M, K, X)
    for c in range(ncol):
        out, _, _ = oracle.gemv_q81(W, M, K, oracle.quantize_q8_1(X[c]), want_dots=True)
        both_nan = np.isnan(got[c]) & np.isnan(out)
        assert np.array_equal(np.isnan(got[c]), np.isnan(out))
        assert np.array_equal(got[c][~both_nan].view(np.uint32), out[~both_nan].view(np.uint32))


def test_gemm_refuses_bad_shapes(ctx):
    from bonsai_vk_b200.lib import BonsaiError
    buf = ctx.alloc(1 << 20)
    with pytest.raises(BonsaiError):
        ctx.gemm_q81(buf, 128, 1000, buf, 4, buf)          # K not a multiple of 1024
    with pytest.raises(BonsaiError):
        ctx.gemm_q81(buf, 4096, 4096, buf, 4, buf, tiled=True)   # the tiled copy would not fit the buffer
    with pytest.raises(BonsaiError):
        ctx.gemm_q81(buf, 128, 1024, buf, 33, buf)         # too many columns
    with pytest.raises(BonsaiError):
        ctx.gemm_act_quant(buf, 1024, 4, buf, signs=buf, hat_block=48)
    buf.free()
