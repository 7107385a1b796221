"""The allocation-free projection entry point (bn_gemv_q81_static) against the regular one.

A host that is not allowed to allocate device memory while it runs - it handed out its whole device budget
when it loaded the model, or it is recording a stream capture - calls this variant: the split-K partial sums
go to an 8 MiB array compiled into the library instead of a buffer the library would have to cudaMalloc.
Both entry points run the same arithmetic, so the outputs must be the same floats. The call is made twice in
a row because the built-in array is shared and keeps the previous call's contents. This file is named so that
pytest collects it last; it must pass alone in a fresh process and after the rest of the suite."""
import numpy as np
import pytest

from bonsai_vk_b200 import BonsaiError, ptq

pytestmark = pytest.mark.gpu


def _setup(ctx, M, K, seed):
    rng = np.random.default_rng(seed)
    W = ptq.synth_matrix(rng, M, K)
    x = rng.standard_normal(K).astype(np.float32)
    xb, wb = ctx.from_numpy(x), ctx.from_numpy(W)
    pack = ctx.alloc(ctx.act_pack_bytes(K))
    ctx.act_quant_q81(xb, K, pack)
    return xb, wb, pack


@pytest.mark.parametrize("M,K", [(4096, 4096), (1000, 12288), (37, 640)])
def test_static_scratch_matches_regular_entry_point_twice(ctx, M, K):
    xb, wb, pack = _setup(ctx, M, K, seed=M + K)
    ref = ctx.alloc(M * 4)
    dots = ctx.alloc(M * (K // 128) * 16)
    ctx.gemv_q81(wb, M, K, pack, ref, dots=dots)          # regular entry point, split-K kernel (scratch from cudaMalloc)
    ctx.sync()
    want = ref.download(np.float32, M)
    out = ctx.alloc(M * 4)
    for call in range(2):
        out.memset(0xFF)
        ctx.gemv_q81_static(wb, M, K, pack, out)
        ctx.sync()
        got = out.download(np.float32, M)
        rms = float(np.sqrt(np.mean(want.astype(np.float64) ** 2)))
        assert np.max(np.abs(got - want)) <= 1e-5 * rms, f"call {call}: static-scratch result differs"
        assert np.array_equal(got.view(np.uint32), want.view(np.uint32)), f"call {call}: not the same floats"
    # a different shape right after: the array still holds the previous call's partial sums
    M2, K2 = 200, 1024
    xb2, wb2, pack2 = _setup(ctx, M2, K2, seed=5)
    r2, o2 = ctx.alloc(M2 * 4), ctx.alloc(M2 * 4)
    d2 = ctx.alloc(M2 * (K2 // 128) * 16)
    ctx.gemv_q81(wb2, M2, K2, pack2, r2, dots=d2)
    ctx.gemv_q81_static(wb2, M2, K2, pack2, o2)
    ctx.sync()
    assert np.array_equal(o2.download(np.uint32, M2), r2.download(np.uint32, M2))
    for b in (xb, wb, pack, ref, dots, out, xb2, wb2, pack2, r2, o2, d2):
        b.free()


def test_static_scratch_refuses_oversized_shapes(ctx):
    # ceil(K/512) * M beyond the built-in 2 Mi floats: refused before anything is launched
    M, K = 300000, 4096
    w = ctx.alloc(64)
    pack = ctx.alloc(ctx.act_pack_bytes(K))
    out = ctx.alloc(64)
    with pytest.raises(BonsaiError, match="built-in scratch"):
        ctx.gemv_q81_static(w, M, K, pack, out)
    for b in (w, pack, out):
        b.free()
