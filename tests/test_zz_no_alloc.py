"""The allocation-free projection entry point (bn_gemv_q81_static) against the regular one and the CPU oracle.

A host that is not allowed to allocate device memory while it runs - it handed out its whole device budget
when it loaded the model, or it is recording a stream capture - calls this variant: the split-K partial sums
go to an 8 MiB array compiled into the library instead of a buffer the library would have to cudaMalloc.
Both entry points run the same arithmetic, so the outputs must be the same floats. The call is made twice in
a row because the built-in array is shared and keeps the previous call's contents. This file is named so that
pytest collects it last; it must pass alone in a fresh process and after the rest of the suite."""
import os

import numpy as np
import pytest

from bonsai_vk_b200 import BonsaiError, ptq

pytestmark = pytest.mark.gpu
THREADS = max(1, os.cpu_count() or 1)


def _matrix(rng, M, K):
    if M <= 16384:
        return ptq.synth_matrix(rng, M, K)
    chunk = ptq.synth_matrix(rng, 16384, K)            # large shapes: a 16384-row chunk repeated (values do not matter here)
    return np.concatenate([chunk] * ((M + 16383) // 16384), axis=0)[:M]


def _setup(ctx, M, K, seed):
    rng = np.random.default_rng(seed)
    W = _matrix(rng, M, K)
    x = rng.standard_normal(K).astype(np.float32)
    xb, wb = ctx.from_numpy(x), ctx.from_numpy(W)
    pack = ctx.alloc(ctx.act_pack_bytes(K))
    ctx.act_quant_q81(xb, K, pack)
    return W, x, xb, wb, pack


# the last two shapes: the output head of the 9B model (1 986 560 partial sums) and a shape that fills the built-in
# array exactly (2 x 1 048 576 = 2 097 152 partial sums)
@pytest.mark.parametrize("M,K", [(4096, 4096), (1000, 12288), (37, 640), (248320, 4096), (1048576, 1024)])
def test_static_scratch_matches_regular_entry_point_and_oracle_twice(ctx, oracle, M, K):
    W, x, xb, wb, pack = _setup(ctx, M, K, seed=M + K)
    ref = ctx.alloc(M * 4)
    ctx.gemv_q81(wb, M, K, pack, ref)                     # regular entry point as a host calls it (streamed kernel where the shape allows)
    ctx.sync()
    want = ref.download(np.float32, M)
    o_out, _, _ = oracle.gemv_q81(W, M, K, oracle.quantize_q8_1(x), threads=THREADS)
    assert np.array_equal(want.view(np.uint32), o_out.view(np.uint32)), "regular entry point differs from the oracle"
    out = ctx.alloc(M * 4)
    ctx.gemv_q81_static(wb, M, K, pack, out)              # first use on this device: looks the array's address up
    ctx.sync()
    free_before = ctx.info()["free_bytes"]
    for call in range(2):
        out.memset(0xFF)
        ctx.gemv_q81_static(wb, M, K, pack, out)
        ctx.sync()
        got = out.download(np.float32, M)
        assert np.array_equal(got.view(np.uint32), o_out.view(np.uint32)), f"call {call}: differs from the oracle"
        assert np.array_equal(got.view(np.uint32), want.view(np.uint32)), f"call {call}: not the floats of bn_gemv_q81"
    assert ctx.info()["free_bytes"] == free_before, "the allocation-free entry point changed the free device memory"
    # a different shape right after: the array still holds the previous call's partial sums
    M2, K2 = 200, 1024
    W2, x2, xb2, wb2, pack2 = _setup(ctx, M2, K2, seed=5)
    r2, o2 = ctx.alloc(M2 * 4), ctx.alloc(M2 * 4)
    ctx.gemv_q81(wb2, M2, K2, pack2, r2)
    ctx.gemv_q81_static(wb2, M2, K2, pack2, o2)
    ctx.sync()
    assert np.array_equal(o2.download(np.uint32, M2), r2.download(np.uint32, M2))
    for b in (xb, wb, pack, ref, out, xb2, wb2, pack2, r2, o2):
        b.free()


def test_static_scratch_refuses_oversized_shapes(ctx):
    # ceil(K/512) * M beyond the built-in 2 Mi floats: refused before anything is launched
    w = ctx.alloc(64)
    out = ctx.alloc(64)
    for M, K in ((300000, 4096), (1048577, 1024)):
        pack = ctx.alloc(ctx.act_pack_bytes(K))
        with pytest.raises(BonsaiError, match="built-in scratch"):
            ctx.gemv_q81_static(w, M, K, pack, out)
        pack.free()
    for b in (w, out):
        b.free()
