"""Kernel lab: one synthetic PTQ1_0 x q8_1 GEMV, timed (the counterpart of the reference's
`bonsai_vk <M> <K> <S> <ITER>` mode, runtime_vk/bonsai_vk.cpp:227-924).

  python -m bonsai_vk_b200.kernel_lab M K [ITER]
  python -m bonsai_vk_b200.kernel_lab attn CTX [ITER]      one decode-attention layer (16/4 heads x 256, q8_0 K and V)
  python -m bonsai_vk_b200.kernel_lab gemm M K NCOL [ITER]  the multi-column tensor-core projection (tcgen05), timed
  python -m bonsai_vk_b200.kernel_lab stage NBLOCKS NCOL CTX [ITER]   one pipeline stage (first NBLOCKS blocks of the 9B
                                            shape) for NCOL sequences per pass at context CTX, timed per pass
  python -m bonsai_vk_b200.kernel_lab stamps [TOKENS]       where one B=1 token of the 9B shape spends its time: device time
                                            stamps of CTA 0 of every fused projection launch (the reference's per-token
                                            ledger idea, BONSAI_PROFILE, bonsai_forward.h:650-662)

Prints ms/op, Gop/s and GB/s of PTQ1_0 bytes from CUDA events. Timing rotates through enough copies of the matrix to
exceed L2. (Results are checked against the CPU checker by the test-suite, not here.)
"""
from __future__ import annotations

import sys

import numpy as np


def attn_lab(argv, ctx=None, quiet=False):
    """One decode-attention layer: 16 query / 4 KV heads, head_dim 256, q8_0 cache of CTX keys, one query token.
    Returns (ms per layer, algorithmic bytes)."""
    from bonsai_vk_b200 import Context
    from bonsai_vk_b200 import lib as L
    ctx_len = int(argv[0])
    iters = int(argv[1]) if len(argv) > 1 else 20
    n_head, n_kv, hd = 16, 4, 256
    QD, KD = n_head * hd, n_kv * hd
    rng = np.random.default_rng(1)
    ctx = ctx or Context(0)
    dims = L.AttnDimsC(n_head=n_head, n_kv=n_kv, head_dim=hd, n_rot=64, cap=ctx_len + (ctx_len & 1), k_mode=0, v_mode=0,
                       rms_eps=1e-6, rope_base=1e7)
    kvb, scb = ctx.attn_sizes(dims)
    nlay = max(2, int(300e6 // kvb) + 1)                 # rotate over layers so the cache does not sit in L2
    kvs = [ctx.alloc(kvb) for _ in range(nlay)]
    scratch = ctx.alloc(scb)
    rows = 4096
    bk = ctx.from_numpy(rng.standard_normal((rows, KD)).astype(np.float32))
    bv = ctx.from_numpy(rng.standard_normal((rows, KD)).astype(np.float32))
    bq = ctx.from_numpy(rng.standard_normal((n_head, 2 * hd)).astype(np.float32))
    ones = ctx.from_numpy(np.ones(hd, dtype=np.float32))
    for kv in kvs:
        for p0 in range(0, ctx_len, rows):
            ctx.attn_insert(dims, kv, bk, bv, min(rows, ctx_len - p0), p0, bq, ones, ones, scratch)
    out = ctx.alloc(QD * 4)
    for kv in kvs:
        ctx.attn_attend(dims, kv, ctx_len - 1, scratch, None, out)
    ctx.sync()
    e0, e1 = ctx.event(), ctx.event()
    ctx.record(e0)
    for _ in range(iters):
        for kv in kvs:
            ctx.attn_attend(dims, kv, ctx_len - 1, scratch, None, out)
    ctx.record(e1)
    ms = ctx.elapsed_ms(e0, e1) / (iters * nlay)
    nbytes = ctx_len * n_kv * hd * 34 // 32 * 2
    if not quiet:
        print(f"attention ctx={ctx_len}: {ms * 1000:.2f} us/layer, {nbytes / ms / 1e6:.1f} GB/s of q8_0 K+V bytes "
              f"({nbytes} algorithmic bytes; {nlay} caches = {nlay * kvb / 1e6:.0f} MB rotation)")
    for b in kvs + [scratch, bk, bv, bq, ones, out]:
        b.free()
    return ms, nbytes
    ctx.close()


def gemm_lab(argv, ctx=None, quiet=False):
    """NCOL activation columns against one M x K PTQ1_0 matrix; column 0 is checked against the single-column kernel.
    Returns (ms per pass, PTQ1_0 bytes of the matrix)."""
    from bonsai_vk_b200 import Context, ptq
    M, K, ncol = int(argv[0]), int(argv[1]), int(argv[2])
    iters = int(argv[3]) if len(argv) > 3 and not argv[3].startswith("-") else 5
    tiled = "--native" not in argv
    ctx = ctx or Context(0)
    rng = np.random.default_rng(3)
    rows = min(M, 8192)
    base = ptq.synth_matrix(rng, rows, K)
    W = np.concatenate([base] * ((M + rows - 1) // rows), axis=0)[:M]
    nbytes = M * (K // 128) * 28
    ncopies = max(2, int(300e6 // nbytes) + 1)
    wb = ctx.alloc(ncopies * nbytes)
    for i in range(ncopies):
        wb.upload(W, off=i * nbytes)
    native = wb
    if tiled:                       # the kernel's own tile-major copy of every rotation copy of the matrix
        tbytes = int(ctx.lib.bn_gemm_tiled_bytes(M, K))
        wt = ctx.alloc(ncopies * tbytes)
        for i in range(ncopies):
            one = ctx.gemm_repack(wb, M, K, w_off=i * nbytes)
            wt.upload(one.download(np.uint8, tbytes), off=i * tbytes)
            one.free()
        wb, step = wt, tbytes
    else:
        step = nbytes
    X = rng.standard_normal((ncol, K)).astype(np.float32)
    xb = ctx.from_numpy(X)
    image = ctx.alloc(ctx.gemm_image_bytes(K, ncol))
    out = ctx.alloc(ncol * M * 4)
    ctx.gemm_act_quant(xb, K, ncol, image)
    ctx.gemm_q81(wb, M, K, image, ncol, out, tiled=tiled)
    ctx.sync()
    got = out.download(np.float32, ncol * M).reshape(ncol, M)
    pack = ctx.alloc(ctx.act_pack_bytes(K))
    ref = ctx.alloc(M * 4)
    ctx.act_quant_q81(xb, K, pack)
    ctx.gemv_q81(native, M, K, pack, ref)
    ctx.sync()
    same = np.array_equal(got[0].view(np.uint32), ref.download(np.float32, M).view(np.uint32))
    if not quiet:
        print(f"column 0 vs single-column kernel: {'bit-identical' if same else 'DIFFERENT'}")
    e0, e1 = ctx.event(), ctx.event()
    for i in range(ncopies):
        ctx.gemm_q81(wb, M, K, image, ncol, out, w_off=i * step, tiled=tiled)
    ctx.record(e0)
    for _ in range(iters):
        for i in range(ncopies):
            ctx.gemm_q81(wb, M, K, image, ncol, out, w_off=i * step, tiled=tiled)
    ctx.record(e1)
    import os
    ms = ctx.elapsed_ms(e0, e1) / (iters * ncopies * max(1, int(os.environ.get("BONSAI_GEMM_REPS", "1"))))
    ops = 2.0 * M * K * ncol
    if quiet:                       # called from the benchmark: hand back the numbers, keep the caller's context
        for b in {id(x): x for x in (wb, native, xb, image, out, pack, ref)}.values():
            b.free()
        return ms, nbytes
    print(f"gemm {M}x{K} x {ncol} columns ({'tile-major' if tiled else 'native'} weights): {ms * 1000:.1f} us, {nbytes / ms / 1e6:.1f} GB/s of PTQ1_0 bytes, {ops / ms / 1e9:.2f} Top/s "
          f"({ncopies} matrix copies = {ncopies * nbytes / 1e6:.0f} MB rotation)")
    ctx.close()
    return 0 if same else 1


def stage_lab(argv):
    """One stage of the layer pipeline on one GPU: blocks [0, NBLOCKS) of the 9B shape, NCOL sequences per pass."""
    from bonsai_vk_b200 import Context, Model, synth
    nblocks, ncol, ctx_len = int(argv[0]), int(argv[1]), int(argv[2])
    iters = int(argv[3]) if len(argv) > 3 else 5
    ctx = Context(0)
    hp = synth.HParams(cap=ctx_len + 64, n_streams=ncol, block_begin=0, block_end=nblocks, batch_cols=ncol if ncol > 1 else 0)
    tensors, signs = synth.make_model_repeated(hp)
    m = Model(ctx, hp, tensors, signs)
    del tensors
    out = ctx.alloc(ncol * hp.hidden * 4)
    m.stage_prepare(0, ncol if ncol > 1 else 0)
    for s in range(ncol):
        m.fill_kv(s, ctx_len)
    pos = ctx_len

    def one(p):
        if ncol > 1:
            m.stage_batch(0, [1 + c for c in range(ncol)], [p] * ncol, None, out)
        else:
            m.stage(0, 1, p, None, out)

    for i in range(3):
        one(pos + i)
    ctx.sync()
    e0, e1 = ctx.event(), ctx.event()
    ctx.record(e0)
    for i in range(iters):
        one(pos + 3 + i)
    ctx.record(e1)
    ms = ctx.elapsed_ms(e0, e1) / iters
    print(f"stage of {nblocks} blocks, {ncol} sequences per pass, context {ctx_len}: {ms:.3f} ms per pass, "
          f"{ms / ncol * 1000:.1f} us per sequence, {ms / nblocks * 1000:.1f} us per block")
    m.close()
    ctx.close()


def stamps_lab(argv):
    """Per-token ledger of the B=1 schedule from the projection kernels' own time stamps (ns, global timer)."""
    from bonsai_vk_b200 import Context, Model, synth
    reps = int(argv[0]) if argv else 5
    ctx = Context(0)
    hp = synth.HParams(cap=256)
    tensors, signs = synth.make_model_repeated(hp)
    m = Model(ctx, hp, tensors, signs)
    del tensors
    nxt = 0
    for pos in range(20):                                   # warm-up: state, cache and clocks
        nxt = m.token(int(nxt) % hp.vocab, pos)
    names = ["launch -> first copies issued", "waiting for the previous grid", "norm", "signs + Hadamard (+ q8_1 of earlier blocks)", "q8_1 (last Hadamard block)",
             "operand registers", "main loop + epilogue", "gap after the previous launch's CTA 0", "in kernel"]
    acc, span = None, 0.0
    for rep in range(reps):
        st = m.profile_token(int(nxt) % hp.vocab, 20 + rep).astype(np.int64)
        nxt = 5
        d = np.diff(st, axis=1)
        gap = np.concatenate([[0], st[1:, 0] - st[:-1, 7]])
        row = np.concatenate([d, gap[:, None], (st[:, 7] - st[:, 0])[:, None]], axis=1)
        acc = row if acc is None else acc + row
        span += (st[-1, 7] - st[0, 0]) / 1000.0
    acc = acc / reps
    print(f"{acc.shape[0]} projection launches per token, mean of {reps} tokens; first start -> last end {span / reps:.1f} us")
    print(f"{'interval':44s} {'sum us':>9s} {'mean us':>8s}  first block's 4 launches (us)")
    for k, name in enumerate(names):
        first = " ".join(f"{acc[i, k] / 1000:6.2f}" for i in range(min(4, acc.shape[0])))
        print(f"{name:44s} {acc[:, k].sum() / 1000:9.1f} {acc[:, k].mean() / 1000:8.2f}  {first}")
    m.close()


def main(argv):
    from bonsai_vk_b200 import Context, ptq
    if argv and argv[0] == "stamps":
        return stamps_lab(argv[1:])
    if argv and argv[0] == "stage":
        return stage_lab(argv[1:])
    if argv and argv[0] == "attn":
        return attn_lab(argv[1:])
    if argv and argv[0] == "gemm":
        return gemm_lab(argv[1:])
    M, K = int(argv[0]), int(argv[1])
    iters = int(argv[2]) if len(argv) > 2 and not argv[2].startswith("-") else 3
    ctx = Context(0)
    rng = np.random.default_rng(0x2545F491)
    nb = K // 128
    rows = min(M, 8192)
    base = ptq.synth_matrix(rng, rows, K)
    W = np.concatenate([base] * ((M + rows - 1) // rows), axis=0)[:M]
    x = rng.standard_normal(K).astype(np.float32)
    nbytes = M * nb * 28
    ncopies = max(2, int(300e6 // nbytes) + 1)
    wb = ctx.alloc(ncopies * nbytes)
    for i in range(ncopies):
        wb.upload(W, off=i * nbytes)
    xb = ctx.from_numpy(x)
    pack = ctx.alloc(ctx.act_pack_bytes(K))
    out = ctx.alloc(M * 4)
    ctx.act_quant_q81(xb, K, pack)
    ctx.gemv_q81(wb, M, K, pack, out)
    ctx.sync()
    for i in range(ncopies):
        ctx.gemv_q81(wb, M, K, pack, out, w_off=i * nbytes)
    e0, e1 = ctx.event(), ctx.event()
    ctx.record(e0)
    for _ in range(iters):
        for i in range(ncopies):
            ctx.gemv_q81(wb, M, K, pack, out, w_off=i * nbytes)
    ctx.record(e1)
    ms = ctx.elapsed_ms(e0, e1) / (iters * ncopies)
    print(f"M={M} K={K}: {ms:.5f} ms/op, {2.0 * M * K / ms / 1e6:.1f} Gop/s, {nbytes / ms / 1e6:.1f} GB/s of PTQ1_0 bytes "
          f"({ncopies} matrix copies = {ncopies * nbytes / 1e6:.0f} MB rotation)")
    ctx.close()


if __name__ == "__main__":
    main(sys.argv[1:])
