"""Parity at the shapes the benchmark times: the 9B-shape model (32 blocks, hidden 4096, FFN 12288, vocabulary
248 320, 24 gated-delta-net + 8 attention blocks) and its largest projection, against the CPU oracle.

Weights are the seeded synthetic tensors of synth.make_model_repeated (one recurrent block, one attention block and one
FFN set reused for every block - the oracle reads the very same arrays). The oracle needs a few seconds per token at
this shape on a multi-core host, so the stream test takes a few minutes."""
import os

import numpy as np
import pytest

from bonsai_vk_b200 import Model, synth
from bonsai_vk_b200 import lib as L
from tests._oracle import OracleModel

pytestmark = pytest.mark.gpu
THREADS = max(1, os.cpu_count() or 1)


def _bits(a):
    return np.ascontiguousarray(a).view(np.uint32)


def test_greedy_stream_16_prompt_48_steps_full_shape(ctx):
    """16 random prompt ids, then 48 greedy steps (the reference's run loop, bonsai_forward.h:2752-2775,2890-2997): the
    picked ids must be identical and the final logits the same floats; recurrent state, conv taps and KV bytes of the
    first and last layers of each kind are compared exactly after the 64 tokens."""
    hp = synth.HParams(cap=128)
    tensors, signs = synth.make_model_repeated(hp, seed=0)
    gm = Model(ctx, hp, tensors, signs)
    om = OracleModel(hp, tensors, signs, threads=THREADS)
    rng = np.random.default_rng(42)
    prompt = [int(t) for t in rng.integers(0, hp.vocab, size=16)]
    gt = ot = None
    for pos, t in enumerate(prompt):
        gt = gm.token(t, pos)
        ol, _ = om.token(t, pos)
        ot = om.argmax(ol)
        if pos in (0, 15):
            assert np.array_equal(_bits(gm.logits()), _bits(ol)), f"prompt position {pos}: logits are not the same floats"
    assert gt == ot
    # the 48 decode steps run chained on the device (the production path of the benchmark), the oracle follows its own picks
    g_stream = [gt] + gm.decode(gt, 16, 48)
    o_stream, margins = [ot], []
    for i in range(48):
        ol, _ = om.token(o_stream[-1], 16 + i)
        o_stream.append(om.argmax(ol))
        top2 = np.partition(ol, -2)[-2:]
        margins.append(float(top2[1] - top2[0]))
    assert g_stream == o_stream, f"greedy streams diverge; smallest top-2 margin {min(margins):.3e}"
    assert np.array_equal(_bits(gm.logits()), _bits(ol)), "final logits are not bit-identical"
    n_gdn = sum(1 for b in range(hp.n_layer) if not hp.is_attn(b))
    for gi in (0, n_gdn - 1):
        gs = gm.read(L.READ_GDN_STATE, np.float32, hp.gdn_heads * hp.gdn_dim ** 2, gi)
        assert np.array_equal(_bits(gs), _bits(om.gdn_state(gi))), f"recurrent state of layer {gi} differs"
        ch = gm.read(L.READ_CONV_HIST, np.float32, hp.qkv_dim * 3, gi)
        assert np.array_equal(_bits(ch), _bits(om.conv_hist(gi))), f"conv taps of layer {gi} differ"
    fill = 64 * hp.n_kv * hp.head_dim
    for li in (0, hp.n_layer - n_gdn - 1):
        (kq, ks), (vq, vs) = om.kv(li)
        assert np.array_equal(gm.read(L.READ_K_DATA, np.int8, fill, li), kq[:fill])
        assert np.array_equal(gm.read(L.READ_V_DATA, np.int8, fill, li), vq[:fill])
        assert np.array_equal(gm.read(L.READ_K_SCALE, np.uint16, fill // 32, li), ks[: fill // 32])
        assert np.array_equal(gm.read(L.READ_V_SCALE, np.uint16, fill // 32, li), vs[: fill // 32])
    gm.close(); om.close()


def test_output_head_projection_and_multi_column(ctx, oracle):
    """The 248 320 x 4096 head: single-column streamed kernel and the 8- and 32-column tensor-core kernel against the
    oracle, every checked column the same floats."""
    from bonsai_vk_b200 import ptq
    M, K = 248320, 4096
    chunk = ptq.synth_matrix(np.random.default_rng(1), 16384, K)
    W = np.concatenate([chunk] * ((M + 16383) // 16384), axis=0)[:M]
    rng = np.random.default_rng(3)
    X = rng.standard_normal((32, K)).astype(np.float32)
    wb = ctx.from_numpy(W)
    xb = ctx.from_numpy(X[0])
    pack = ctx.alloc(ctx.act_pack_bytes(K))
    out = ctx.alloc(M * 4)
    ctx.act_quant_q81(xb, K, pack)
    ctx.gemv_q81(wb, M, K, pack, out)
    ctx.sync()
    ref0, exact0, _ = oracle.gemv_q81(W, M, K, oracle.quantize_q8_1(X[0]), threads=THREADS)
    got = out.download(np.float32, M)
    assert np.array_equal(_bits(got), _bits(ref0)), "head projection differs from the oracle"
    rms = float(np.sqrt(np.mean(exact0 ** 2)))
    assert np.max(np.abs(got - exact0) / np.maximum(np.abs(exact0), 0.05 * rms)) <= 1e-5
    Xb = ctx.from_numpy(X)
    for ncol in (8, 32):
        image = ctx.alloc(ctx.gemm_image_bytes(K, ncol))
        outs = ctx.alloc(ncol * M * 4)
        ctx.gemm_act_quant(Xb, K, ncol, image)
        ctx.gemm_q81(wb, M, K, image, ncol, outs)
        ctx.sync()
        cols = outs.download(np.float32, ncol * M).reshape(ncol, M)
        assert np.array_equal(_bits(cols[0]), _bits(ref0)), f"{ncol} columns: column 0 differs"
        c = ncol - 1
        refc, _, _ = oracle.gemv_q81(W, M, K, oracle.quantize_q8_1(X[c]), threads=THREADS)
        assert np.array_equal(_bits(cols[c]), _bits(refc)), f"{ncol} columns: column {c} differs"
        image.free(); outs.free()
    for b in (wb, xb, pack, out, Xb):
        b.free()


def test_recurrent_block_full_width_consecutive_positions(ctx):
    """One gated-delta-net block + FFN at the 9B widths (32 value heads / 16 key heads of 128, 8192 conv channels) over
    8 consecutive positions: from the second token on the state is non-zero and both conv-tap buffers (even / odd
    positions) have been read and written. Residual, state and taps compared exactly after every token."""
    hp = synth.HParams(n_layer=1, vocab=2048, cap=16)
    assert not hp.is_attn(0)
    tensors, signs = synth.make_model(hp, seed=7)
    gm = Model(ctx, hp, tensors, signs)
    om = OracleModel(hp, tensors, signs, threads=THREADS)
    for pos, t in enumerate([5, 1999, 42, 7, 1024, 3, 900, 11]):
        gm.token(t, pos, want_next=False)
        ol, ores = om.token(t, pos)
        assert np.array_equal(_bits(gm.residual()), _bits(ores)), f"position {pos}: residual differs"
        gs = gm.read(L.READ_GDN_STATE, np.float32, hp.gdn_heads * hp.gdn_dim ** 2, 0)
        assert np.array_equal(_bits(gs), _bits(om.gdn_state(0))), f"position {pos}: recurrent state differs"
        ch = gm.read(L.READ_CONV_HIST, np.float32, hp.qkv_dim * 3, 0)
        assert np.array_equal(_bits(ch), _bits(om.conv_hist(0))), f"position {pos}: conv taps differ"
        assert np.array_equal(_bits(gm.logits()), _bits(ol))
    gm.close(); om.close()
