"""One GQA decode-attention layer (16 query / 4 KV heads - and 8, 2 or 1 query heads per KV head -, head_dim 256, rope theta 1e7 on the first 64 dims, cache
filled from N(0,1) rows) at contexts 4096 and 32768, through the op-level C ABI: q8_0 K and V, and the reference's
own cache layout (fp16 K with q8_0 V, runtime_vk/shaders/attn_norm_rope2.comp:26-49; fp16 K and V, attn_vk.h).
Checked against the CPU oracle on the same rows: cache bytes (q8_0 codes, fp16 words) and per-head outputs.
The oracle runs its sums in the kernels' grouping, so outputs are expected to be the same floats; the 1e-5 bound is
asserted too. (How far that grouping is from the reference's serial order - whose oracle form is bit-identical to
attn_vk.h - is measured in tests/test_oracle_model.py: worst element 1e-4 of the row RMS, worst row 3e-5.)"""
import ctypes as C

import numpy as np
import pytest

from bonsai_vk_b200 import synth
from bonsai_vk_b200 import lib as L
from tests._oracle import OracleModel

pytestmark = pytest.mark.gpu


def _p(a):
    return a.ctypes.data_as(C.c_void_p)


@pytest.mark.parametrize("ctx_len,k_mode,v_mode,heads", [(300, 0, 0, (16, 4)), (4096, 0, 0, (16, 4)), (32768, 0, 0, (16, 4)), (300, 1, 0, (16, 4)),
                                                         (4096, 1, 0, (16, 4)), (4096, 1, 1, (16, 4)),
                                                         # other numbers of query heads per kv head (8, 2, 1): the general scores kernel
                                                         (1500, 0, 0, (8, 1)), (1500, 1, 0, (8, 4)), (777, 0, 0, (4, 4)), (777, 1, 1, (8, 1))])
def test_decode_attention_layer(ctx, ctx_len, k_mode, v_mode, heads):
    n_head, n_kv, hd = heads[0], heads[1], 256
    QD, KD = n_head * hd, n_kv * hd
    rng = np.random.default_rng(ctx_len)
    k_rows = rng.standard_normal((ctx_len, KD)).astype(np.float32)
    v_rows = rng.standard_normal((ctx_len, KD)).astype(np.float32)
    qg = rng.standard_normal((n_head, 2 * hd)).astype(np.float32)
    qn = (1.0 + 0.1 * rng.standard_normal(hd)).astype(np.float32)
    kn = (1.0 + 0.1 * rng.standard_normal(hd)).astype(np.float32)

    dims = L.AttnDimsC(n_head=n_head, n_kv=n_kv, head_dim=hd, n_rot=64, cap=ctx_len + (ctx_len & 1), k_mode=k_mode, v_mode=v_mode,
                       rms_eps=1e-6, rope_base=1e7)
    kvb, scb = ctx.attn_sizes(dims)
    kv, scratch = ctx.alloc(kvb), ctx.alloc(scb)
    kv.memset(0)
    bk, bv, bq, bqn, bkn = (ctx.from_numpy(x) for x in (k_rows, v_rows, qg, qn, kn))
    pre, gated = ctx.alloc(QD * 4), ctx.alloc(QD * 4)
    ctx.attn_insert(dims, kv, bk, bv, ctx_len, 0, bq, bqn, bkn, scratch)
    ctx.attn_attend(dims, kv, ctx_len - 1, scratch, pre, gated)
    ctx.sync()
    g_pre = pre.download(np.float32, QD).reshape(n_head, hd)
    g_gated = gated.download(np.float32, QD).reshape(n_head, hd)
    n = ctx_len * KD
    g_kcodes = kv.download(np.int8, n) if k_mode == 0 else kv.download(np.uint16, n)

    # oracle: a model shell that only carries this layer's norm weights
    hp = synth.HParams(n_layer=4, hidden=n_head * hd, n_head=n_head, n_kv=n_kv, cap=dims.cap, vocab=128, k_mode=k_mode, v_mode=v_mode)
    om = OracleModel(hp, {"blk.3.attn_q_norm.weight": qn, "blk.3.attn_k_norm.weight": kn}, np.ones(4, dtype=np.int32))
    o_pre = np.empty(QD, dtype=np.float32); o_gated = np.empty(QD, dtype=np.float32)
    om.o.lib.bo_attn_fill_and_attend(om.m, 3, 0, ctx_len, _p(qg), _p(k_rows), _p(v_rows), _p(o_pre), _p(o_gated))
    (kq, ks), (vq, vs) = om.kv(0)
    assert np.array_equal(g_kcodes, kq[:n]), "cached K (q8_0 codes or fp16 words) differs"
    o_pre = o_pre.reshape(n_head, hd); o_gated = o_gated.reshape(n_head, hd)
    rms = np.sqrt(np.mean(o_pre.astype(np.float64) ** 2, axis=1, keepdims=True))
    assert np.max(np.abs(g_pre - o_pre) / rms) <= 1e-5
    assert np.max(np.abs(g_gated - o_gated) / rms) <= 1e-5
    assert np.array_equal(g_pre.view(np.uint32), o_pre.view(np.uint32)), "per-head outputs are not the same floats"
    om.close()
    for b in (kv, scratch, bk, bv, bq, bqn, bkn, pre, gated):
        b.free()
