"""CPU checks of the block-level oracle: attention against the reference's own CPU mirror
(attn_vk.h, through the reference shim), Hadamard identities the reference tests, determinism."""
import ctypes as C

import numpy as np

from bonsai_vk_b200 import synth
from tests._oracle import OracleModel


def _p(a):
    return a.ctypes.data_as(C.c_void_p) if a is not None else None


def test_fwht_identities(oracle):
    """runtime_vk/shaders/hat4096.comp:13-18 and regression_v14.log:60-70: involution, sum identity
    sum(Hx) = sqrt(N) x[0], 1/sqrt(4096) == 1/64, and H matches the explicit Sylvester matrix."""
    rng = np.random.default_rng(0)
    for N in (16, 64, 128, 1024, 4096):
        x = rng.standard_normal(N).astype(np.float32)
        y = oracle.fwht(x, N)
        assert abs(float(y.astype(np.float64).sum()) - np.sqrt(N) * float(x[0])) < 1e-3
        back = oracle.fwht(y, N)
        assert np.max(np.abs(back - x)) < 1e-5
    N = 128
    H = np.array([[(-1) ** bin(i & j).count("1") for j in range(N)] for i in range(N)], dtype=np.float64) / np.sqrt(N)
    x = rng.standard_normal(N).astype(np.float32)
    assert np.max(np.abs(oracle.fwht(x, N) - H @ x)) < 1e-5
    assert np.allclose(H @ H.T, np.eye(N), atol=1e-12)
    e0 = np.zeros(4096, dtype=np.float32); e0[0] = 1.0
    assert np.all(oracle.fwht(e0, 4096) == np.float32(1.0 / 64.0))


def test_rotation_order(oracle):
    """forward = signs then H; embedding side = H then signs (bonsai_forward.h:471-476, 689-691)."""
    rng = np.random.default_rng(1)
    n = 1024
    x = rng.standard_normal(n).astype(np.float32)
    s = (rng.integers(0, 2, n) * 2 - 1).astype(np.int32)
    assert np.array_equal(oracle.rotate_fwd(x, s, n), oracle.fwht(x * s, n))
    assert np.array_equal(oracle.rotate_inv(x, s, n), oracle.fwht(x, n) * s)
    # 3 independent blocks for a 3*block wide vector
    x3 = rng.standard_normal(3 * n).astype(np.float32)
    s3 = (rng.integers(0, 2, 3 * n) * 2 - 1).astype(np.int32)
    y3 = oracle.rotate_fwd(x3, s3, n)
    for b in range(3):
        assert np.array_equal(y3[b * n:(b + 1) * n], oracle.fwht(x3[b * n:(b + 1) * n] * s3[b * n:(b + 1) * n], n))


def test_attention_vs_reference_mirror(oracle, ref):
    """fp16 K / fp16 V with fp16-rounded probabilities is the configuration attn_vk.h mirrors
    (attn_forward<true>). The oracle's attention must agree with it to float rounding: the two differ
    only in the summation order of the 256 squares of the head norm (tree here, serial there)."""
    hp = synth.tiny(k_mode=1, v_mode=1, cap=32, n_layer=4)
    tensors, signs = synth.make_model(hp, seed=3)
    om = OracleModel(hp, tensors, signs, attn_order=0)
    rng = np.random.default_rng(9)
    seq = 12
    QD, KD, hd = hp.n_head * hp.head_dim, hp.n_kv * hp.head_dim, hp.head_dim
    qg = rng.standard_normal((seq, hp.n_head, 2 * hd)).astype(np.float32)
    kin = rng.standard_normal((seq, KD)).astype(np.float32)
    vin = rng.standard_normal((seq, KD)).astype(np.float32)
    pos = np.arange(seq, dtype=np.int32)
    pre = np.empty(QD, dtype=np.float32); gated = np.empty(QD, dtype=np.float32)
    b = 3   # the attention block of the tiny model
    oracle.lib.bo_attn_insert_and_attend(om.m, b, 0, seq, _p(pos), _p(qg), _p(kin), _p(vin), _p(pre), _p(gated))
    # reference mirror takes q and gate de-interleaved
    q_in = np.ascontiguousarray(qg[:, :, :hd]).reshape(seq, QD)
    g_in = np.ascontiguousarray(qg[:, :, hd:]).reshape(seq, QD)
    r_pre = np.empty((seq, QD), dtype=np.float32); r_gated = np.empty((seq, QD), dtype=np.float32)
    qn = np.ascontiguousarray(tensors[f"blk.{b}.attn_q_norm.weight"]); kn = np.ascontiguousarray(tensors[f"blk.{b}.attn_k_norm.weight"])
    upos = pos.astype(np.uint32)
    ref.ref_attn_forward(seq, hp.cap, hp.n_head, hp.n_kv, hd, hp.n_rot, C.c_float(hp.rms_eps), C.c_float(hp.rope_base),
                         _p(q_in), _p(kin), _p(vin), _p(g_in), _p(qn), _p(kn), _p(upos), 1,
                         _p(r_pre), _p(r_gated), None, None, None)
    scale = np.sqrt(np.mean(r_pre[-1].astype(np.float64) ** 2))
    assert np.max(np.abs(pre - r_pre[-1])) <= 2e-3 * scale      # fp16 operand rounding can flip on a 1-ulp norm change
    assert np.median(np.abs(pre - r_pre[-1])) <= 1e-6 * scale
    assert np.max(np.abs(gated - r_gated[-1])) <= 2e-3 * scale
    om.close()


def test_oracle_token_is_deterministic_and_state_carries():
    hp = synth.tiny()
    tensors, signs = synth.make_model(hp, seed=2)
    om = OracleModel(hp, tensors, signs, threads=4)
    a0, _ = om.token(7, 0); a1, _ = om.token(9, 1)
    om.reset()
    b0, _ = om.token(7, 0); b1, _ = om.token(9, 1)
    assert np.array_equal(a0, b0) and np.array_equal(a1, b1)
    om.reset()
    c1, _ = om.token(9, 0)         # same token without history must differ (state and cache matter)
    assert not np.array_equal(a1, c1)
    assert np.any(om.gdn_state(0) != 0) and np.any(om.conv_hist(0) != 0)
    om.close()


def test_attention_orders_agree():
    """The reference's serial order and the regrouped order the CUDA kernels use are the same
    arithmetic: per-head outputs agree within 1e-5 relative (contexts 40 and 1500, q8_0 cache)."""
    for cap, seq, splits in ((64, 40, 1), (2048, 1500, 8)):
        hp = synth.tiny(cap=cap)
        tensors, signs = synth.make_model(hp, seed=4)
        om = OracleModel(hp, tensors, signs)
        rng = np.random.default_rng(seq)
        QD, KD, hd = hp.n_head * hp.head_dim, hp.n_kv * hp.head_dim, hp.head_dim
        qg = rng.standard_normal((seq, hp.n_head, 2 * hd)).astype(np.float32)
        kin = rng.standard_normal((seq, KD)).astype(np.float32)
        vin = rng.standard_normal((seq, KD)).astype(np.float32)
        pos = np.arange(seq, dtype=np.int32)
        outs = []
        for order in (0, 1):
            om.reset(); om.set_attn_order(order, splits)
            pre = np.empty(QD, dtype=np.float32); gated = np.empty(QD, dtype=np.float32)
            om.o.lib.bo_attn_insert_and_attend(om.m, 3, 0, seq, _p(pos), _p(qg), _p(kin), _p(vin), _p(pre), _p(gated))
            outs.append(pre.reshape(hp.n_head, hd).astype(np.float64))
        rms = np.sqrt(np.mean(outs[0] ** 2, axis=1, keepdims=True))
        # a probability within float rounding of an fp16 tie may round the other way: bound by one fp16 ulp of it
        assert np.max(np.abs(outs[0] - outs[1]) / rms) <= 5e-4
        assert np.median(np.abs(outs[0] - outs[1]) / rms) <= 1e-5
        om.close()


def test_explicit_layer_mask_equals_the_interval_rule():
    """A per-layer list that spells the interval pattern must run the same schedule (bonsai_model.h:136-148, 470-472)."""
    import dataclasses
    hp = synth.tiny()                                           # interval 4 over 4 blocks: R R R A
    tensors, signs = synth.make_model(hp, seed=2)
    listed = dataclasses.replace(hp, attn_interval=0, attn_mask=0b1000)
    assert [listed.is_attn(b) for b in range(4)] == [hp.is_attn(b) for b in range(4)]
    a, b = OracleModel(hp, tensors, signs, threads=4), OracleModel(listed, tensors, signs, threads=4)
    for pos, t in enumerate([5, 1000, 42]):
        la, _ = a.token(t, pos)
        lb, _ = b.token(t, pos)
        assert np.array_equal(la.view(np.uint32), lb.view(np.uint32))
    a.close(); b.close()
