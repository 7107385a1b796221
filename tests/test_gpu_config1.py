"""The ternary SwiGLU FFN block at its real shape: hidden 4096, FFN 12288 (gate/up/down as PTQ1_0), the input rotated by the
normalized Walsh-Hadamard transform at block 4096, the 12288-wide intermediate as 3 blocks of 4096 with its own sign
vector; batch 1 (GEMV path) and 16 tokens (tensor-core GEMM path). The FFN is exercised inside a one-block model of
the 9B's layer shape, so the recurrent mixer in front of it runs at its real shape too. Both paths must give the CPU
checker's floats bit for bit."""
import numpy as np
import pytest

from bonsai_vk_b200 import Model, synth
from bonsai_vk_b200 import lib as L
from tests._oracle import OracleModel

pytestmark = pytest.mark.gpu


def test_ffn_block_batch1_and_16_tokens(ctx):
    hp = synth.HParams(n_layer=1, vocab=2048, cap=32)
    tensors, signs = synth.make_model(hp, seed=3)
    om = OracleModel(hp, tensors, signs)
    toks = [int(t) for t in np.random.default_rng(1).integers(0, hp.vocab, size=16)]
    want_res, want_logits = [], []
    for t in toks:
        om.reset()
        lg, res = om.token(t, 0)
        want_res.append(res.copy()); want_logits.append(lg.copy())
    om.close()

    # batch 1: the streamed GEMV kernels
    m1 = Model(ctx, hp, tensors, signs)
    for i, t in enumerate(toks[:4]):
        m1.reset()
        m1.token(t, 0)
        assert np.array_equal(m1.residual().view(np.uint32), want_res[i].view(np.uint32)), f"token {i}: residual differs"
        assert np.array_equal(m1.logits().view(np.uint32), want_logits[i].view(np.uint32)), f"token {i}: logits differ"
    m1.close()

    # 16 tokens in one pass (16 independent sequences of one token each): the tcgen05 projection kernel
    hb = synth.HParams(n_layer=1, vocab=2048, cap=32, n_streams=16, batch_cols=16)
    mb = Model(ctx, hb, tensors, signs)
    out = ctx.alloc(16 * 4)
    mb.stage_prepare(0, 16)
    mb.stage_batch(0, toks, [0] * 16, None, out)
    ctx.sync()
    picks = out.download(np.int32, 16)
    assert [int(p) for p in picks] == [int(np.argmax(lg)) for lg in want_logits]
    # column 0's residual and logits are readable through the model's own views
    assert np.array_equal(mb.residual().view(np.uint32), want_res[0].view(np.uint32))
    assert np.array_equal(mb.logits().view(np.uint32), want_logits[0].view(np.uint32))
    mb.close()
    out.free()
