"""Failure detection on the device without a fault: a bounded wait that nothing satisfies must give up, set the
context's error word, and leave the context usable (no trap, no hang, no lost context)."""
import numpy as np
import pytest

from bonsai_vk_b200 import ptq
from bonsai_vk_b200.lib import BonsaiError

pytestmark = pytest.mark.gpu


@pytest.mark.parametrize("which,where", [(0, "copy ring"), (1, "tensor-core projection pipeline")])
def test_bounded_wait_gives_up_and_context_survives(ctx, oracle, which, where):
    ctx.sync()                                    # nothing pending, no stale error
    ctx.selftest_wait(which)
    with pytest.raises(BonsaiError) as ei:
        ctx.sync()
    assert "(-5)" in str(ei.value) and where in str(ei.value)      # BN_ERR_TIMEOUT, naming the wait that gave up
    ctx.sync()                                    # the error word was cleared: the next sync is clean
    # and the context still computes: a projection after the failed wait is bit-identical to the oracle
    M, K = 256, 1024
    rng = np.random.default_rng(3 + which)
    W = ptq.synth_matrix(rng, M, K)
    x = rng.standard_normal(K).astype(np.float32)
    xq = oracle.quantize_q8_1(x)
    wb, xb, out = ctx.from_numpy(W), ctx.from_numpy(x), ctx.alloc(M * 4)
    pack = ctx.alloc(ctx.act_pack_bytes(K))
    ctx.act_quant_q81(xb, K, pack)
    ctx.gemv_q81(wb, M, K, pack, out)
    ctx.sync()
    ref, _, _ = oracle.gemv_q81(W, M, K, xq, want_dots=True)
    assert np.array_equal(out.download(np.float32, M).view(np.uint32), ref.view(np.uint32))
    for b in (wb, xb, pack, out):
        b.free()
