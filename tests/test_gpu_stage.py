"""Pipeline stages and multiple streams on ONE GPU: two stage models (blocks [0,2) and [2,4)) chained through
device buffers reproduce the whole model's greedy stream for every sequence, with interleaved sequences (each
keeps its own KV cache, recurrent state and conv taps)."""
import numpy as np
import pytest

from bonsai_vk_b200 import Model, synth

pytestmark = pytest.mark.gpu


def test_two_stages_three_streams_match_whole_model(ctx):
    base = dict(seed=7)
    hp = synth.tiny()
    tensors, signs = synth.make_model(hp, **base)
    whole = Model(ctx, hp, tensors, signs)
    S, T = 3, 10
    first = [5, 77, 1234]
    want = []
    for s in range(S):
        whole.reset()
        tok, row = first[s], []
        for pos in range(T):
            tok = whole.token(tok, pos)
            row.append(tok)
        want.append(row)
    whole.close()

    hp_a = synth.tiny(n_streams=S, block_begin=0, block_end=2)
    hp_b = synth.tiny(n_streams=S, block_begin=2, block_end=4)
    a = Model(ctx, hp_a, tensors, signs)
    b = Model(ctx, hp_b, tensors, signs)
    hid = [ctx.alloc(hp.hidden * 4) for _ in range(S)]
    tokb = [ctx.alloc(16) for _ in range(S)]
    got = [[] for _ in range(S)]
    for pos in range(T):
        for s in range(S):                     # sequences interleaved, as the pipeline runs them
            if pos == 0:
                a.stage(s, first[s], pos, None, hid[s])
            else:
                a.stage(s, -1, pos, tokb[s], hid[s])      # token id read from the device buffer
            b.stage(s, 0, pos, hid[s], tokb[s])
        ctx.sync()
        for s in range(S):
            got[s].append(int(tokb[s].download(np.int32, 1)[0]))
    assert got == want
    a.close(); b.close()
    for x in hid + tokb:
        x.free()
