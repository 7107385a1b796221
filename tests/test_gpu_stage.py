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
    from bonsai_vk_b200 import BonsaiError
    with pytest.raises(BonsaiError, match="not prepared"):          # a stage never builds its schedule on the fly
        a.stage(0, first[0], 0, None, hid[0])
    for s in range(S):
        a.stage_prepare(s); b.stage_prepare(s)
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


def test_batched_stages_match_whole_model(ctx):
    """The multi-sequence pass (tensor-core projections, one grid slice per sequence elsewhere): two stages, six
    sequences run as micro-batches of 4 + 2 at different positions per sequence, against the whole model run one
    sequence at a time. Streams AND final state must be identical: the batched pass computes every column in the
    single-sequence operation order."""
    from bonsai_vk_b200 import lib as L
    hp = synth.tiny()
    tensors, signs = synth.make_model(hp, seed=7)
    S, T = 6, 9
    first = [5, 77, 1234, 900, 3, 2000]
    lag = [0, 1, 0, 2, 1, 0]                     # sequence s starts at step lag[s]: positions differ inside a micro-batch
    whole = Model(ctx, hp, tensors, signs)
    want, want_state = [], []
    for s in range(S):
        whole.reset()
        tok, row = first[s], []
        for pos in range(T - lag[s]):
            tok = whole.token(tok, pos)
            row.append(tok)
        want.append(row)
        want_state.append(whole.read(L.READ_GDN_STATE, np.float32, hp.gdn_heads * hp.gdn_dim ** 2, 0).copy())
    whole.close()

    a = Model(ctx, synth.tiny(n_streams=S, block_begin=0, block_end=2, batch_cols=4), tensors, signs)
    b = Model(ctx, synth.tiny(n_streams=S, block_begin=2, block_end=4, batch_cols=4), tensors, signs)
    hid, tokb = ctx.alloc(S * hp.hidden * 4), ctx.alloc(S * 4)
    from bonsai_vk_b200 import BonsaiError
    with pytest.raises(BonsaiError, match="not prepared"):
        a.stage_batch(0, first[:4], [0] * 4, None, hid)
    for r0 in range(S):                          # every run of consecutive sequences the loop below may form
        for n in range(1, 5):
            if r0 + n <= S:
                a.stage_prepare(r0, n); b.stage_prepare(r0, n)
    got = [[] for _ in range(S)]
    cur = list(first)
    groups = [(0, 4), (4, 2)]
    for step in range(T):
        for s0, n in groups:
            live = [s for s in range(s0, s0 + n) if step >= lag[s]]
            if not live:
                continue
            # a micro-batch is a run of consecutive sequences: here all of a group are live from step 2 on; before that
            # the live ones are run in consecutive sub-runs
            runs, run = [], [live[0]]
            for s in live[1:]:
                if s == run[-1] + 1:
                    run.append(s)
                else:
                    runs.append(run); run = [s]
            runs.append(run)
            for run in runs:
                r0, pos = run[0], [step - lag[s] for s in run]
                a.stage_batch(r0, [cur[s] for s in run], pos, None, hid, out_off=r0 * hp.hidden * 4)
                b.stage_batch(r0, None, pos, hid, tokb, in_off=r0 * hp.hidden * 4, out_off=r0 * 4)
        ctx.sync()
        picks = tokb.download(np.int32, S)
        for s in range(S):
            if step >= lag[s]:
                cur[s] = int(picks[s])
                got[s].append(cur[s])
    assert got == want
    # recurrent state of the first GDN layer (stage a holds it) of the sequence the last call started with
    st4 = a.read(L.READ_GDN_STATE, np.float32, hp.gdn_heads * hp.gdn_dim ** 2, 0)
    assert np.array_equal(st4.view(np.uint32), want_state[4].view(np.uint32))
    a.close(); b.close()
    hid.free(); tokb.free()


def test_token_id_from_device_memory_is_checked(ctx):
    """The first stage reads the next token id from device memory (the message of the last stage). An id outside the
    vocabulary must not be turned into an address: id 0 is used, the next sync reports it, and the context stays usable."""
    from bonsai_vk_b200 import BonsaiError
    hp = synth.tiny(n_streams=1, block_begin=0, block_end=2)
    tensors, signs = synth.make_model(hp, seed=7)
    a = Model(ctx, hp, tensors, signs)
    a.stage_prepare(0)
    hid, hid0 = ctx.alloc(hp.hidden * 4), ctx.alloc(hp.hidden * 4)
    bad = ctx.from_numpy(np.array([hp.vocab + 12345, 0, 0, 0], dtype=np.int32))
    a.stage(0, -1, 0, bad, hid)
    with pytest.raises(BonsaiError, match="outside the vocabulary"):
        ctx.sync()
    a.reset()
    a.stage(0, 0, 0, None, hid0)              # what the refused step computed instead: token id 0
    ctx.sync()
    assert np.array_equal(hid.download(np.uint32, hp.hidden), hid0.download(np.uint32, hp.hidden))
    a.close()
    for x in (hid, hid0, bad):
        x.free()


def test_output_head_sharded_over_the_stages(ctx):
    """Two stages, each holding half of the output head's rows: the last stage hands the final hidden state to both,
    every stage gives its shard's (value, row) candidates, and the pick over the shards must be the token the whole
    model picks (first maximum). Four sequences in one pass, eight steps; also the refusals around the mode."""
    from bonsai_vk_b200 import BonsaiError
    hp = synth.tiny()
    tensors, signs = synth.make_model(hp, seed=11)
    S, T = 4, 8
    first = [9, 1500, 321, 77]
    whole = Model(ctx, hp, tensors, signs)
    want = []
    for s in range(S):
        whole.reset()
        tok, row = first[s], []
        for pos in range(T):
            tok = whole.token(tok, pos)
            row.append(tok)
        want.append(row)
    whole.close()
    half = hp.vocab // 2
    assert half % 128 == 0
    a = Model(ctx, synth.tiny(n_streams=S, block_begin=0, block_end=2, batch_cols=4), tensors, signs, head_rows=(0, half))
    b = Model(ctx, synth.tiny(n_streams=S, block_begin=2, block_end=4, batch_cols=4), tensors, signs, head_rows=(half, hp.vocab))
    with pytest.raises(BonsaiError, match="128-row"):
        Model(ctx, synth.tiny(n_streams=S, batch_cols=4), tensors, signs, head_rows=(64, hp.vocab))
    a.stage_prepare(0, S); b.stage_prepare(0, S)
    hid, fin = ctx.alloc(S * hp.hidden * 4), ctx.alloc(S * hp.hidden * 4)
    cands, tokb = ctx.alloc(2 * S * 8), ctx.alloc(S * 4)
    with pytest.raises(BonsaiError, match="sharded output head"):
        a.stage(0, 1, 0, None, hid)
    got = [[] for _ in range(S)]
    for step in range(T):
        a.stage_batch(0, first if step == 0 else None, [step] * S, None if step == 0 else tokb, hid)
        b.stage_batch(0, None, [step] * S, hid, fin)          # last stage: hidden state out, not picks
        a.head_batch(S, fin, cands, out_off=0)
        b.head_batch(S, fin, cands, out_off=S * 8)
        a.pick_batch(S, 2, cands, tokb)
        ctx.sync()
        picks = tokb.download(np.int32, S)
        for s in range(S):
            got[s].append(int(picks[s]))
    assert got == want
    # the candidates of the last step: each shard's row lies in its own range, and one of them is the pick
    c = cands.download(np.int32, 2 * S * 2).reshape(2, S, 2)
    assert np.all((c[0, :, 1] >= 0) & (c[0, :, 1] < half)) and np.all((c[1, :, 1] >= half) & (c[1, :, 1] < hp.vocab))
    a.close(); b.close()
    for x in (hid, fin, cands, tokb):
        x.free()
