"""The /v1 server and its multi-conversation scheduler (reference: runtime_vk/bonsai_http.h:514-737 routes and reply
shapes, :549-556 the one-at-a-time try-lock this replaces, :592-623 per-request reset). CPU: the scheduler against a
stand-in engine and the HTTP layer over it. GPU: three overlapping conversations on the tiny model against the whole
model's own single-sequence decode."""
import json
import threading
import urllib.error
import urllib.request

import numpy as np
import pytest

from bonsai_vk_b200 import server, synth


class FakeEngine:
    """next token = a fixed function of (token, position); remembers resets and what every pass was fed."""
    slots, group, cap, vocab = 4, 2, 32, 1000

    def __init__(self):
        self.resets, self.passes = [], []

    def reset_slot(self, s):
        self.resets.append(s)

    def step(self, g, toks, pos):
        self.passes.append((g, list(toks), list(pos)))
        return [(7 * t + 3 * p + 1) % self.vocab for t, p in zip(toks, pos)]


def _serial(prompt, n, stop=()):
    tok, out = None, []
    seq = list(prompt)
    for p in range(len(prompt) + n - 1):
        t = seq[p]
        nxt = (7 * t + 3 * p + 1) % 1000
        if p >= len(prompt) - 1:
            out.append(nxt); seq.append(nxt)
            if nxt in stop or len(out) == n:
                break
    return out


def _drain(c):
    while True:
        k, v = c.events.get(timeout=10)
        if k == "end":
            return v


def test_scheduler_continuous_batching():
    e = FakeEngine()
    b = server.Batcher(e)
    a = b.submit([5, 6, 7], 6)
    c = b.submit([9], 4)                       # joins while a is running
    fa, fc = _drain(a), _drain(c)
    assert a.out == _serial([5, 6, 7], 6) and c.out == _serial([9], 4)
    assert fa == fc == "length"
    assert a.slot // e.group == c.slot // e.group, "the second conversation should fill the group that is already running"
    assert sorted(e.resets) == sorted([a.slot, c.slot])
    # every pass covers a whole group; idle columns carry the dummy token at position 0
    assert all(len(t) == e.group for _, t, _ in e.passes)
    # a stop id ends the conversation with finish "stop"
    want = _serial([5, 6, 7], 6)
    d = b.submit([5, 6, 7], 6, stop=[want[2]])
    assert _drain(d) == "stop" and d.out == want[:3]
    b.close()


def test_scheduler_samples_on_the_host_when_asked():
    """A conversation with a sampler picks from its own column's logits over its own generation; its neighbour in the
    same group keeps the engine's greedy pick."""
    from bonsai_vk_b200.sampler import Sampler

    class LogitEngine(FakeEngine):
        def step(self, g, toks, pos):
            self.last = (g, list(toks), list(pos))
            return super().step(g, toks, pos)

        def logits(self, g, i):                       # a peak at the greedy pick, a second one ten ids further
            gg, toks, pos = self.last
            assert gg == g
            lg = np.full(self.vocab, -30.0, dtype=np.float32)
            top = (7 * toks[i] + 3 * pos[i] + 1) % self.vocab
            lg[top] = 5.0
            lg[(top + 10) % self.vocab] = 4.5
            return lg

    e = LogitEngine()
    b = server.Batcher(e)
    greedy = b.submit([5, 6, 7], 6)
    argmax = b.submit([5, 6, 7], 6, sampler=Sampler(temp=1.0, top_k=1, rep_penalty=1.0, presence_penalty=0.0))
    mixed = b.submit([5, 6, 7], 200, sampler=Sampler(temp=1.0, rep_penalty=1.0, presence_penalty=0.0, seed=11))
    for c in (greedy, argmax, mixed):
        _drain(c)
    assert greedy.out == _serial([5, 6, 7], 6)
    assert argmax.out == greedy.out                   # top_k = 1 leaves only the maximum
    # the sampled conversation follows its own tokens: every step is one of the two peaks of the token it fed
    seq = [5, 6, 7] + mixed.out
    seconds = 0
    for p in range(2, len(seq) - 1):
        top = (7 * seq[p] + 3 * p + 1) % 1000
        assert seq[p + 1] in (top, (top + 10) % 1000)
        seconds += seq[p + 1] != top
    assert 0 < seconds < len(mixed.out)               # both peaks are drawn (weights 0.62 : 0.38)
    b.close()


def test_scheduler_refuses_when_full_and_checks_requests():
    e = FakeEngine()
    gate = threading.Event()
    orig = e.step
    e.step = lambda g, t, p: (gate.wait(10), orig(g, t, p))[1]      # hold the engine so that the slots stay taken
    b = server.Batcher(e)
    held = [b.submit([1, 2], 3) for _ in range(e.slots)]
    with pytest.raises(server.Busy):
        b.submit([1], 1)
    with pytest.raises(ValueError):
        b.submit([], 1)
    with pytest.raises(ValueError):
        b.submit([e.vocab], 1)
    with pytest.raises(ValueError):
        b.submit(list(range(e.cap)), 1)
    gate.set()
    for c in held:
        assert _drain(c) == "length" and c.out == _serial([1, 2], 3)
    assert b.busy_slots() == 0
    b.close()


def _http(port, path, body=None, method=None):
    req = urllib.request.Request(f"http://127.0.0.1:{port}{path}", data=None if body is None else json.dumps(body).encode(),
                                 method=method or ("POST" if body is not None else "GET"), headers={"Content-Type": "application/json"})
    try:
        with urllib.request.urlopen(req, timeout=20) as r:
            return r.status, r.read()
    except urllib.error.HTTPError as ex:
        return ex.code, ex.read()


def test_http_routes_and_reply_shapes():
    b = server.Batcher(FakeEngine())
    srv = server.serve(b, "fake", port=0)
    port = srv.server_address[1]
    st, raw = _http(port, "/health")
    assert st == 200 and json.loads(raw)["slots"] == 4
    st, raw = _http(port, "/v1/models")
    assert st == 200 and json.loads(raw)["data"][0]["id"] == "fake"
    st, raw = _http(port, "/v1/completions", {"prompt": [5, 6, 7], "max_tokens": 4})
    out = json.loads(raw)
    assert st == 200 and out["choices"][0]["token_ids"] == _serial([5, 6, 7], 4) and out["usage"]["completion_tokens"] == 4
    st, raw = _http(port, "/v1/chat/completions", {"prompt_ids": [9], "max_tokens": 3})
    out = json.loads(raw)
    assert st == 200 and out["object"] == "chat.completion" and out["choices"][0]["token_ids"] == _serial([9], 3)
    assert out["choices"][0]["message"]["role"] == "assistant" and out["choices"][0]["finish_reason"] == "length"
    # server-sent events
    st, raw = _http(port, "/v1/chat/completions", {"prompt_ids": [9], "max_tokens": 3, "stream": True})
    events = [json.loads(l[6:]) for l in raw.decode().split("\n\n") if l.startswith("data: {")]
    assert st == 200 and raw.decode().rstrip().endswith("data: [DONE]")
    assert [ev["choices"][0]["delta"]["token_id"] for ev in events[:-1]] == _serial([9], 3)
    assert events[-1]["choices"][0]["finish_reason"] == "length" and events[-1]["usage"]["prompt_tokens"] == 1
    # refusals: text without ids, bad json, wrong method, unknown path, ids outside the vocabulary
    st, raw = _http(port, "/v1/chat/completions", {"messages": [{"role": "user", "content": "hi"}]})
    assert st == 400 and "no tokenizer" in json.loads(raw)["error"]["message"]
    assert _http(port, "/v1/chat/completions", method="GET")[0] == 405
    assert _http(port, "/v1/nothing")[0] == 404
    st, raw = _http(port, "/v1/completions", {"prompt": [100000]})
    assert st == 400 and json.loads(raw)["error"]["type"] == "invalid_request_error"
    req = urllib.request.Request(f"http://127.0.0.1:{port}/health", headers={"Host": "example.com"})
    with pytest.raises(urllib.error.HTTPError) as ei:
        urllib.request.urlopen(req, timeout=10)
    assert ei.value.code == 400
    srv.shutdown(); b.close()


def test_gguf_reader_round_trip(tmp_path):
    from bonsai_vk_b200 import gguf_reader, gguf_writer
    hp = synth.tiny()
    p = str(tmp_path / "m.gguf")
    gguf_writer.write(p, hp, seed=2)
    hp2, tensors, signs = gguf_reader.load(p, cap=hp.cap)
    want, wsigns = synth.make_model(hp, seed=2)
    assert (hp2.n_layer, hp2.hidden, hp2.ffn, hp2.vocab, hp2.attn_interval, hp2.hat_block) == (hp.n_layer, hp.hidden, hp.ffn, hp.vocab, hp.attn_interval, hp.hat_block)
    assert np.array_equal(signs, wsigns) and set(tensors) == set(want)
    for n in want:
        assert np.array_equal(np.asarray(tensors[n]).reshape(-1).view(np.uint8), np.ascontiguousarray(want[n]).reshape(-1).view(np.uint8)), n


@pytest.mark.gpu
def test_three_overlapping_conversations_on_the_gpu(ctx):
    from bonsai_vk_b200 import Model
    hp = synth.tiny()
    tensors, signs = synth.make_model(hp, seed=4)
    prompts = [[3, 77, 1500, 12], [900], [41, 7, 2047, 5, 6, 8, 10]]
    n_gen = [9, 12, 5]
    whole = Model(ctx, hp, tensors, signs)
    want = []
    for pr, n in zip(prompts, n_gen):
        whole.reset()
        for pos, t in enumerate(pr):
            tok = whole.token(t, pos)
        row = [tok]
        for i in range(n - 1):
            tok = whole.token(tok, len(pr) + i)
            row.append(tok)
        want.append(row)
    whole.close()
    eng = server.GpuEngine(ctx, hp, tensors, signs, slots=4, group=4)
    b = server.Batcher(eng)
    srv = server.serve(b, "tiny", port=0)
    port = srv.server_address[1]
    got = [None] * 3

    def ask(i):
        st, raw = _http(port, "/v1/completions", {"prompt": prompts[i], "max_tokens": n_gen[i]})
        got[i] = (st, json.loads(raw))

    th = [threading.Thread(target=ask, args=(i,)) for i in range(3)]
    for t in th:
        t.start()
    for t in th:
        t.join(60)
    for i in range(3):
        assert got[i][0] == 200 and got[i][1]["choices"][0]["token_ids"] == want[i], i
    # a slot that served one conversation serves the next from a clean state
    st, raw = _http(port, "/v1/completions", {"prompt": prompts[0], "max_tokens": n_gen[0]})
    assert json.loads(raw)["choices"][0]["token_ids"] == want[0]
    # a request that samples reads its column's logits on the host; with top_k = 1 and the penalties off only the
    # maximum survives, so the stream must be the greedy one (whatever column the conversation landed in)
    st, raw = _http(port, "/v1/completions", {"prompt": prompts[2], "max_tokens": n_gen[2], "temperature": 0.8, "top_k": 1,
                                              "repetition_penalty": 1.0, "presence_penalty": 0.0})
    assert st == 200 and json.loads(raw)["choices"][0]["token_ids"] == want[2]
    srv.shutdown(); b.close(); eng.close()


def test_full_size_writer_mode_reuses_tensors(tmp_path):
    """gguf_writer's repeat mode (one generated tensor per kind for every block): same header, shapes and byte counts as
    the plain mode, readable by the Python reader; blocks of the same kind hold the same bytes."""
    from bonsai_vk_b200 import gguf_reader, gguf_writer
    hp = synth.tiny()
    a, b = str(tmp_path / "plain.gguf"), str(tmp_path / "rep.gguf")
    ra, rb = gguf_writer.write(a, hp, seed=2), gguf_writer.write(b, hp, seed=2, repeat=True)
    assert ra == rb
    hp2, tensors, _ = gguf_reader.load(b, cap=hp.cap)
    assert hp2.n_layer == hp.n_layer and len(tensors) == ra["tensors"]
    assert np.array_equal(np.asarray(tensors["blk.0.ffn_up.weight"]), np.asarray(tensors["blk.1.ffn_up.weight"]))
    assert np.array_equal(np.asarray(tensors["token_embd.weight"]), np.asarray(tensors["output.weight"]))
