"""The `/v1` server with a multi-conversation scheduler.

Reference behaviour (runtime_vk/bonsai_http.h): GET /v1/models, GET /v1/status and /health, POST
/v1/chat/completions with server-sent events when "stream" is true (:514-737), OpenAI-shaped error bodies, loopback
Host names only (:139), and ONE conversation at a time behind a try-lock that answers 429 while the GPU is busy
(:549-556), every request resetting the engine's state first (:592-623).

What changes here: the try-lock becomes continuous batching. The model is created for S sequences ("slots") that
run as fixed groups of G consecutive sequences through bn_model_stage_batch - one pass per group and step reads every
projection's weights once for all G - and a request takes a free slot (its recurrent state and cache are cleared,
bn_model_reset_stream), joins the running group at the next step, feeds its prompt one token per step and then its
own picks, and leaves when it hits a stop id, max_tokens or the context capacity. Slots without a conversation run a
dummy token at position 0 (a pass costs the same whatever the number of live columns). 429 is kept for the case the
reference uses it for - no capacity left - which is now S conversations instead of one.

Sampling: a request that asks for a temperature above zero (fields as the reference reads them, bonsai_http.h:595-608:
temperature, top_p, top_k, seed, repetition_penalty, presence_penalty, frequency_penalty) is sampled on the host from its
column's logits with the reference's sampler arithmetic (sampler.py); every other request takes the device's greedy pick.

The tokenizer and the chat template stay on the reference's side of the boundary (its Bpe / chat::render produce ids):
requests carry token ids - "prompt": [ids] on /v1/completions (the token-array form of that API) or "prompt_ids" on
/v1/chat/completions - and replies carry "token_ids" beside a text field that lists the ids. A text-only request is
answered 400 with that explanation.

  python -m bonsai_vk_b200.server --gguf model.gguf [--port 8080] [--slots 64] [--group 32] [--cap 8192]
"""
from __future__ import annotations

import json
import queue
import threading
import time
from http.server import BaseHTTPRequestHandler, ThreadingHTTPServer
from typing import List, Optional

from .sampler import sampler_from_request


class Busy(Exception):
    """Every slot holds a conversation."""


class Conversation:
    def __init__(self, prompt: List[int], max_tokens: int, stop: set, sampler=None):
        self.prompt, self.max_tokens, self.stop = list(prompt), int(max_tokens), set(stop)
        self.sampler = sampler             # None: the device's greedy pick; else sampler.Sampler over the step's logits
        self.pos = 0                       # position of the token fed at the next step
        self.out: List[int] = []
        self.events: "queue.Queue" = queue.Queue()     # ("tok", id) ... ("end", finish_reason)
        self.finish: Optional[str] = None
        self.slot = -1

    def next_feed(self) -> int:
        return self.prompt[self.pos] if self.pos < len(self.prompt) else self.out[self.pos - len(self.prompt)]


class Batcher:
    """Continuous batching over an engine with `slots` sequences in groups of `group`:
    engine.step(g, toks, pos) -> picks (one per column of group g), engine.reset_slot(s), engine.cap, engine.vocab, and -
    only for conversations that sample - engine.logits(g, i): the logits of column i after the last step of group g."""

    def __init__(self, engine):
        self.e = engine
        self.S, self.G = engine.slots, engine.group
        assert self.S % self.G == 0
        self.conv: List[Optional[Conversation]] = [None] * self.S
        self.lock = threading.Condition()
        self.stop_flag = False
        self.steps = 0
        self.served = 0
        self.thread = threading.Thread(target=self._loop, daemon=True)
        self.thread.start()

    def busy_slots(self) -> int:
        with self.lock:
            return sum(c is not None for c in self.conv)

    def submit(self, prompt: List[int], max_tokens: int, stop=(), sampler=None) -> Conversation:
        if not prompt:
            raise ValueError("the prompt holds no token id")
        if any((not isinstance(t, int)) or t < 0 or t >= self.e.vocab for t in prompt):
            raise ValueError(f"prompt ids must be integers in [0, {self.e.vocab})")
        if len(prompt) >= self.e.cap:
            raise ValueError(f"the prompt ({len(prompt)} tokens) does not fit the context capacity {self.e.cap}")
        c = Conversation(prompt, max(1, max_tokens), stop, sampler)
        with self.lock:
            free = [s for s in range(self.S) if self.conv[s] is None]
            if not free:
                raise Busy()
            # fill the groups that are already running first: a pass costs the same with one live column or G
            live_groups = {s // self.G for s in range(self.S) if self.conv[s] is not None}
            free.sort(key=lambda s: (s // self.G not in live_groups, s))
            c.slot = free[0]
            self.e.reset_slot(c.slot)
            self.conv[c.slot] = c
            self.lock.notify_all()
        return c

    def _loop(self):
        while True:
            with self.lock:
                while not self.stop_flag and all(c is None for c in self.conv):
                    self.lock.wait()
                if self.stop_flag:
                    return
                plan = []
                for g in range(self.S // self.G):
                    cs = self.conv[g * self.G:(g + 1) * self.G]
                    if any(c is not None for c in cs):
                        plan.append((g, cs, [c.next_feed() if c else 0 for c in cs], [c.pos if c else 0 for c in cs]))
            for g, cs, toks, pos in plan:
                picks = self.e.step(g, toks, pos)
                for i, c in enumerate(cs):
                    if c is None:
                        continue
                    c.pos += 1
                    if c.pos < len(c.prompt):
                        continue                                  # still feeding the prompt: the pick is not used
                    # a sampling conversation reads its column's logits and picks on the host over its own generation so
                    # far, as the reference does (bonsai_forward.h:2892); everybody else takes the device's first maximum
                    t = int(c.sampler.pick(self.e.logits(g, i), c.out)) if c.sampler is not None else int(picks[i])
                    c.out.append(t)
                    c.events.put(("tok", t))
                    if t in c.stop:
                        c.finish = "stop"
                    elif len(c.out) >= c.max_tokens or c.pos >= self.e.cap - 1:
                        c.finish = "length"
                    if c.finish:
                        c.events.put(("end", c.finish))
                        with self.lock:
                            self.conv[c.slot] = None
                            self.served += 1
            self.steps += 1

    def close(self):
        with self.lock:
            self.stop_flag = True
            self.lock.notify_all()
        self.thread.join(timeout=10)


class GpuEngine:
    """The whole model on one GPU for `slots` sequences in groups of `group` (bn_model_stage_batch)."""

    def __init__(self, ctx, hp, tensors, signs, slots: int, group: int):
        import dataclasses

        import numpy as np
        from .lib import Model
        self.np = np
        self.ctx, self.slots, self.group = ctx, slots, group
        self.hp = dataclasses.replace(hp, n_streams=slots, batch_cols=group, block_begin=0, block_end=0)
        self.cap, self.vocab = self.hp.cap, self.hp.vocab
        self.m = Model(ctx, self.hp, tensors, signs)
        self.tok = ctx.alloc(group * 4)
        for g in range(slots // group):
            self.m.stage_prepare(g * group, group)
        ctx.sync()

    def reset_slot(self, s: int):
        self.m.reset_stream(s)

    def step(self, g: int, toks, pos):
        self.m.stage_batch(g * self.group, toks, pos, None, self.tok)
        self.ctx.sync()
        return self.tok.download(self.np.int32, self.group)

    def logits(self, g: int, i: int):
        return self.m.logits(i)            # column i of the pass that just ran (the caller reads before the next step)

    def close(self):
        self.m.close()
        self.tok.free()


def _error(code: int, kind: str, message: str):
    return code, {"error": {"message": message, "type": kind, "param": None, "code": None}}


def make_handler(batcher: Batcher, model_name: str):
    started = time.time()
    counter = {"requests": 0}

    class Handler(BaseHTTPRequestHandler):
        protocol_version = "HTTP/1.1"

        def log_message(self, *a):              # quiet
            pass

        def _send(self, code: int, body: dict):
            raw = json.dumps(body).encode()
            self.send_response(code)
            self.send_header("Content-Type", "application/json")
            self.send_header("Content-Length", str(len(raw)))
            self.end_headers()
            self.wfile.write(raw)

        def _loopback(self) -> bool:
            host = (self.headers.get("Host") or "").rsplit(":", 1)[0].strip("[]")
            return host in ("127.0.0.1", "localhost", "::1")

        def do_GET(self):
            if not self._loopback():
                return self._send(*_error(400, "invalid_request_error", "this server only answers loopback Host names"))
            path = self.path.split("?")[0]
            if path == "/v1/models":
                return self._send(200, {"object": "list", "data": [{"id": model_name, "object": "model", "owned_by": "local"}]})
            if path in ("/v1/status", "/health"):
                return self._send(200, {"status": "ok", "model": model_name, "slots": batcher.S, "busy": batcher.busy_slots(),
                                        "group": batcher.G, "requests": counter["requests"], "served": batcher.served,
                                        "steps": batcher.steps, "uptime_s": round(time.time() - started, 1)})
            if path in ("/v1/chat/completions", "/v1/completions"):
                return self._send(*_error(405, "invalid_request_error", f"use POST for {path}"))
            return self._send(*_error(404, "invalid_request_error", "unknown path " + path))

        def do_POST(self):
            if not self._loopback():
                return self._send(*_error(400, "invalid_request_error", "this server only answers loopback Host names"))
            path = self.path.split("?")[0]
            if path not in ("/v1/chat/completions", "/v1/completions"):
                return self._send(*_error(404, "invalid_request_error", "unknown path " + path))
            try:
                n = int(self.headers.get("Content-Length") or 0)
                req = json.loads(self.rfile.read(n) or b"{}")
                if not isinstance(req, dict):
                    raise ValueError
            except ValueError:
                return self._send(*_error(400, "invalid_request_error", "the body is not a JSON object"))
            counter["requests"] += 1
            chat = path.endswith("chat/completions")
            ids = req.get("prompt_ids") if chat else req.get("prompt")
            if not (isinstance(ids, list) and ids and all(isinstance(t, int) for t in ids)):
                return self._send(*_error(400, "invalid_request_error",
                                          "this server has no tokenizer (it stays on the host side of the boundary): send the prompt as "
                                          "token ids - \"prompt_ids\": [...] on /v1/chat/completions, \"prompt\": [...] on /v1/completions"))
            stop = req.get("stop_ids") or []
            try:
                conv = batcher.submit(ids, int(req.get("max_tokens", 1024)), [int(t) for t in stop], sampler_from_request(req))
            except Busy:
                return self._send(*_error(429, "rate_limit_error", f"all {batcher.S} conversation slots are generating; retry shortly"))
            except ValueError as ex:
                return self._send(*_error(400, "invalid_request_error", str(ex)))
            rid, created = f"cmpl-{counter['requests']}", int(time.time())
            model = req.get("model") or model_name
            if req.get("stream"):
                self.send_response(200)
                self.send_header("Content-Type", "text/event-stream")
                self.send_header("Cache-Control", "no-cache")
                self.send_header("Connection", "close")
                self.end_headers()
                while True:
                    kind, val = conv.events.get()
                    if kind == "tok":
                        delta = {"content": f"{val} ", "token_id": val} if chat else None
                        ch = {"index": 0, "delta": delta, "finish_reason": None} if chat else {"index": 0, "text": f"{val} ", "token_id": val, "finish_reason": None}
                        body = {"id": rid, "object": "chat.completion.chunk" if chat else "text_completion", "created": created, "model": model, "choices": [ch]}
                    else:
                        ch = {"index": 0, "delta": {}, "finish_reason": val} if chat else {"index": 0, "text": "", "finish_reason": val}
                        body = {"id": rid, "object": "chat.completion.chunk" if chat else "text_completion", "created": created, "model": model, "choices": [ch],
                                "usage": {"prompt_tokens": len(ids), "completion_tokens": len(conv.out), "total_tokens": len(ids) + len(conv.out)}}
                    self.wfile.write(b"data: " + json.dumps(body).encode() + b"\n\n")
                    self.wfile.flush()
                    if kind == "end":
                        self.wfile.write(b"data: [DONE]\n\n")
                        self.wfile.flush()
                        self.close_connection = True
                        return
            while True:
                kind, val = conv.events.get()
                if kind == "end":
                    break
            text = " ".join(str(t) for t in conv.out)
            usage = {"prompt_tokens": len(ids), "completion_tokens": len(conv.out), "total_tokens": len(ids) + len(conv.out)}
            if chat:
                choice = {"index": 0, "message": {"role": "assistant", "content": text}, "token_ids": conv.out, "finish_reason": conv.finish}
                return self._send(200, {"id": rid, "object": "chat.completion", "created": created, "model": model, "choices": [choice], "usage": usage})
            choice = {"index": 0, "text": text, "token_ids": conv.out, "finish_reason": conv.finish}
            return self._send(200, {"id": rid, "object": "text_completion", "created": created, "model": model, "choices": [choice], "usage": usage})

    return Handler


def serve(batcher: Batcher, model_name: str, host: str = "127.0.0.1", port: int = 8080) -> ThreadingHTTPServer:
    """Starts the server on a background thread and returns it (server.server_address holds the bound port)."""
    srv = ThreadingHTTPServer((host, port), make_handler(batcher, model_name))
    srv.daemon_threads = True
    threading.Thread(target=srv.serve_forever, daemon=True).start()
    return srv


def main(argv=None):
    import argparse
    ap = argparse.ArgumentParser(description="OpenAI-style /v1 server over the CUDA decode path (token ids in and out)")
    ap.add_argument("--gguf", help="model file; without it a seeded synthetic model of --shape is served")
    ap.add_argument("--shape", choices=["tiny", "9b"], default="tiny")
    ap.add_argument("--port", type=int, default=8080)
    ap.add_argument("--slots", type=int, default=8)
    ap.add_argument("--group", type=int, default=8)
    ap.add_argument("--cap", type=int, default=4096)
    a = ap.parse_args(argv)
    from . import Context, synth
    ctx = Context(0)
    if a.gguf:
        from . import gguf_reader
        hp, tensors, signs = gguf_reader.load(a.gguf, cap=a.cap)
    else:
        hp = synth.tiny(cap=a.cap) if a.shape == "tiny" else synth.HParams(cap=a.cap)
        tensors, signs = (synth.make_model(hp) if a.shape == "tiny" else synth.make_model_repeated(hp))
    eng = GpuEngine(ctx, hp, tensors, signs, a.slots, a.group)
    b = Batcher(eng)
    srv = serve(b, a.gguf or f"synthetic-{a.shape}", port=a.port)
    print(f"serving on http://127.0.0.1:{srv.server_address[1]}/v1 ({a.slots} slots in groups of {a.group})", flush=True)
    try:
        while True:
            time.sleep(3600)
    except KeyboardInterrupt:
        pass
    srv.shutdown(); b.close(); eng.close()


if __name__ == "__main__":
    main()
