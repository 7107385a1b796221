"""Layer-pipelined decode over several GPUs of one box (one process per GPU, torch.distributed).

Semantics taken from the reference's multi-GPU rig (runtime_vk/gpu_fleet.h:949-1115 split, :1414-1626 runner):
contiguous block ranges, the embedding on the first stage and the output head on the last, recurrent state and
KV cache never leave their stage, one hand-off of the `hidden` fp32 values (16 KiB at hidden 4096) per stage
boundary per token, and micro-batching = several sequences in flight so that every stage is busy. The transport
here is NCCL send/recv over NVLink into the consumer's own buffer (the reference stages through a host-pinned
ring); the only other message is the picked token id going from the last stage back to the first.

Two process groups are used on purpose: hidden states flow forward on one communicator and token ids flow
backward on another, so a token send that is waiting for the first stage to reach the next step can never
sit in front of a hidden-state receive on the same NCCL stream (that ordering would deadlock the ring).
"""
from __future__ import annotations

from typing import Callable, List, Tuple


def split_blocks(n_layer: int, world: int, balance: str = "equal", block_bytes=None, head_bytes: int = 0,
                 embed_bytes: int = 0) -> List[Tuple[int, int]]:
    """Contiguous block ranges per stage. "equal": the same number of blocks per stage (the benchmark config:
    16/8/4 blocks on 2/4/8 GPUs). "bytes": ranges balanced by bytes read per token, with the head's bytes
    charged to the last stage and the embedding's to the first, as fleet_split_schedule does
    (runtime_vk/gpu_fleet.h:1013-1020). Refuses more stages than blocks."""
    if world < 1 or world > n_layer:
        raise ValueError(f"cannot split {n_layer} blocks over {world} stages")
    if balance == "equal":
        base, extra = divmod(n_layer, world)
        out, b = [], 0
        for r in range(world):
            n = base + (1 if r < extra else 0)
            out.append((b, b + n))
            b += n
        return out
    if balance != "bytes":
        raise ValueError(f"unknown balance mode {balance!r}")
    w = list(block_bytes) if block_bytes is not None else [1] * n_layer
    if len(w) != n_layer:
        raise ValueError("block_bytes must have one entry per block")
    total = sum(w) + head_bytes + embed_bytes
    out, b, acc = [], 0, float(embed_bytes)
    for r in range(world):
        remaining_stages = world - r
        if r == world - 1:
            out.append((b, n_layer))
            break
        target = total * (r + 1) / world
        e = b + 1
        acc += w[b]
        # take blocks while we are below this stage's cumulative target and enough blocks remain for the others
        while e < n_layer - (remaining_stages - 1) and acc + w[e] / 2 <= target:
            acc += w[e]
            e += 1
        out.append((b, e))
        b = e
    return out


class Pipeline:
    """Runs `n_steps` greedy decode steps of `n_streams` sequences through the stages.

    stage_fn(stream, step, pos, tok_first, tok_in, hidden_in, out) enqueues this rank's blocks:
      first stage : tok_first (int, step 0) or tok_in (tensor holding one int32, later steps) -> out (hidden)
      middle      : hidden_in -> out (hidden)
      last stage  : hidden_in -> out (tensor holding one int32: the pick)
    new_hidden() / new_token() allocate the message tensors on the right device.

    A "stream" may also be a micro-batch of several sequences that move through the stages together (the stage
    function then runs them in one pass): the messages are [sequences x hidden] and [sequences] tensors, first_tokens[s]
    is a list, and every sequence of the micro-batch is at position pos0[s] + step."""

    def __init__(self, dist, rank: int, world: int, n_streams: int, stage_fn: Callable, new_hidden: Callable,
                 new_token: Callable, fwd_group=None, back_group=None):
        self.dist, self.rank, self.world, self.S = dist, rank, world, n_streams
        self.stage_fn = stage_fn
        self.first, self.last = rank == 0, rank == world - 1
        self.fwd, self.back = fwd_group, back_group
        self.h_in = [new_hidden() for _ in range(n_streams)] if not self.first else None
        self.h_out = [new_hidden() for _ in range(n_streams)] if not self.last else None
        self.t_in = [new_token() for _ in range(n_streams)] if self.first and world > 1 else None
        self.t_out = [new_token() for _ in range(n_streams)] if self.last else None
        self.picks: List[list] = [[] for _ in range(n_streams)]

    def run(self, first_tokens, pos0, n_steps: int, collect: bool = True):
        d, S, P = self.dist, self.S, self.world
        send_h = [None] * S
        send_t = [None] * S
        for step in range(n_steps):
            for s in range(S):
                pos = pos0[s] + step
                tok_in = None
                if self.first:
                    if step > 0:
                        if P > 1:
                            d.irecv(self.t_in[s], src=P - 1, group=self.back).wait()
                            tok_in = self.t_in[s]
                        else:
                            tok_in = self.t_out[s]
                    hin = None
                else:
                    d.irecv(self.h_in[s], src=self.rank - 1, group=self.fwd).wait()
                    hin = self.h_in[s]
                if self.last:
                    if send_t[s] is not None:
                        send_t[s].wait()            # the previous pick of this stream has left the buffer
                        send_t[s] = None            # (a send handle is waited on exactly once)
                    out = self.t_out[s]
                else:
                    if send_h[s] is not None:
                        send_h[s].wait()
                        send_h[s] = None
                    out = self.h_out[s]
                self.stage_fn(s, step, pos, first_tokens[s] if (self.first and step == 0) else None, tok_in, hin, out)
                if self.last:
                    if collect:
                        self.picks[s].append(out.clone())
                    if P > 1 and step + 1 < n_steps:
                        send_t[s] = d.isend(out, dst=0, group=self.back)
                else:
                    send_h[s] = d.isend(out, dst=self.rank + 1, group=self.fwd)
        for h in send_h + send_t:
            if h is not None:
                h.wait()
        if not (self.last and collect):
            return None
        # one int per step for a single sequence, a list of ints per step for a micro-batch of sequences
        return [[int(t.item()) if t.numel() == 1 else [int(v) for v in t.tolist()] for t in row] for row in self.picks]


def split_head_rows(vocab: int, world: int, tile: int = 128) -> List[Tuple[int, int]]:
    """Row ranges of the output head per stage for the sharded head: whole 128-row tiles, as equal as they come,
    ascending with the stage number (the pick over the shards relies on that order for ties)."""
    tiles = (vocab + tile - 1) // tile
    if world < 1 or world > tiles:
        raise ValueError(f"cannot split {tiles} head tiles over {world} stages")
    base, extra = divmod(tiles, world)
    out, t = [], 0
    for r in range(world):
        n = base + (1 if r < extra else 0)
        out.append((t * tile, min(vocab, (t + n) * tile)))
        t += n
    return out


class NoLanes:
    """Head work and stage work on one queue (the default): nothing to order."""

    def head_begin(self, m: int): pass
    def head_end(self, m: int): pass
    def stage_begin(self, n: int): pass
    def stage_end(self, n: int): pass
    def finish(self): pass


class TwoCudaStreams:
    """Head work on a second, high-priority CUDA stream: on every rank but the first it then overlaps the stage passes
    (which are full of small launches that leave most of the GPU idle), and every rank answers the head collectives at
    once instead of after its current pass. `ctx` is the library context whose kernels follow torch's current stream."""

    def __init__(self, torch, ctx, work_stream, n_units: int):
        self.torch, self.ctx, self.work, self.U = torch, ctx, work_stream, n_units
        self.side = torch.cuda.Stream(device=work_stream.device, priority=-1)
        self.ev_stage, self.ev_head = {}, {}

    def _on(self, stream):
        self.torch.cuda.set_stream(stream)
        self.ctx.use_stream(stream.cuda_stream)

    def head_begin(self, m: int):
        ev = self.ev_stage.pop(m, None)
        if ev is not None:
            self.side.wait_event(ev)
        self._on(self.side)

    def head_end(self, m: int):
        ev = self.torch.cuda.Event()
        ev.record(self.side)
        self.ev_head[m] = ev
        self._on(self.work)

    def stage_begin(self, n: int):
        ev = self.ev_head.pop(n - self.U, None)
        if ev is not None:
            self.work.wait_event(ev)

    def stage_end(self, n: int):
        ev = self.torch.cuda.Event()
        ev.record(self.work)
        self.ev_stage[n] = ev
        self.ev_stage.pop(n - 2 * self.U, None)

    def finish(self):
        for ev in self.ev_head.values():
            self.work.wait_event(ev)
        self.ev_head.clear()
        self.ev_stage.clear()


class ShardedHeadPipeline:
    """The same ring of stages with the output head spread over all of them (the reference charges the whole head to the
    last GPU of its split, runtime_vk/gpu_fleet.h:1013-1020, which makes that stage the long one at 4 blocks per GPU).

    Every stage, the last included, hands on a hidden state. For unit (micro-batch) instance m = step * units + u:
      1. the last stage broadcasts the final hidden state of m to every rank        (collective on `head_group`)
      2. every rank runs its rows of the head on it: head_fn(u, hidden, cand_out)   -> (value, row) per sequence
      3. the candidates are gathered on every rank                                   (collective on `head_group`)
      4. rank 0 picks: pick_fn(u, all_cands, tok_out) - the token that enters its stage for u at the next step.
    A rank does the head work of instance m right BEFORE its own stage work of instance m + lag, lag = min(world - 1 - rank,
    units - 1) + 1: when every stage takes the same time the last stage finished m one slot earlier, so the hidden state
    is already there and no rank stalls on a stage that is still running (head work placed after the stage work of the
    same slot made every slot wait for the slowest stage: measured 0.84 ms per slot where the stage pass takes 0.66).
    Rank 0 has the token just before the stage that needs it (lag <= units), and because the lag does not grow with the
    rank every rank reaches collective m without needing anything a later collective would provide - the schedule
    cannot deadlock even on a backend whose collectives block the host.

    stage_fn(u, step, pos, tok_first, tok_in, hidden_in, hidden_out); picks are collected on rank 0.

    `lanes` (optional) lets the head work run on a second device queue beside the stage work. It is told where each kind
    of work starts and ends, in the order the host issues it, and has to keep three orderings between the two queues:
    head work of instance m after stage work of m (the last stage's pass wrote the hidden state that is broadcast);
    stage work of instance n after head work of n - units (rank 0: the token it enters with; last stage: its pass
    overwrites the hidden state the head read); everything joined at finish(). The host-side order of the collectives is
    the same with and without it, so the deadlock argument above does not change. See `NoLanes` for the interface."""

    def __init__(self, dist, rank: int, world: int, n_units: int, stage_fn: Callable, head_fn: Callable, pick_fn: Callable,
                 new_hidden: Callable, new_token: Callable, new_cand: Callable, fwd_group=None, head_group=None, mark: Callable = None,
                 lanes=None):
        self.dist, self.rank, self.world, self.U = dist, rank, world, n_units
        self.mark = mark or (lambda name: None)        # profiling aid: called at the phase boundaries of every slot
        self.lanes = lanes or NoLanes()
        self.stage_fn, self.head_fn, self.pick_fn = stage_fn, head_fn, pick_fn
        self.first, self.last = rank == 0, rank == world - 1
        self.fwd, self.head = fwd_group, head_group
        self.lag = min(world - 1 - rank, n_units - 1) + 1
        self.h_in = [new_hidden() for _ in range(n_units)] if not self.first else None
        self.h_out = [new_hidden() for _ in range(n_units)] if not self.last else None
        self.h_fin = [new_hidden() for _ in range(n_units)]
        self.cand = [new_cand(1) for _ in range(n_units)]
        self.cands_all = [new_cand(world) for _ in range(n_units)]
        self.t_in = [new_token() for _ in range(n_units)] if self.first else None
        self.picks: List[list] = [[] for _ in range(n_units)]

    def _head_work(self, m: int, collect: bool):
        d, u, P = self.dist, m % self.U, self.world
        self.lanes.head_begin(m)
        self.mark("slot")
        if P > 1:
            d.broadcast(self.h_fin[u], src=P - 1, group=self.head, async_op=True).wait()
        self.mark("bcast")
        self.head_fn(u, self.h_fin[u], self.cand[u])
        self.mark("head")
        if P > 1:
            rows = list(self.cands_all[u].view(P, -1).unbind(0))
            d.all_gather(rows, self.cand[u].view(-1), group=self.head, async_op=True).wait()
        else:
            self.cands_all[u].copy_(self.cand[u])
        self.mark("gather")
        if self.first:
            self.pick_fn(u, self.cands_all[u], self.t_in[u])
            self.mark("pick")
            if collect:
                self.picks[u].append(self.t_in[u].clone())
        self.lanes.head_end(m)

    def run(self, first_tokens, pos0, n_steps: int, collect: bool = True):
        d, U, P = self.dist, self.U, self.world
        N = n_steps * U
        send_h = [None] * U
        for n in range(N):
            step, u = divmod(n, U)
            pos = pos0[u] + step
            if n - self.lag >= 0:
                self._head_work(n - self.lag, collect)
            tok_in, hin = None, None
            if self.first:
                if step > 0:
                    tok_in = self.t_in[u]
            else:
                d.irecv(self.h_in[u], src=self.rank - 1, group=self.fwd).wait()
                hin = self.h_in[u]
            if self.last:
                out = self.h_fin[u]
            else:
                if send_h[u] is not None:
                    send_h[u].wait()            # the previous message of this unit has left the buffer
                    send_h[u] = None
                out = self.h_out[u]
            self.mark("recv")
            self.lanes.stage_begin(n)
            self.stage_fn(u, step, pos, first_tokens[u] if (self.first and step == 0) else None, tok_in, hin, out)
            self.lanes.stage_end(n)
            self.mark("stage")
            if not self.last:
                send_h[u] = d.isend(out, dst=self.rank + 1, group=self.fwd)
        for m in range(max(0, N - self.lag), N):
            self._head_work(m, collect)
        for h in send_h:
            if h is not None:
                h.wait()
        self.lanes.finish()
        if not (self.first and collect):
            return None
        return [[int(t.item()) if t.numel() == 1 else [int(v) for v in t.tolist()] for t in row] for row in self.picks]
