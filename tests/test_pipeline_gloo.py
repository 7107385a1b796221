"""Host-side logic of the layer pipeline, without a GPU: split arithmetic (reference: the 55 host-only checks of
`bonsai_fleet selftest`, runtime_vk/bonsai_fleet.cpp:817-1069) and the message schedule run as two / three gloo
ranks on CPU with a stand-in stage function."""
import os
import socket
import subprocess
import sys
import textwrap

import pytest

from bonsai_vk_b200.pipeline import split_blocks

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def test_equal_split_matches_benchmark_config():
    assert split_blocks(32, 2) == [(0, 16), (16, 32)]
    assert split_blocks(32, 4) == [(0, 8), (8, 16), (16, 24), (24, 32)]
    assert [b - a for a, b in split_blocks(32, 8)] == [4] * 8
    assert split_blocks(32, 1) == [(0, 32)]
    assert split_blocks(5, 2) == [(0, 3), (3, 5)]


def test_split_is_contiguous_and_refuses_bad_requests():
    for world in (1, 2, 3, 4, 8):
        for mode in ("equal", "bytes"):
            r = split_blocks(32, world, mode, block_bytes=[48923392 if b % 4 != 3 else 45910016 for b in range(32)],
                             head_bytes=222494720)
            assert r[0][0] == 0 and r[-1][1] == 32
            assert all(a < b for a, b in r) and all(r[i][1] == r[i + 1][0] for i in range(len(r) - 1))
    with pytest.raises(ValueError):
        split_blocks(4, 5)
    with pytest.raises(ValueError):
        split_blocks(4, 0)


def test_byte_balanced_split_gives_the_head_stage_fewer_blocks():
    """Per-block bytes of the 9B in native PTQ1_0 form: GDN 48 923 392, attention 45 910 016
    (runtime_vk/gpu_fleet.h:984-988); the 222 MB head sits on the last stage."""
    bb = [48923392 if b % 4 != 3 else 45910016 for b in range(32)]
    r = split_blocks(32, 8, "bytes", block_bytes=bb, head_bytes=222494720)
    sizes = [b - a for a, b in r]
    assert sizes[-1] < 4 and sum(sizes) == 32
    loads = [sum(bb[a:b]) for a, b in r]
    loads[-1] += 222494720
    assert max(loads) < 1.35 * (sum(bb) + 222494720) / 8


WORKER = textwrap.dedent('''
    import os, sys, torch, torch.distributed as dist
    sys.path.insert(0, os.environ["BONSAI_ROOT"])
    from bonsai_vk_b200.pipeline import Pipeline
    rank, world = int(os.environ["RANK"]), int(os.environ["WORLD_SIZE"])
    dist.init_process_group("gloo", rank=rank, world_size=world)
    fwd, back = dist.new_group(list(range(world))), dist.new_group(list(range(world)))
    S, T, H, V = 5, 4, 8, 97
    def stage(s, step, pos, tok_first, tok_in, hin, out):
        if rank == 0:
            tok = tok_first if tok_first is not None else int(tok_in.item())
            h = torch.arange(H, dtype=torch.float32) * (tok + 1) + pos
        else:
            h = hin.clone()
        h = h * 1.5 + (rank + 1)
        if rank == world - 1:
            out.fill_(int(h.sum().item()) % V)
        else:
            out.copy_(h)
    p = Pipeline(dist, rank, world, S, stage, lambda: torch.zeros(H), lambda: torch.zeros(1, dtype=torch.int32), fwd, back)
    first = [3 + s for s in range(S)]
    picks = p.run(first, [10 * s for s in range(S)], T)
    if rank == world - 1:
        # the same recurrence in one process
        want = []
        for s in range(S):
            tok, row = first[s], []
            for step in range(T):
                h = torch.arange(H, dtype=torch.float32) * (tok + 1) + (10 * s + step)
                for r in range(world):
                    h = h * 1.5 + (r + 1)
                tok = int(h.sum().item()) % V
                row.append(tok)
            want.append(row)
        assert picks == want, (picks, want)
        print("PIPELINE_OK")
    dist.barrier()
    dist.destroy_process_group()
''')


@pytest.mark.parametrize("world", [2, 3])
def test_message_schedule_on_gloo(world, tmp_path):
    script = tmp_path / "worker.py"
    script.write_text(WORKER)
    with socket.socket() as sck:
        sck.bind(("127.0.0.1", 0))
        port = sck.getsockname()[1]
    procs = []
    for r in range(world):
        env = dict(os.environ, RANK=str(r), WORLD_SIZE=str(world), MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port),
                   BONSAI_ROOT=ROOT)
        procs.append(subprocess.Popen([sys.executable, str(script)], env=env, stdout=subprocess.PIPE, stderr=subprocess.STDOUT, text=True))
    try:
        outs = [p.communicate(timeout=120)[0] for p in procs]
    finally:
        for p in procs:            # never leave a rank behind (each is ended through its own handle)
            if p.poll() is None:
                p.kill()
    assert all(p.returncode == 0 for p in procs), outs
    assert "PIPELINE_OK" in outs[-1]


WORKER_MB = textwrap.dedent('''
    import os, sys, torch, torch.distributed as dist
    sys.path.insert(0, os.environ["BONSAI_ROOT"])
    from bonsai_vk_b200.pipeline import Pipeline
    rank, world = int(os.environ["RANK"]), int(os.environ["WORLD_SIZE"])
    dist.init_process_group("gloo", rank=rank, world_size=world)
    fwd, back = dist.new_group(list(range(world))), dist.new_group(list(range(world)))
    U, MB, T, H, V = 3, 4, 4, 8, 97          # 3 micro-batches of 4 sequences
    def stage(u, step, pos, tok_first, tok_in, hin, out):
        if rank == 0:
            toks = tok_first if tok_first is not None else [int(v) for v in tok_in.tolist()]
            h = torch.stack([torch.arange(H, dtype=torch.float32) * (t + 1) + pos + c for c, t in enumerate(toks)]).reshape(-1)
        else:
            h = hin.clone()
        h = h * 1.5 + (rank + 1)
        if rank == world - 1:
            out.copy_((h.reshape(MB, H).sum(dim=1).to(torch.int64) % V).to(torch.int32))
        else:
            out.copy_(h)
    p = Pipeline(dist, rank, world, U, stage, lambda: torch.zeros(MB * H), lambda: torch.zeros(MB, dtype=torch.int32), fwd, back)
    first = [[3 + u * MB + c for c in range(MB)] for u in range(U)]
    picks = p.run(first, [10 * u for u in range(U)], T)
    if rank == world - 1:
        want = []
        for u in range(U):
            toks, row = list(first[u]), []
            for step in range(T):
                nxt = []
                for c, tok in enumerate(toks):
                    h = torch.arange(H, dtype=torch.float32) * (tok + 1) + (10 * u + step) + c
                    for r in range(world):
                        h = h * 1.5 + (r + 1)
                    nxt.append(int(h.sum().item()) % V)
                toks = nxt
                row.append(nxt)
            want.append(row)
        assert picks == want, (picks, want)
        print("PIPELINE_OK")
    dist.barrier()
    dist.destroy_process_group()
''')


def test_micro_batched_schedule_on_gloo(tmp_path):
    """The same ring with micro-batches of several sequences as the unit (vector messages)."""
    world = 2
    script = tmp_path / "worker_mb.py"
    script.write_text(WORKER_MB)
    with socket.socket() as sck:
        sck.bind(("127.0.0.1", 0))
        port = sck.getsockname()[1]
    procs = []
    for r in range(world):
        env = dict(os.environ, RANK=str(r), WORLD_SIZE=str(world), MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port),
                   BONSAI_ROOT=ROOT)
        procs.append(subprocess.Popen([sys.executable, str(script)], env=env, stdout=subprocess.PIPE, stderr=subprocess.STDOUT, text=True))
    try:
        outs = [p.communicate(timeout=120)[0] for p in procs]
    finally:
        for p in procs:
            if p.poll() is None:
                p.kill()
    assert all(p.returncode == 0 for p in procs), outs
    assert "PIPELINE_OK" in outs[-1]


def test_head_rows_split():
    from bonsai_vk_b200.pipeline import split_head_rows
    r = split_head_rows(248320, 8)
    assert r[0][0] == 0 and r[-1][1] == 248320 and all(r[i][1] == r[i + 1][0] for i in range(7))
    assert all(a % 128 == 0 for a, _ in r) and max(b - a for a, b in r) - min(b - a for a, b in r) <= 128
    assert split_head_rows(2048, 1) == [(0, 2048)]
    assert split_head_rows(1000, 2) == [(0, 512), (512, 1000)]
    with pytest.raises(ValueError):
        split_head_rows(256, 3)


WORKER_SH = textwrap.dedent('''
    import os, sys, torch, torch.distributed as dist
    sys.path.insert(0, os.environ["BONSAI_ROOT"])
    from bonsai_vk_b200.pipeline import ShardedHeadPipeline
    rank, world = int(os.environ["RANK"]), int(os.environ["WORLD_SIZE"])
    dist.init_process_group("gloo", rank=rank, world_size=world)
    fwd, head = dist.new_group(list(range(world))), dist.new_group(list(range(world)))
    U, MB, T, H, V = int(os.environ["UNITS"]), 2, 5, 8, 96
    rows = V // world                      # rank r holds "head rows" [r * rows, (r + 1) * rows)
    def logits(h):                         # a stand-in head: V rows from one hidden vector
        return torch.stack([(h * ((v % 7) + 1)).sum() % 11 for v in range(V)])
    def stage(u, step, pos, tok_first, tok_in, hin, out):
        if rank == 0:
            toks = tok_first if tok_first is not None else [int(v) for v in tok_in.tolist()]
            h = torch.stack([torch.arange(H, dtype=torch.float32) * (t + 1) + pos + c for c, t in enumerate(toks)]).reshape(-1)
        else:
            h = hin.clone()
        out.copy_(h * 1.5 + (rank + 1))
    def head_fn(u, hfin, cand):
        for c in range(MB):
            lg = logits(hfin.view(MB, H)[c])[rank * rows:(rank + 1) * rows]
            i = int(torch.argmax(lg))                     # first maximum within the shard
            cand.view(MB, 2)[c, 0] = lg[i]
            cand.view(MB, 2)[c, 1] = float(rank * rows + i)
    def pick_fn(u, allc, tok):
        a = allc.view(world, MB, 2)
        for c in range(MB):
            best, idx = -1e30, 2 ** 31 - 1
            for s in range(world):
                v, i = float(a[s, c, 0]), int(a[s, c, 1])
                if v > best or (v == best and i < idx):
                    best, idx = v, i
            tok[c] = idx
    class Lanes:                           # records what a two-queue implementation is told, in host order
        def __init__(self): self.log = []
        def head_begin(self, m): self.log.append(("hb", m))
        def head_end(self, m): self.log.append(("he", m))
        def stage_begin(self, n): self.log.append(("sb", n))
        def stage_end(self, n): self.log.append(("se", n))
        def finish(self): self.log.append(("fin", -1))
    lanes = Lanes()
    p = ShardedHeadPipeline(dist, rank, world, U, stage, head_fn, pick_fn, lambda: torch.zeros(MB * H),
                            lambda: torch.zeros(MB, dtype=torch.int32), lambda n: torch.zeros(n * MB * 2), fwd, head, lanes=lanes)
    first = [[3 + u * MB + c for c in range(MB)] for u in range(U)]
    picks = p.run(first, [10 * u for u in range(U)], T)
    # the orderings a second queue has to be able to express with events that already exist when they are needed:
    at = {e: i for i, e in enumerate(lanes.log)}
    N = T * U
    assert lanes.log[-1] == ("fin", -1) and len(lanes.log) == 4 * N + 1
    for n in range(N):
        assert at[("sb", n)] < at[("se", n)] and at[("hb", n)] < at[("he", n)]
        assert at[("se", n)] < at[("hb", n)], "head work of an instance is issued after its stage work"
        if n >= U:
            assert at[("he", n - U)] < at[("sb", n)], "the pick of the previous step is issued before the stage work that needs it"
    for (k0, _), (k1, _) in zip(lanes.log, lanes.log[1:]):      # head and stage sections never nest
        assert (k0, k1) not in (("hb", "sb"), ("sb", "hb"), ("hb", "hb"), ("sb", "sb"))
    if rank == 0:
        want = []
        for u in range(U):
            toks, row = list(first[u]), []
            for step in range(T):
                nxt = []
                for c, tok in enumerate(toks):
                    h = torch.arange(H, dtype=torch.float32) * (tok + 1) + (10 * u + step) + c
                    for r in range(world):
                        h = h * 1.5 + (r + 1)
                    nxt.append(int(torch.argmax(logits(h))))
                toks = nxt
                row.append(nxt)
            want.append(row)
        assert picks == want, (picks, want)
        print("PIPELINE_OK")
    dist.barrier()
    dist.destroy_process_group()
''')


@pytest.mark.parametrize("world,units", [(2, 2), (3, 3), (3, 5), (3, 1)])
def test_sharded_head_schedule_on_gloo(world, units, tmp_path):
    """The ring with the output head spread over the stages: broadcast of the final hidden state, per-rank candidates,
    gather, pick on rank 0 - as gloo ranks with blocking collectives (the schedule must not deadlock), with as many
    units as stages, more, and fewer."""
    script = tmp_path / "worker_sh.py"
    script.write_text(WORKER_SH)
    with socket.socket() as sck:
        sck.bind(("127.0.0.1", 0))
        port = sck.getsockname()[1]
    procs = []
    for r in range(world):
        env = dict(os.environ, RANK=str(r), WORLD_SIZE=str(world), MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port),
                   BONSAI_ROOT=ROOT, UNITS=str(units))
        procs.append(subprocess.Popen([sys.executable, str(script)], env=env, stdout=subprocess.PIPE, stderr=subprocess.STDOUT, text=True))
    try:
        outs = [p.communicate(timeout=180)[0] for p in procs]
    finally:
        for p in procs:
            if p.poll() is None:
                p.kill()
    assert all(p.returncode == 0 for p in procs), outs
    assert "PIPELINE_OK" in outs[0]


def test_two_cuda_streams_orders_the_two_queues():
    """`TwoCudaStreams` against a stand-in for torch.cuda: the head queue waits for the stage work of the same instance,
    the stage queue for the head work one step of units earlier, the library context follows the queue in use, and
    finish() joins what is left."""
    from bonsai_vk_b200.pipeline import TwoCudaStreams

    log = []

    class Event:
        def __init__(self): self.on = None
        def record(self, stream): self.on = stream.name

    class Stream:
        def __init__(self, device=None, priority=0, name="side"): self.device, self.name, self.cuda_stream = device, name, hash(name)
        def wait_event(self, ev): log.append(("wait", self.name, ev.on))

    event_cls, stream_cls = Event, Stream

    class Cuda:
        Event = event_cls
        def Stream(self, device=None, priority=0): assert priority == -1; return stream_cls(device, priority)
        def set_stream(self, s): log.append(("current", s.name))

    class Torch: cuda = Cuda()

    class Ctx:
        def use_stream(self, h): log.append(("ctx", h))

    work = Stream(name="work")
    lanes = TwoCudaStreams(Torch, Ctx(), work, n_units=2)
    lanes.stage_begin(0); lanes.stage_end(0)
    lanes.stage_begin(1); lanes.stage_end(1)
    lanes.head_begin(0); lanes.head_end(0)          # head work of instance 0 ...
    lanes.stage_begin(2); lanes.stage_end(2)        # ... before the stage work of instance 2 = 0 + units
    lanes.head_begin(1); lanes.head_end(1)
    lanes.finish()
    waits = [(e[1], e[2]) for e in log if e[0] == "wait"]           # (the queue that waits, the queue the event was recorded on)
    # head 0 waits for stage 0's event (recorded on work); stage 2 waits for head 0's (recorded on side); head 1 for stage 1;
    # finish joins head 1 into work
    assert waits == [("side", "work"), ("work", "side"), ("side", "work"), ("work", "side")]
    cur = [e[1] for e in log if e[0] == "current"]
    assert cur == ["side", "work", "side", "work"]
    assert [e[1] for e in log if e[0] == "ctx"] == [hash("side"), hash("work"), hash("side"), hash("work")]
    assert not lanes.ev_head and not lanes.ev_stage
