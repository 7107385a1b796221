#!/usr/bin/env python
"""Benchmark of the decode hot path: greedy decode tok/s of the 9B-shape synthetic PTQ1_0 model.

  python bench.py [--gpus N] [--steps K] [--warmup W] [--impl ours|reference]

One "step" is one decoded token (one pass of the whole-token schedule). Prints ONE JSON line.
  value  - tok/s with everything resident in HBM: K tokens chained on the device (CUDA graph replay,
           the greedy pick is fed back without a host round trip), CUDA events on the launch stream.
  e2e    - the same metric through the per-token C-ABI call a host makes (bn_model_token): the token
           id and position go host->device and the pick comes device->host inside the timed region.
  roofline - the token's fused projection launches (the dominant kernel) timed back to back with CUDA events:
           algorithmic PTQ1_0 bytes / time, against the measured copy bandwidth of this GPU pool.
  cpu_baseline - the reference's CPU arithmetic for the path, timed on the host cores on a bounded sample.
  streams64 - (N=1 only) the 64-sequence workload of the multi-GPU configuration on this one GPU, the base of its scaling.
--impl reference times the reference's own CPU arithmetic for the path (dequantise + fp64 dot,
oracle/_ref when built, else the oracle port) on all host cores, in the same unit.
N > 1 (torchrun, one rank per GPU): the 64-stream pipeline workload - the model is layer-pipelined over the N GPUs
(contiguous block stages, hidden state handed off over NVLink with NCCL send/recv), 64 concurrent sequences at
context 8192 are micro-batched through the stages; a step is one decode step of all 64 sequences and `value`
is the aggregate tok/s. The KV caches are marked filled up to the start position (the reference's own
BONSAI_KVFILL practice for long-context timing): timings are valid, token values are not meaningful.
"""
from __future__ import annotations

import argparse
import json
import os
import subprocess
import sys
import threading
import time

import numpy as np

ROOT = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, ROOT)

PTQ_WEIGHTS_PER_TOKEN = 8_946_450_432 - 1_017_118_720      # the 201 projections (token_embd is only gathered)
PTQ_BYTES_PER_TOKEN = 1_734_541_312                        # their PTQ1_0 bytes
ALGO_BYTES_PER_TOKEN = 1_734_541_312 + 29_411_328 + 2 * 50_331_648 + 2 * 2_359_296 + 896   # + f32, GDN state r/w, conv


NCU_TRAFFIC_RATIO = 1.023      # dram read+write / PTQ1_0 bytes of the launch (ncu, head projection 248320 x 4096)


def peaks():
    p = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.exists(p):
        return json.load(open(p)).get("hbm_gbs", 6650.0), "measured"
    return 6650.0, "fallback"


class ClockSampler:
    Q = ("clocks.sm,clocks.max.sm,clocks_event_reasons.hw_slowdown,clocks_event_reasons.hw_thermal_slowdown,"
         "clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap")

    def __init__(self, index: int):
        self.index, self.rows, self.proc = index, [], None

    def start(self):
        try:
            self.proc = subprocess.Popen(["nvidia-smi", f"--id={self.index}", f"--query-gpu={self.Q}",
                                          "--format=csv,noheader,nounits", "-lms", "20"],
                                         stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True)
            threading.Thread(target=self._read, daemon=True).start()
            t0 = time.perf_counter()          # nvidia-smi needs about a second before its first row
            while not self.rows and time.perf_counter() - t0 < 5.0:
                time.sleep(0.02)
        except OSError:
            self.proc = None

    def mark(self):
        """start of the window the summary is taken over (rows before it are idle-clock samples)"""
        self.t_mark = time.perf_counter()

    def _read(self):
        for line in self.proc.stdout:
            self.rows.append([c.strip() for c in line.split(",")] + [time.perf_counter()])

    def stop(self):
        if self.proc:
            self.proc.terminate()
        t_mark = getattr(self, "t_mark", 0.0)
        inside = [r for r in self.rows if r[-1] >= t_mark]
        self.rows = [r[:-1] for r in (inside or self.rows)]
        sm = [int(r[0]) for r in self.rows if r and r[0].isdigit()]
        mx = [int(r[1]) for r in self.rows if len(r) > 1 and r[1].isdigit()]
        names = ["hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"]
        reasons = [n for i, n in enumerate(names) if any(len(r) > 2 + i and r[2 + i].startswith("Active") for r in self.rows)]
        return {"sm_mhz": int(np.median(sm)) if sm else None, "sm_max_mhz": max(mx) if mx else None,
                "reasons": reasons, "samples": len(sm)}


def build_full_model(hp, seed=0, head_everywhere=False):
    from bonsai_vk_b200 import synth
    return synth.make_model_repeated(hp, seed, head_everywhere)


def cpu_gemv_tokens_per_s(seconds=12.0, threads=None):
    """Reference CPU arithmetic for the path: dequantise each PTQ1_0 block and accumulate w*x in double
    (runtime_vk/bonsai_weights.h:751-768 around ptq_dequant_ours). Bounded sample: repeated 4096x4096
    GEMVs for about `seconds`; weights/s divided by the weights one token's 201 projections read."""
    import ctypes as C
    from bonsai_vk_b200 import ptq
    from tests import _oracle
    threads = threads or os.cpu_count() or 1
    ref = _oracle.load_ref()
    kind = "reference" if ref is not None else "port"
    M = K = 4096
    W = np.ascontiguousarray(ptq.synth_matrix(np.random.default_rng(0), M, K))
    x = np.random.default_rng(1).standard_normal(K).astype(np.float32)
    out = np.empty(M, dtype=np.float64)
    p = lambda a: a.ctypes.data_as(C.c_void_p)
    if ref is not None:
        fn = lambda: ref.ref_gemv_dequant_f64(p(W), M, K, p(x), p(out), threads)
    else:
        o = _oracle.load_oracle()
        fn = lambda: o.lib.bo_gemv_dequant_f64(p(W), M, K, p(x), p(out), threads)
    fn()
    n, t0 = 0, time.perf_counter()
    while time.perf_counter() - t0 < seconds:
        fn(); n += 1
    dt = time.perf_counter() - t0
    tok_s = (n * M * K / dt) / PTQ_WEIGHTS_PER_TOKEN
    return {"value": tok_s, "unit": "tok/s", "cores": threads, "kind": kind,
            "sample": f"{n} x 4096x4096 PTQ1_0 GEMV (dequantise + fp64 dot) in {dt:.1f}s, scaled by the "
                      f"{PTQ_WEIGHTS_PER_TOKEN} projection weights one token reads"}


def streams64_one_gpu(ctx, tensors_again=None, steps=6, warm=2):
    """Config 4's load on ONE GPU: all 32 blocks, 64 sequences at context 8192 (KV marked filled) as two passes of 32
    sequences per decode step (tensor-core projection kernel: the weights are read once per pass)."""
    from bonsai_vk_b200 import Model, synth
    S, MB, CTX = 64, 32, 8192
    hp = synth.HParams(cap=CTX, n_streams=S, batch_cols=MB)
    tensors, signs = synth.make_model_repeated(hp)
    m = Model(ctx, hp, tensors, signs)
    del tensors
    pos0 = CTX - (steps + warm) - 2
    for s in range(S):
        m.fill_kv(s, pos0)
    toks = [ctx.alloc(MB * 4) for _ in range(S // MB)]
    first = [int(t) for t in np.random.default_rng(7).integers(0, hp.vocab, size=S)]
    for u in range(S // MB):
        m.stage_prepare(u * MB, MB)

    def step(i):
        for u in range(S // MB):
            m.stage_batch(u * MB, first[u * MB:(u + 1) * MB] if i == 0 else None, [pos0 + i] * MB, None if i == 0 else toks[u], toks[u])

    for i in range(warm):
        step(i)
    ctx.sync()
    e0, e1 = ctx.event(), ctx.event()
    l0 = ctx.launches
    ctx.record(e0)
    for i in range(warm, warm + steps):
        step(i)
    ctx.record(e1)
    ms = ctx.elapsed_ms(e0, e1) / steps
    launches = (ctx.launches - l0) // steps
    m.close()
    return {"value": S / (ms / 1000.0), "unit": "tok/s", "ms_per_step": ms, "streams": S, "context": CTX, "microbatch": MB,
            "gpu_launches_per_step": int(launches),
            "workload": "config 4 on one GPU: 64 sequences at context 8192, 2 passes of 32 sequences per decode step"}


def pipeline_main(a, base, rank, world, local, K, Wm):
    """N > 1: layer pipeline, 64 streams, context 8192 (see the module docstring)."""
    import torch
    import torch.distributed as dist
    from bonsai_vk_b200 import Context, Model, synth
    from bonsai_vk_b200.pipeline import Pipeline, ShardedHeadPipeline, TwoCudaStreams, split_blocks, split_head_rows
    torch.cuda.set_device(local)
    dist.init_process_group("nccl", device_id=torch.device("cuda", local))
    fwd, back = dist.new_group(list(range(world))), dist.new_group(list(range(world)))
    S, CTX = 64, 8192
    sharded = a.head == "sharded"
    # micro-batch = sequences that move through the stages together (one pass of the tensor-core projection kernel
    # reads the stage's weights once for all of them). Default: as many micro-batches as stages (32 / 16 / 8 sequences on 2 / 4 / 8 GPUs).
    MB = a.microbatch if a.microbatch > 0 else max(1, min(32, S // world))
    assert S % MB == 0, "the micro-batch size must divide 64"
    U = S // MB
    # "equal": the partition the benchmark configuration names (16 / 8 / 4 blocks per GPU). "bytes": the reference's own
    # rule (fleet_split_schedule: ranges balanced by bytes read per token, the output head charged to the last stage)
    bb = [48_923_392 if b % 4 != 3 else 45_910_016 for b in range(32)]
    b0, b1 = split_blocks(32, world, a.balance, block_bytes=bb, head_bytes=222_494_720)[rank]
    ctx = Context(local)
    # the same load on ONE GPU, measured by rank 0 on this box before the pipeline starts: the base of the scaling figure
    # (the N = 1 headline line of this file is a different metric, single-sequence decode)
    base1 = None
    if rank == 0 and not a.no_base:
        base1 = streams64_one_gpu(ctx)
        ctx.sync()
    dist.barrier()
    # one explicit (non-default) stream for our kernels and, through torch, for the NCCL dependencies: the legacy
    # default stream cannot be captured into the per-stream stage graphs
    work_stream = torch.cuda.Stream(device=local)
    torch.cuda.set_stream(work_stream)
    ctx.use_stream(work_stream.cuda_stream)
    hp = synth.HParams(cap=CTX, n_streams=S, block_begin=b0, block_end=b1, batch_cols=MB if MB > 1 else 0)
    tensors, signs = build_full_model(hp, head_everywhere=sharded)
    m = Model(ctx, hp, tensors, signs, head_rows=split_head_rows(hp.vocab, world)[rank] if sharded else None)
    del tensors
    total = 2 * (K + Wm) + 8
    pos0 = [CTX - total - 1] * U
    dev = torch.device("cuda", local)
    # Capture and instantiate every micro-batch's stage graph now, before any NCCL kernel is in flight: a graph
    # instantiation may synchronise the device, and a device that is running a send/recv kernel which waits
    # for its peer must not be asked to do that.
    width = MB * (hp.hidden if rank > 0 else 1)
    scratch_in = ctx.wrap(torch.zeros(MB * hp.hidden, dtype=torch.float32, device=dev).data_ptr(), MB * hp.hidden * 4)
    scratch_out = ctx.alloc(MB * hp.hidden * 4)
    for u in range(U):
        m.stage_prepare(u * MB if MB > 1 else u, MB if MB > 1 else 0)
        if MB > 1:
            m.stage_batch(u * MB, [1] * MB if rank == 0 else None, [pos0[u]] * MB, None if rank == 0 else scratch_in, scratch_out)
        else:
            m.stage(u, 1 if rank == 0 else 0, pos0[u], None if rank == 0 else scratch_in, scratch_out)
    if sharded:                  # first use of the head kernels, also before any NCCL kernel is in flight
        warm_c, warm_t = ctx.alloc(world * MB * 8), ctx.alloc(MB * 4)
        warm_c.memset(0)
        m.head_batch(MB, scratch_out, warm_c)
        m.pick_batch(MB, world, warm_c, warm_t)
    torch.cuda.synchronize()
    m.reset()
    for s in range(S):
        m.fill_kv(s, pos0[0])
    torch.cuda.synchronize()
    wraps = {}

    def wrap(t):
        key = t.data_ptr()
        if key not in wraps:
            wraps[key] = ctx.wrap(key, t.numel() * t.element_size())
        return wraps[key]

    def stage(u, step, pos, tok_first, tok_in, hin, out):
        if MB > 1:
            if rank == 0:
                m.stage_batch(u * MB, tok_first, [pos] * MB, wrap(tok_in) if tok_in is not None else None, wrap(out))
            else:
                m.stage_batch(u * MB, None, [pos] * MB, wrap(hin), wrap(out))
        elif rank == 0:
            m.stage(u, tok_first if tok_first is not None else -1, pos, wrap(tok_in) if tok_in is not None else None, wrap(out))
        else:
            m.stage(u, 0, pos, wrap(hin), wrap(out))

    if sharded:
        assert MB > 1, "the sharded head belongs to the multi-sequence pass"

        def head_fn(u, hfin, cand):
            m.head_batch(MB, wrap(hfin), wrap(cand))

        def pick_fn(u, allc, tok):
            m.pick_batch(MB, world, wrap(allc), wrap(tok))

        # BONSAI_PIPE_MARKS=1: CUDA events at the phase boundaries of every slot; per-phase device time is printed per rank
        marks = [] if os.environ.get("BONSAI_PIPE_MARKS") else None

        def mark(name):
            if marks is not None:
                ev = torch.cuda.Event(enable_timing=True)
                ev.record()
                marks.append((name, ev, time.perf_counter()))

        pipe = ShardedHeadPipeline(dist, rank, world, U, stage, head_fn, pick_fn,
                                   lambda: torch.zeros(MB * hp.hidden, dtype=torch.float32, device=dev),
                                   lambda: torch.zeros(MB, dtype=torch.int32, device=dev),
                                   lambda n: torch.zeros(n * MB * 2, dtype=torch.float32, device=dev), fwd, back, mark=mark,
                                   lanes=TwoCudaStreams(torch, ctx, work_stream, U) if a.head_lanes == 2 else None)
    else:
        pipe = Pipeline(dist, rank, world, U, stage, lambda: torch.zeros(MB * hp.hidden, dtype=torch.float32, device=dev),
                        lambda: torch.zeros(MB, dtype=torch.int32, device=dev), fwd, back)
    toks = [int(t) for t in np.random.default_rng(42).integers(0, hp.vocab, size=S)]
    first = [toks[u * MB:(u + 1) * MB] for u in range(U)] if MB > 1 else toks

    def timed(n_steps, p0, collect):
        torch.cuda.synchronize(); dist.barrier()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        l0 = ctx.launches
        e0.record()
        pipe.run(first, p0, n_steps, collect=collect)
        e1.record()
        torch.cuda.synchronize(); dist.barrier()
        tt = torch.tensor([e0.elapsed_time(e1)], device=dev, dtype=torch.float64)
        dist.all_reduce(tt, op=dist.ReduceOp.MAX)
        return float(tt[0]), ctx.launches - l0

    sampler = ClockSampler(local)
    sampler.start()
    timed(Wm, pos0, False)
    sampler.mark()
    p1 = [p + Wm for p in pos0]
    if sharded and marks is not None:
        marks.clear()
    ms_dev, launches = timed(K, p1, False)
    if sharded and marks is not None:
        import collections
        acc, host = collections.defaultdict(float), collections.defaultdict(float)
        for (n0, e0, h0), (n1, e1, h1) in zip(marks, marks[1:]):
            acc[n1] += e0.elapsed_time(e1)
            host[n1] += (h1 - h0) * 1e3
        slots = max(1, sum(1 for n, _, _ in marks if n == "stage"))
        print(f"[rank {rank}] per slot, device ms up to each mark: " + ", ".join(f"{k} {v / slots:.3f}" for k, v in acc.items())
              + " | host ms: " + ", ".join(f"{k} {v / slots:.3f}" for k, v in host.items()), file=sys.stderr, flush=True)
        marks.clear()
        marks = None
    clocks = sampler.stop()
    p2 = [p + K for p in p1]
    t0 = time.perf_counter()
    ms_e2e, _ = timed(K, p2, True)           # every pick is brought back to the host
    tok_s = S * K / (ms_dev / 1000.0)
    e2e = S * K / (ms_e2e / 1000.0)
    cfg = dict(base["config"], workload=f"config 4: 9B-shape synthetic model layer-pipelined over {world} GPUs "
               f"({b1 - b0} blocks per stage), 64 concurrent sequences at context {CTX} (KV marked filled) in {U} micro-batches "
               f"of {MB}, greedy decode; output head " + ("sharded by rows over the stages" if sharded else "on the last stage"),
               parallelism=f"pp{world}", streams=S, context=CTX, microbatch=MB, balance=a.balance, head=a.head,
               head_lanes=a.head_lanes if sharded else 1)
    # the 64-sequence workload is the same at every N: total work fixed
    line = dict(base, metric="decode tok/s, 9B ternary (PTQ1_0), 64 streams pipelined", scaling="strong", config=cfg, value=tok_s,
                ms_per_step=ms_dev / K, clocks=clocks, gpu_launches=int(launches),
                e2e={"value": e2e, "unit": "tok/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 4 * S})
    if rank == 0:
        if base1 is not None:
            # the driver's own efficiency divides by the N = 1 headline (another metric); this is the like-for-like figure
            line["scaling_base"] = base1
            line["scaling_efficiency_vs_base"] = tok_s / (world * base1["value"])
        peak, which = peaks()
        # per GPU and step: every micro-batch reads the stage's weights once; every sequence its own state and KV
        w_stage = (PTQ_BYTES_PER_TOKEN - 222_494_720) / world
        per_gpu = U * w_stage + S * ((2 * 50_331_648 + 29_411_328) / world) + S * (8 / world) * CTX * 2176
        ach = per_gpu / (ms_dev / K / 1000.0) / 1e9
        line["roofline"] = {"bound": "hbm", "achieved": ach, "peak": peak, "unit": "GB/s", "frac": ach / peak, "traffic": None,
                            "peak_source": which, "kernel": "per-GPU stage bytes per step (weights once per micro-batch + per-sequence state + KV)"}
        print(json.dumps(line))
    m.close()
    ctx.close()
    dist.destroy_process_group()


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=256)
    ap.add_argument("--warmup", type=int, default=8)
    ap.add_argument("--impl", default="ours")
    ap.add_argument("--prompt", type=int, default=16, help="prompt length in tokens (16 = the benchmark config)")
    ap.add_argument("--balance", default="equal", choices=["equal", "bytes"],
                    help="N > 1: stage split - equal block counts (the benchmark configuration) or byte-balanced with the head on the last stage")
    ap.add_argument("--head", default="sharded", choices=["sharded", "last"],
                    help="N > 1: output head sharded by rows over all stages (default) or whole on the last stage")
    ap.add_argument("--head-lanes", dest="head_lanes", type=int, default=1, choices=[1, 2],
                    help="N > 1, sharded head: 1 = head work on the stage passes' stream (default, measured faster), "
                         "2 = on a second high-priority CUDA stream beside them")
    ap.add_argument("--no-base", dest="no_base", action="store_true", help="N > 1: skip the one-GPU 64-stream base measurement")
    ap.add_argument("--microbatch", type=int, default=0, help="N > 1: sequences per micro-batch (0 = 64 / GPUs, at most 32; 1 = one sequence per pass)")
    a = ap.parse_args()
    rank = int(os.environ.get("RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    local = int(os.environ.get("LOCAL_RANK", "0"))
    K, Wm = max(1, a.steps), max(3, a.warmup)
    base = {"metric": "decode tok/s, 9B ternary (PTQ1_0), B=1 greedy", "unit": "tok/s", "n_gpus": a.gpus, "steps": K,
            "warmup": Wm, "higher_is_better": True, "scaling": "weak", "vs_baseline": None, "dtype": "u8 trits x int8 -> int32, fp32 scale",
            "data": "synthetic",
            "config": {"workload": "config 3: 9B-shape synthetic PTQ1_0 model, 32 blocks (24 GDN + 8 attention), prompt 16 ids "
                                   "then greedy decode, one stream per GPU", "l2": "inputs larger than L2 (1.87 GB read per token)",
                       "kv": "q8_0 K and V", "act": "q8_1"}}

    if a.impl == "reference":
        if rank != 0:
            return
        cb = cpu_gemv_tokens_per_s(seconds=min(60.0, 4.0 + 0.5 * (K + Wm)))
        line = dict(base, impl="reference", value=cb["value"], ms_per_step=1000.0 / cb["value"], cpu_baseline=cb,
                    e2e={"value": cb["value"], "unit": "tok/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
                    gpu_launches=0)
        if max(world, a.gpus) > 1:
            # the arm that is compared with the pipelined line: same metric, a step = one token of each of the 64 sequences.
            # The CPU path has no pipeline and no batching gain: its aggregate rate is its per-token rate.
            line.update(metric="decode tok/s, 9B ternary (PTQ1_0), 64 streams pipelined", scaling="strong", ms_per_step=64 * 1000.0 / cb["value"],
                        config=dict(base["config"], workload="config 4: 64 concurrent sequences of the 9B-shape synthetic model, greedy decode - the "
                                    "reference's CPU arithmetic on the host cores (projection weights only, as in the one-GPU arm)", streams=64))
        print(json.dumps(line))
        return

    from bonsai_vk_b200 import Context, Model, synth
    dist = None
    if world > 1:
        return pipeline_main(a, base, rank, world, local, K, Wm)
    ctx = Context(local)
    cap = max(256, (max(1, a.prompt) + 2 * (K + Wm) + 64 + 1) // 2 * 2)
    hp = synth.HParams(cap=cap)
    tensors, signs = build_full_model(hp)
    m = Model(ctx, hp, tensors, signs)
    tensors_cpu, signs_cpu = (tensors, signs) if rank == 0 else (None, None)     # kept for the CPU baseline's whole-token point
    del tensors
    prompt = [int(t) for t in np.random.default_rng(42).integers(0, hp.vocab, size=max(1, a.prompt))]
    nxt = 0
    for pos, t in enumerate(prompt):
        nxt = m.token(t, pos)
    pos = len(prompt)

    def barrier():
        ctx.sync()
        if dist is not None:
            dist.barrier()

    # ---- device-resident: warm-up then K chained tokens ------------------------------------------------
    sampler = ClockSampler(local)
    sampler.start()
    out = m.decode(nxt, pos, Wm)
    nxt, pos = out[-1], pos + Wm
    e0, e1 = ctx.event(), ctx.event()
    barrier()
    sampler.mark()
    l0 = ctx.launches
    ctx.record(e0)
    m.decode(nxt, pos, K, fetch=False)
    ctx.record(e1)
    ms_dev = ctx.elapsed_ms(e0, e1)
    barrier()
    launches = ctx.launches - l0
    pos += K
    # ---- end to end through the per-token call ---------------------------------------------------------
    t = 1
    for i in range(3):
        t = m.token(t, pos); pos += 1
    barrier()
    ctx.record(e0)
    for i in range(K):
        t = m.token(t, pos); pos += 1
    ctx.record(e1)
    ms_e2e = ctx.elapsed_ms(e0, e1)
    barrier()
    clocks = sampler.stop()          # covers both timed regions (device-chained and per-token)

    if dist is not None:
        import torch
        tt = torch.tensor([ms_dev, ms_e2e], device="cuda", dtype=torch.float64)
        dist.all_reduce(tt, op=dist.ReduceOp.MAX)
        ms_dev, ms_e2e = float(tt[0]), float(tt[1])
    tok_s = world * K / (ms_dev / 1000.0)
    e2e_tok_s = world * K / (ms_e2e / 1000.0)

    line = dict(base, value=tok_s, ms_per_step=ms_dev / K, clocks=clocks, gpu_launches=int(launches),
                e2e={"value": e2e_tok_s, "unit": "tok/s", "h2d_bytes_per_step": 8, "d2h_bytes_per_step": 4})
    if rank == 0:
        peak, which = peaks()
        # dominant kernel: the PTQ1_0 GEMV. Its 201 launches of one token, back to back over the model's own
        # weights (1.73 GB, far larger than L2), timed with events on the launch stream.
        reps = 3
        l1 = ctx.launches
        ms_g = m.gemv_sweep_ms(reps=reps)
        n_l = (ctx.launches - l1) // (reps + 1)
        ach = PTQ_BYTES_PER_TOKEN / (ms_g / 1000.0) / 1e9
        # DRAM bytes per algorithmic byte of k_phase_gemv, from the ncu capture summarised under profiles/
        # (head projection: 227.7 MB moved for 222.5 MB of weights); the sweep's launches move the same ratio
        line["roofline"] = {"bound": "hbm", "achieved": ach, "peak": peak, "unit": "GB/s", "frac": ach / peak,
                            "traffic": NCU_TRAFFIC_RATIO * PTQ_BYTES_PER_TOKEN / n_l, "peak_source": which,
                            "kernel": f"k_phase_gemv: the {n_l} fused projection launches of one token (201 projections, "
                                      "grouped where they share an input), with their prologues, back to back",
                            "algorithmic_bytes_per_launch": PTQ_BYTES_PER_TOKEN / n_l,
                            "avg_launch_us": ms_g * 1000.0 / n_l,
                            "token_level": {"algorithmic_bytes_per_token": ALGO_BYTES_PER_TOKEN,
                                            "achieved_gbs": ALGO_BYTES_PER_TOKEN / (ms_dev / K / 1000.0) / 1e9,
                                            "frac_of_measured": ALGO_BYTES_PER_TOKEN / (ms_dev / K / 1000.0) / 1e9 / peak,
                                            "frac_of_8000": ALGO_BYTES_PER_TOKEN / (ms_dev / K / 1000.0) / 1e9 / 8000.0}}
        # the other kernels of the path, each against the same measured peak (algorithmic bytes / device time):
        # the recurrent core at this run's position, then - after the model is gone - attention and the multi-column
        # projection through the op-level C ABI on buffers larger than L2
        us_gdn, _ = m.mixer_sweep_us(reps=5)
        others = [{"kernel": "k_gdn_split: gated-delta-net core of one layer (2 MiB state read + written, the layer's state of the "
                             "previous token is still in L2)", "algorithmic_bytes": 4_194_304 + 98_304, "us": us_gdn,
                   "achieved": (4_194_304 + 98_304) / us_gdn / 1e3, "frac": (4_194_304 + 98_304) / us_gdn / 1e3 / peak}]
        line["cpu_baseline"] = cpu_gemv_tokens_per_s(seconds=12.0)
        # the end-to-end CPU point: whole decode tokens of this workload through the CPU checker's forward (integer
        # block dots, fp32 scales - the same arithmetic as the GPU path), single-threaded: 2 tokens after a 1-token prompt
        try:
            from tests._oracle import OracleModel
            t_cpu = time.perf_counter()
            om = OracleModel(hp, tensors_cpu, signs_cpu, threads=1)
            ol, _ = om.token(1, 0)
            t1 = time.perf_counter()
            for i in range(2):
                ol, _ = om.token(om.argmax(ol), 1 + i)
            dt = (time.perf_counter() - t1) / 2
            om.close()
            line["cpu_baseline"]["full_token"] = {"value": 1.0 / dt, "unit": "tok/s", "cores": 1, "kind": "port",
                                                  "sample": "2 whole decode tokens of the 9B-shape model through the CPU checker, single thread"}
        except Exception as exc:
            line["cpu_baseline"]["full_token"] = {"error": str(exc)[:200]}
    m.close()
    if rank == 0:
        from bonsai_vk_b200 import kernel_lab
        try:
            for keys in (4096, 32768):
                ms_a, nb = kernel_lab.attn_lab([str(keys), "10"], ctx=ctx, quiet=True)
                others.append({"kernel": f"decode attention, one layer, {keys} keys (prep, scores, softmax sums, PV, combine; q8_0 K and V)",
                               "algorithmic_bytes": nb, "us": ms_a * 1e3, "achieved": nb / ms_a / 1e6, "frac": nb / ms_a / 1e6 / peak})
            for ncol in (8, 32):
                ms_g2, nb = kernel_lab.gemm_lab(["18944", "4096", str(ncol), "3"], ctx=ctx, quiet=True)
                others.append({"kernel": f"k_ptq_gemm_tc: 18944 x 4096 projection, {ncol} sequences per pass (tcgen05 kind::i8)",
                               "algorithmic_bytes": nb, "us": ms_g2 * 1e3, "achieved": nb / ms_g2 / 1e6, "frac": nb / ms_g2 / 1e6 / peak})
        except Exception as exc:
            others.append({"error": str(exc)[:200]})
        line["roofline"]["others"] = others
    if rank == 0:
        # the 64-sequence workload of config 4 on this one GPU (no pipeline): the base of the multi-GPU scaling
        try:
            line["streams64"] = streams64_one_gpu(ctx, tensors_again=None)
        except Exception as exc:                       # the headline line must survive a failure of the extra measurement
            line["streams64"] = {"error": str(exc)[:200]}
        print(json.dumps(line))
    ctx.close()
    if dist is not None:
        dist.destroy_process_group()


if __name__ == "__main__":
    main()
