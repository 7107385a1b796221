"""The host-side sampler against an independent scalar restatement of the reference's `Sampler::pick`
(runtime_vk/bonsai_forward.h:2525-2600) and against the properties its parts must have. No GPU."""
import math

import numpy as np
import pytest

from bonsai_vk_b200.sampler import Sampler, sampler_from_request


def _scalar_pick(lg, hist, temp, top_k, top_p, rng, rep, pres, freq, last_n):
    """The reference's algorithm written out element by element (float32 where it computes in float, Python floats
    where it computes in double). Returns (token, rng state after)."""
    f = np.float32
    n = len(lg)
    lg = [f(v) for v in lg]
    if hist and (rep != 1.0 or pres != 0.0 or freq != 0.0):
        win = hist[-last_n:] if last_n > 0 else hist
        cnt = {}
        for t in win:
            if 0 <= t < n:
                cnt[t] = cnt.get(t, 0) + 1
        for t, c in cnt.items():
            v = lg[t]
            if rep != 1.0:
                v = f(v * f(rep)) if v < 0 else f(v / f(rep))
            if pres != 0.0:
                v = f(v - f(pres))
            if freq != 0.0:
                v = f(v - f(f(freq) * f(c)))
            lg[t] = v
    best, bv = 0, lg[0]
    for i in range(1, n):
        if lg[i] > bv:
            bv, best = lg[i], i
    if temp <= 0.0:
        return best, rng
    floor_v = f(-3.4e38)
    if 0 < top_k < n:
        floor_v = sorted(lg, reverse=True)[top_k - 1]
    pr, total = [0.0] * n, 0.0
    for i in range(n):
        if lg[i] < floor_v:
            continue
        pr[i] = math.exp(float(f(f(lg[i] - bv) / f(temp))))
        total += pr[i]
    if total <= 0.0:
        return best, rng
    if top_p < 1.0:
        idx = sorted((i for i in range(n) if pr[i] > 0.0), key=lambda i: (-pr[i], i))
        c, keep = 0.0, len(idx)
        for j, i in enumerate(idx):
            c += pr[i] / total
            if c >= top_p:
                keep = j + 1
                break
        for i in idx[keep:]:
            total -= pr[i]
            pr[i] = 0.0
    M = (1 << 64) - 1
    rng ^= rng >> 12; rng ^= (rng << 25) & M; rng ^= rng >> 27
    u = float(((rng * 2685821657736338717) & M) >> 11) * (1.0 / 9007199254740992.0) * total
    a = 0.0
    for i in range(n):
        a += pr[i]
        if a >= u:
            return i, rng
    return best, rng


@pytest.mark.parametrize("cfg", [dict(temp=0.7, top_k=0, top_p=1.0), dict(temp=1.3, top_k=5, top_p=1.0), dict(temp=0.9, top_k=0, top_p=0.8),
                                 dict(temp=0.5, top_k=12, top_p=0.6), dict(temp=0.0, top_k=0, top_p=1.0)])
def test_matches_the_scalar_restatement(cfg):
    rng = np.random.default_rng(3)
    for case in range(40):
        n = int(rng.integers(8, 200))
        logits = (rng.standard_normal(n) * 3).astype(np.float32)
        hist = [int(t) for t in rng.integers(0, n + 3, size=int(rng.integers(0, 100)))]
        rep, pres, freq, last_n = (1.15, 0.5, 0.0, 64) if case % 2 == 0 else (1.3, 0.0, 0.25, 0)
        seed = int(rng.integers(1, 2 ** 62))
        s = Sampler(seed=seed, rep_penalty=rep, presence_penalty=pres, freq_penalty=freq, penalty_last_n=last_n, **cfg)
        got = s.pick(logits, hist)
        want, state = _scalar_pick(list(logits), hist, cfg["temp"], cfg["top_k"], cfg["top_p"], seed, rep, pres, freq, last_n)
        assert got == want, (case, cfg)
        assert s.rng == state, "the generator advances exactly when the reference's does"


def test_generator_is_xorshift64_star():
    s = Sampler()
    x = 88172645463325252
    M = (1 << 64) - 1
    for _ in range(5):
        x ^= x >> 12; x ^= (x << 25) & M; x ^= x >> 27
        assert s.next_rand() == (x * 2685821657736338717) & M
    assert 0.0 <= s.uniform01() < 1.0


def test_parts_behave():
    lg = np.array([0.0, math.log(3.0), -50.0], dtype=np.float32)
    assert Sampler(temp=0.0).pick(lg) == 1
    assert Sampler(temp=5.0, top_k=1).pick(lg) == 1                       # only the largest survives
    s = Sampler(temp=1.0, rep_penalty=1.0, presence_penalty=0.0)
    draws = np.bincount([s.pick(lg) for _ in range(8000)], minlength=3)
    assert draws[2] == 0 and abs(draws[1] / 8000 - 0.75) < 0.02          # 1 : 3
    lg3 = np.log(np.array([0.5, 0.3, 0.2], dtype=np.float32))
    s = Sampler(temp=1.0, top_p=0.6, rep_penalty=1.0, presence_penalty=0.0)
    assert set(s.pick(lg3) for _ in range(500)) == {0, 1}                # 0.5 + 0.3 reaches 0.6, the tail is cut
    # penalties: positive logits shrink, negative ones grow in magnitude, presence once, frequency per occurrence
    pen = Sampler(rep_penalty=2.0, presence_penalty=0.5, freq_penalty=0.25).penalised(np.array([4.0, -4.0, 1.0], dtype=np.float32), [0, 1, 1, 7])
    assert np.allclose(pen, [4.0 / 2 - 0.5 - 0.25, -4.0 * 2 - 0.5 - 0.5, 1.0])


def test_request_fields():
    assert sampler_from_request({}) is None and sampler_from_request({"temperature": 0}) is None
    s = sampler_from_request({"temperature": 0.9, "top_k": 40, "top_p": 0.95, "seed": 7, "repetition_penalty": 1.2, "presence_penalty": -1})
    assert (s.temp, s.top_k, s.top_p, s.rng, s.rep_penalty, s.presence_penalty) == (0.9, 40, 0.95, 7, 1.2, 0.5)


@pytest.mark.parametrize("env", [dict(BONSAI_TEMP="0.7"), dict(BONSAI_TEMP="1.1", BONSAI_TOPK="7", BONSAI_SEED="12345"),
                                 dict(BONSAI_TEMP="0.9", BONSAI_TOPP="0.7", BONSAI_REP_PENALTY="1.3", BONSAI_PRESENCE="0", BONSAI_FREQ="0.2")])
def test_cpp_host_sampler_equals_the_python_one(env):
    """The `run` command's sampler (host/bonsai_sampler.h) through `bonsai_run sampler-check` (no GPU needed): the same picks
    and the same generator states as sampler.Sampler over a sequence of cases that share one generator."""
    import os
    import subprocess

    from bonsai_vk_b200 import build
    exe = build.build_host()
    rng = np.random.default_rng(5)
    py = Sampler(temp=float(env["BONSAI_TEMP"]), top_k=int(env.get("BONSAI_TOPK", 0)), top_p=float(env.get("BONSAI_TOPP", 1.0)),
                 seed=int(env.get("BONSAI_SEED", 88172645463325252)), rep_penalty=float(env.get("BONSAI_REP_PENALTY", 1.15)),
                 presence_penalty=float(env.get("BONSAI_PRESENCE", 0.5)), freq_penalty=float(env.get("BONSAI_FREQ", 0.0)))
    text, want = [], []
    for _ in range(30):
        n = int(rng.integers(5, 120))
        logits = (rng.standard_normal(n) * 3).astype(np.float32)
        hist = [int(t) for t in rng.integers(0, n, size=int(rng.integers(0, 90)))]
        text.append(f"{n} " + " ".join(repr(float(v)) for v in logits) + f" {len(hist)} " + " ".join(map(str, hist)))
        t = py.pick(logits, hist)
        want.append(f"{t} {py.rng}")
    r = subprocess.run([exe, "sampler-check"], input="\n".join(text) + "\n0\n", capture_output=True, text=True, env=dict(os.environ, **env), timeout=60)
    assert r.returncode == 0, r.stderr
    assert r.stdout.split("\n")[:len(want)] == want
