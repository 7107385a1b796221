"""Host-side token sampler: what the reference's `Sampler::pick` does with a row of logits
(runtime_vk/bonsai_forward.h:2525-2600), restated over numpy arrays.

Order of operations, as there: repetition / presence / frequency penalties on a COPY of the logits over a window of
the recent generation (a positive logit is divided by the repetition penalty, a negative one multiplied; presence is
subtracted once per distinct token, frequency in proportion to its count); first maximum; temperature <= 0 returns it;
top-k keeps the logits not below the k-th largest; probabilities exp((logit - max) / temperature) in double, summed in
index order; top-p sorts the candidates by probability and cuts the tail past the cumulative mass; one xorshift64*
draw picks the first index whose running sum reaches u * sum. The float32 / float64 split of the arithmetic is the
reference's (penalties and the scaled difference in float32, exponentials and sums in float64).

The reference samples by default (temperature 0.70, repetition 1.15, presence 0.50); the server of this package picks
greedily on the device unless a request asks for a temperature above zero, and only then uses this class.
One difference that cannot show in a result: the reference's std::sort leaves the order of equal probabilities
unspecified, here equal probabilities keep their index order."""
from __future__ import annotations

from typing import Optional, Sequence

import numpy as np

_M64 = (1 << 64) - 1


class Sampler:
    def __init__(self, temp: float = 0.70, top_k: int = 0, top_p: float = 1.0, seed: int = 88172645463325252,
                 rep_penalty: float = 1.15, presence_penalty: float = 0.50, freq_penalty: float = 0.0, penalty_last_n: int = 64):
        self.temp, self.top_k, self.top_p = float(temp), int(top_k), float(top_p)
        self.rng = int(seed) & _M64 or 88172645463325252          # xorshift state must not be zero
        self.rep_penalty, self.presence_penalty, self.freq_penalty = float(rep_penalty), float(presence_penalty), float(freq_penalty)
        self.penalty_last_n = int(penalty_last_n)

    # xorshift64*, deterministic across runs (bonsai_forward.h:2538-2542)
    def next_rand(self) -> int:
        x = self.rng
        x ^= x >> 12
        x ^= (x << 25) & _M64
        x ^= x >> 27
        self.rng = x
        return (x * 2685821657736338717) & _M64

    def uniform01(self) -> float:
        return float(self.next_rand() >> 11) * (1.0 / 9007199254740992.0)

    def penalised(self, logits: np.ndarray, hist: Optional[Sequence[int]]) -> np.ndarray:
        lg = np.asarray(logits, dtype=np.float32)
        if not hist or (self.rep_penalty == 1.0 and self.presence_penalty == 0.0 and self.freq_penalty == 0.0):
            return lg
        window = list(hist[-self.penalty_last_n:]) if self.penalty_last_n > 0 else list(hist)
        ids, counts = np.unique(np.asarray([t for t in window if 0 <= t < lg.size], dtype=np.int64), return_counts=True)
        if ids.size == 0:
            return lg
        work = lg.copy()
        v = work[ids]
        if self.rep_penalty != 1.0:
            r = np.float32(self.rep_penalty)
            v = np.where(v < 0, v * r, v / r).astype(np.float32)
        if self.presence_penalty != 0.0:
            v = (v - np.float32(self.presence_penalty)).astype(np.float32)
        if self.freq_penalty != 0.0:
            v = (v - np.float32(self.freq_penalty) * counts.astype(np.float32)).astype(np.float32)
        work[ids] = v
        return work

    def pick(self, logits: np.ndarray, hist: Optional[Sequence[int]] = None) -> int:
        lg = self.penalised(logits, hist)
        n = lg.size
        best = int(np.argmax(lg))                                  # first maximum
        if self.temp <= 0.0:
            return best
        bv = lg[best]
        floor_v = np.float32(-3.4e38)
        if 0 < self.top_k < n:
            floor_v = np.partition(lg, n - self.top_k)[n - self.top_k]      # the k-th largest logit is the floor
        scaled = ((lg - bv) / np.float32(self.temp)).astype(np.float64)
        pr = np.where(lg < floor_v, 0.0, np.exp(scaled))
        total = float(np.cumsum(pr)[-1])                           # summed in index order
        if not total > 0.0:
            return best
        if self.top_p < 1.0:
            idx = np.flatnonzero(pr > 0.0)
            idx = idx[np.argsort(-pr[idx], kind="stable")]
            c = np.cumsum(pr[idx] / total)
            reach = np.flatnonzero(c >= self.top_p)
            keep = int(reach[0]) + 1 if reach.size else idx.size
            for j in idx[keep:]:                                   # the reference subtracts the cut tail term by term
                total -= float(pr[j])
                pr[j] = 0.0
        u = self.uniform01() * total
        hit = np.flatnonzero(np.cumsum(pr) >= u)
        return int(hit[0]) if hit.size else best


def sampler_from_request(req: dict) -> Optional[Sampler]:
    """The request fields the reference reads (runtime_vk/bonsai_http.h:595-608: temperature, top_p, top_k, seed,
    repetition_penalty, presence_penalty, frequency_penalty; a negative or absent value leaves the default). Returns None
    when the request does not ask for a temperature above zero: the device's greedy pick is used then."""
    def num(key, default):
        v = req.get(key, None)
        return default if not isinstance(v, (int, float)) or isinstance(v, bool) or v < 0 else v

    temp = num("temperature", 0.0)
    if not temp > 0.0:
        return None
    seed = req.get("seed", 0)
    s = Sampler(temp=temp, top_k=int(num("top_k", 0)), top_p=num("top_p", 1.0),
                rep_penalty=num("repetition_penalty", 1.15), presence_penalty=num("presence_penalty", 0.50),
                freq_penalty=num("frequency_penalty", 0.0))
    if isinstance(seed, (int, float)) and not isinstance(seed, bool) and seed > 0:
        s.rng = int(seed) & _M64
    return s
