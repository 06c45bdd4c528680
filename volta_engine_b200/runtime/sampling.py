"""Host-side sampler over top-16 candidates.

Same contract as the reference sampler (inc/engine/runtime/sampling.h:9-15,82-110,115-167,197-223):
the device produces, per row, the 16 best logits of every vocabulary shard (+ shard log-sum-exp); the host
merges shards, applies presence / frequency / repetition penalties to the candidates, temperature,
top-k (<= 16), top-p inside the candidates, and draws with xoshiro256++ seeded through splitmix64.
Greedy picks the best candidate (ties -> lowest id). ``spec_step`` is the exact speculative-sampling
acceptance against a point-mass proposal (the drafters propose one token per position).
"""
from __future__ import annotations

import math
from dataclasses import dataclass, field

MASK64 = (1 << 64) - 1
NUM_CANDIDATES = 16


def _rotl(x: int, k: int) -> int:
    return ((x << k) | (x >> (64 - k))) & MASK64


class Xoshiro256pp:
    """xoshiro256++ with splitmix64 seeding."""

    def __init__(self, seed: int):
        s = seed & MASK64
        self.s = []
        for _ in range(4):
            s = (s + 0x9E3779B97F4A7C15) & MASK64
            z = s
            z = ((z ^ (z >> 30)) * 0xBF58476D1CE4E5B9) & MASK64
            z = ((z ^ (z >> 27)) * 0x94D049BB133111EB) & MASK64
            self.s.append(z ^ (z >> 31))

    def next_u64(self) -> int:
        s = self.s
        result = (_rotl((s[0] + s[3]) & MASK64, 23) + s[0]) & MASK64
        t = (s[1] << 17) & MASK64
        s[2] ^= s[0]
        s[3] ^= s[1]
        s[1] ^= s[2]
        s[0] ^= s[3]
        s[2] ^= t
        s[3] = _rotl(s[3], 45)
        return result

    def uniform(self) -> float:
        return (self.next_u64() >> 11) * (1.0 / (1 << 53))


@dataclass
class SamplingParams:
    temperature: float = 0.0
    top_p: float = 1.0
    top_k: int = 0
    presence_penalty: float = 0.0
    frequency_penalty: float = 0.0
    repetition_penalty: float = 1.0
    seed: int | None = None
    logprobs: int = 0

    @property
    def greedy(self) -> bool:
        return self.temperature <= 0.0


@dataclass
class Candidates:
    ids: list[int]
    logits: list[float]
    lse: float = float("nan")       # log-sum-exp over the full vocabulary (for logprobs)


def merge_shards(shards: list[Candidates], k: int = NUM_CANDIDATES) -> Candidates:
    """Merge per-shard top-k lists (descending) and shard LSEs into one candidate list."""
    pairs = []
    for sh in shards:
        pairs.extend((l, i) for i, l in zip(sh.ids, sh.logits) if i >= 0)
    pairs.sort(key=lambda p: (-p[0], p[1]))
    pairs = pairs[:k]
    lses = [sh.lse for sh in shards if not math.isnan(sh.lse)]
    lse = float("nan")
    if lses:
        m = max(lses)
        lse = m + math.log(sum(math.exp(x - m) for x in lses))
    return Candidates([p[1] for p in pairs], [p[0] for p in pairs], lse)


def penalize(c: Candidates, p: SamplingParams, counts: dict[int, int]) -> Candidates:
    if not counts or (p.presence_penalty == 0 and p.frequency_penalty == 0 and p.repetition_penalty == 1.0):
        return c
    out = []
    for i, l in zip(c.ids, c.logits):
        n = counts.get(i, 0)
        if n:
            if p.repetition_penalty != 1.0:
                l = l / p.repetition_penalty if l > 0 else l * p.repetition_penalty
            l -= p.presence_penalty + p.frequency_penalty * n
        out.append(l)
    order = sorted(range(len(out)), key=lambda k: (-out[k], c.ids[k]))
    return Candidates([c.ids[k] for k in order], [out[k] for k in order], c.lse)


def distribution(c: Candidates, p: SamplingParams) -> list[float]:
    """Probabilities over the candidates after temperature, top-k and top-p (renormalised)."""
    n = len(c.ids)
    if n == 0:
        return []
    if p.greedy:
        return [1.0] + [0.0] * (n - 1)
    k = min(n, p.top_k) if p.top_k and p.top_k > 0 else n
    m = c.logits[0]
    w = [math.exp((l - m) / p.temperature) for l in c.logits[:k]]
    tot = sum(w)
    w = [x / tot for x in w]
    if p.top_p < 1.0:
        acc, keep = 0.0, 0
        for x in w:
            acc += x
            keep += 1
            if acc >= p.top_p:
                break
        w = w[:keep]
        tot = sum(w)
        w = [x / tot for x in w]
    return w + [0.0] * (n - len(w))


def sample_token(c: Candidates, p: SamplingParams, rng: Xoshiro256pp | None) -> int:
    if p.greedy or rng is None:
        return c.ids[0]
    probs = distribution(c, p)
    u = rng.uniform()
    acc = 0.0
    for i, q in zip(c.ids, probs):
        acc += q
        if u < acc:
            return i
    return next(i for i, q in reversed(list(zip(c.ids, probs))) if q > 0)


def logprob_of(c: Candidates, token: int) -> float:
    """log p(token) under the unmodified model distribution (needs the full-vocabulary LSE)."""
    for i, l in zip(c.ids, c.logits):
        if i == token:
            return l - c.lse
    return float("-inf")


def spec_step(c: Candidates, p: SamplingParams, draft: int, rng: Xoshiro256pp | None) -> tuple[bool, int]:
    """Exact speculative sampling for a point-mass proposal q = delta(draft).

    Accept with probability p(draft); on rejection draw from the residual (p with the draft removed,
    renormalised). Returns (accepted, token). Greedy: accepted iff the draft is the argmax.
    """
    if p.greedy or rng is None:
        return (c.ids[0] == draft, c.ids[0])
    probs = distribution(c, p)
    pd = 0.0
    for i, q in zip(c.ids, probs):
        if i == draft:
            pd = q
    if rng.uniform() < pd:
        return True, draft
    rest = [(i, q) for i, q in zip(c.ids, probs) if i != draft and q > 0]
    tot = sum(q for _, q in rest)
    if tot <= 0:
        return True, draft
    u = rng.uniform() * tot
    acc = 0.0
    for i, q in rest:
        acc += q
        if u < acc:
            return False, i
    return False, rest[-1][0]


@dataclass
class TokenCounts:
    """Per-request occurrence counts for the penalties."""
    counts: dict[int, int] = field(default_factory=dict)

    def add(self, tok: int) -> None:
        self.counts[tok] = self.counts.get(tok, 0) + 1
