"""Host side of the sparse drafter head: WHICH vocabulary columns the draft steps use, and WHETHER they use them.

* counts: a generated token adds 1, a prompt token ``prompt_weight``; all counts halve every ``decay_tokens`` generated tokens;
* subset: the ``capacity`` ids with the largest counts, an incumbent's count weighted by ``1 + swap_margin`` so that a
  challenger must clearly beat it; proposed again every ``interval`` generated tokens once ``min_evidence`` has been seen,
  and only when at least ``min_change`` of the subset would change (an extraction costs a few passes over the full head);
* use: a committed token outside the subset is a draft miss that the sparse head caused. Drafting through the subset pays
  while the miss rate stays below ``2 * (time saved per round) / (round time)``; the step times of both modes are running
  averages (one full round every ``full_probe_rounds`` sparse rounds keeps the full head's time fresh) and the decision has
  hysteresis (1.2x to stay on, 0.8x to switch on).
Counts persist between runs in a small file (magic, vocabulary size, evidence, fp32 counts).

Reference: inc/engine/runtime/sparse_head_policy.h:9-72, src/runtime/sparse_head_policy.cpp (constants and the break-even rule).
"""
from __future__ import annotations

import os
import struct
from dataclasses import dataclass

import numpy as np

MISS_EMA = 1.0 / 512.0      # time constant of the miss rate, in committed tokens
TIME_EMA = 0.05             # weight of a new round in the timing averages
MIN_SCORED = 64             # committed tokens scored against a subset before it may be used
SAVE_EVERY = 4096
MAGIC = 0x53504844          # "DHPS" little-endian


@dataclass
class SparseHeadParams:
    capacity: int = 16384
    interval: int = 2048
    decay_tokens: int = 8192
    swap_margin: float = 0.25
    prompt_weight: float = 0.2
    min_evidence: float = 256.0
    min_change: float = 0.02
    full_probe_rounds: int = 256


class SparseHeadPolicy:
    def __init__(self, vocab: int, params: SparseHeadParams | None = None):
        self.p = params or SparseHeadParams()
        self.vocab = vocab
        self.counts = np.zeros(vocab, dtype=np.float32)
        self.member = np.zeros(vocab, dtype=bool)
        self.subset_n = 0
        self.evidence = 0.0
        self.since_rebuild = self.since_decay = self.since_save = 0
        self.built = False
        self.miss = 0.0
        self.scored = 0
        self.t_full = self.t_sparse = self.t_round = self.steps = 0.0
        self.on = False
        self.sparse_rounds = 0

    # ------------------------------------------------------------------------------------------ evidence
    def observe_prompt(self, tokens) -> None:
        t = np.asarray(tokens, dtype=np.int64)
        t = t[(t >= 0) & (t < self.vocab)]
        np.add.at(self.counts, t, np.float32(self.p.prompt_weight))
        self.evidence += self.p.prompt_weight * len(tokens)

    def observe_generated(self, token: int) -> None:
        if not 0 <= token < self.vocab:
            return
        self.counts[token] += 1.0
        self.evidence += 1.0
        self.since_save += 1
        self.since_rebuild += 1
        self.since_decay += 1
        if self.since_decay >= self.p.decay_tokens:
            self.counts *= 0.5
            self.evidence *= 0.5
            self.since_decay = 0
        if self.built:       # a plain mean over the first tokens scored against a subset, then the exponential average
            self.scored += 1
            self.miss += ((0.0 if self.member[token] else 1.0) - self.miss) * max(MISS_EMA, 1.0 / self.scored)

    # ------------------------------------------------------------------------------------------ subset
    def ranked(self) -> list[int]:
        """The ids the next subset would hold, most important first (ties to the lower id)."""
        ids = np.nonzero((self.counts > 0) | self.member)[0]
        score = self.counts[ids] * np.where(self.member[ids], np.float32(1.0 + self.p.swap_margin), np.float32(1.0))
        order = np.lexsort((ids, -score))
        return ids[order][: self.p.capacity].tolist()

    def rebuild_due(self) -> bool:
        if self.evidence < self.p.min_evidence:
            return False
        if self.built and self.since_rebuild < self.p.interval:
            return False
        self.since_rebuild = 0
        if not self.built:
            return True
        nxt = self.ranked()
        changed = int((~self.member[np.asarray(nxt, dtype=np.int64)]).sum()) if nxt else 0
        return changed >= self.p.min_change * max(self.subset_n, 1)

    def set_subset(self, kept) -> None:
        self.member[:] = False
        k = np.asarray(list(kept), dtype=np.int64)
        k = k[(k >= 0) & (k < self.vocab)]
        self.member[k] = True
        self.subset_n = len(kept)
        if not self.built:
            self.scored = 0          # the first subset is scored from scratch; later ones continue the average
        self.built = self.subset_n > 0

    # ------------------------------------------------------------------------------------------ timing and the decision
    def draft_step_time(self, sparse: bool, ms: float) -> None:
        if sparse:
            self.t_sparse = self.t_sparse + (ms - self.t_sparse) * TIME_EMA if self.t_sparse > 0 else ms
        else:
            self.t_full = self.t_full + (ms - self.t_full) * TIME_EMA if self.t_full > 0 else ms

    def round_time(self, ms: float, draft_steps: int) -> None:
        self.t_round = self.t_round + (ms - self.t_round) * TIME_EMA if self.t_round > 0 else ms
        self.steps = self.steps + (draft_steps - self.steps) * TIME_EMA if self.steps > 0 else float(draft_steps)

    def breakeven(self) -> float:
        saving = max(0.0, self.t_full - self.t_sparse) * max(self.steps, 1.0)
        return 2.0 * saving / self.t_round if self.t_round > 0 else 0.0

    force = False          # draft through the subset whenever one exists, whatever the miss rate (A/B measurement)

    def use_sparse(self) -> bool:
        """Whether the next round drafts through the subset."""
        if self.force and self.built:
            self.on = True
            return True
        if not self.built or self.t_full <= 0 or self.scored < MIN_SCORED:
            self.on = False
            return False
        if self.t_sparse <= 0:           # measure the sparse steps once
            self.on = True
            return True
        if self.on:
            self.sparse_rounds += 1
            if self.sparse_rounds >= self.p.full_probe_rounds:
                self.sparse_rounds = 0
                return False             # one full round refreshes the full head's step time (the mode stays on)
        self.on = self.miss < self.breakeven() * (1.2 if self.on else 0.8)
        return self.on

    # ------------------------------------------------------------------------------------------ persistence
    def save_due(self) -> bool:
        if self.since_save < SAVE_EVERY:
            return False
        self.since_save = 0
        return True

    def save(self, path) -> bool:
        if not path or self.evidence <= 0:
            return False
        tmp = str(path) + ".tmp"
        with open(tmp, "wb") as f:
            f.write(struct.pack("<IId", MAGIC, self.vocab, self.evidence))
            f.write(self.counts.tobytes())
        os.replace(tmp, path)
        return True

    def load(self, path) -> bool:
        try:
            with open(path, "rb") as f:
                head = f.read(16)
                if len(head) != 16:
                    return False
                magic, vocab, ev = struct.unpack("<IId", head)
                raw = f.read(4 * self.vocab)
        except OSError:
            return False
        if magic != MAGIC or vocab != self.vocab or len(raw) != 4 * self.vocab:
            return False
        self.counts = np.frombuffer(raw, dtype=np.float32).copy()
        self.evidence = ev
        return True
