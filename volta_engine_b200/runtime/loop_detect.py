"""Detection of degenerate repetition in generated tokens by rolling-hash period search.

Reference behaviour (inc/engine/runtime/loop_detect.h, src/runtime/loop_detect.cpp): a request whose tail
repeats the same k-gram with a fixed period for long enough is finished with reason ``loop``.
"""
from __future__ import annotations


class LoopDetector:
    def __init__(self, min_period: int = 1, max_period: int = 256, min_repeats: int = 4, min_span: int = 64):
        self.min_period, self.max_period = min_period, max_period
        self.min_repeats, self.min_span = min_repeats, min_span
        self.toks: list[int] = []
        self._run = {}   # period -> current run length of toks[i] == toks[i - period]

    def push(self, tok: int) -> bool:
        """Append a token; True when the tail is periodic (period p repeated >= min_repeats times and the
        periodic span covers >= min_span tokens)."""
        t = self.toks
        t.append(tok)
        n = len(t)
        hit = False
        for p in range(self.min_period, min(self.max_period, n - 1) + 1):
            if t[n - 1] == t[n - 1 - p]:
                r = self._run.get(p, 0) + 1
                self._run[p] = r
                span = r + p
                if span >= max(self.min_span, p * self.min_repeats):
                    hit = True
            elif p in self._run:
                del self._run[p]
        return hit

    def reset(self):
        self.toks.clear()
        self._run.clear()
