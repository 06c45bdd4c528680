"""Per-slot controller that decides between speculative rounds and plain steps from measured throughput
(reference: inc/engine/runtime/spec_controller.h:17-93): exponential moving averages of tokens per
millisecond for both modes, periodic probing of the losing mode, back-off after poor rounds."""
from __future__ import annotations

import logging

log = logging.getLogger("volta.spec")


class SpecController:
    def __init__(self, alpha: float = 0.1, probe_every: int = 32, min_accept: float = 0.3):
        self.alpha, self.probe_every, self.min_accept = alpha, probe_every, min_accept
        self.spec_rate = None     # tokens / ms of speculative rounds
        self.plain_rate = None
        self.accept_ema = None
        self.since_probe = 0
        self.rounds = self.proposed = self.accepted = 0
        self.log_decisions = False       # launch option spec_ctrl_log: log every change of mode and every probe
        self._last = None

    def _decide(self, spec: bool, why: str) -> bool:
        if self.log_decisions and (spec != self._last or why == "probe"):
            log.info("spec controller: %s (%s; rounds %.3f tok/ms, plain %.3f tok/ms, acceptance %.2f)",
                     "speculative round" if spec else "plain step", why, self.spec_rate or 0.0, self.plain_rate or 0.0,
                     self.accept_ema or 0.0)
        self._last = spec
        return spec

    def _ema(self, old, x):
        return x if old is None else old + self.alpha * (x - old)

    def record_round(self, tokens_out: int, proposed: int, accepted: int, ms: float):
        self.rounds += 1
        self.proposed += proposed
        self.accepted += accepted
        if ms > 0:
            self.spec_rate = self._ema(self.spec_rate, tokens_out / ms)
        if proposed > 0:
            self.accept_ema = self._ema(self.accept_ema, accepted / proposed)

    def record_plain(self, ms: float):
        if ms > 0:
            self.plain_rate = self._ema(self.plain_rate, 1.0 / ms)

    def use_speculation(self) -> bool:
        self.since_probe += 1
        if self.spec_rate is None or self.plain_rate is None:
            return self._decide(self.spec_rate is None or self.since_probe % 2 == 0, "measuring")   # measure both modes first
        better_spec = self.spec_rate >= self.plain_rate
        if self.since_probe >= self.probe_every:
            self.since_probe = 0
            return self._decide(not better_spec, "probe")                # probe the losing mode once
        return self._decide(better_spec, "rate")

    def depth(self, max_depth: int) -> int:
        """Draft depth cut by the acceptance estimate (survival below min_accept is not worth a row)."""
        if self.accept_ema is None:
            return max_depth
        d, surv = 0, 1.0
        while d < max_depth and surv >= self.min_accept:
            surv *= self.accept_ema
            d += 1
        return max(1, d)

    @property
    def accept_rate(self) -> float:
        return self.accepted / self.proposed if self.proposed else 0.0
