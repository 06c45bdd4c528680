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


class DepthByRate:
    """Draft depth chosen for the most expected tokens per millisecond (launch option spec_depth_rate). The drafter's
    recent per-position accuracy (p[k]: how often draft k was accepted when every earlier one was) gives the expected
    tokens of a depth, E(d) = 1 + sum_{k <= d} prod_{j <= k} p[j]; the measured round times, fitted as a fixed and a
    per-row cost, give its time. Until both have data the configured depth is used.
    Reference: docs/CONFIG.md:136 (spec_depth_rate)."""

    def __init__(self, max_depth: int, alpha: float = 0.1):
        self.max_depth, self.alpha = max_depth, alpha
        self.p = [0.5] * max_depth
        self.seen = [0] * max_depth
        self.n = self.sx = self.sy = self.sxx = self.sxy = 0.0

    def record(self, drafted: int, accepted: int, ms: float) -> None:
        for k in range(min(drafted, accepted + 1, self.max_depth)):
            hit = 1.0 if k < accepted else 0.0
            self.p[k] += self.alpha * (hit - self.p[k])
            self.seen[k] += 1
        x = drafted + 1.0                                  # verify rows of the round
        self.n, self.sx, self.sy, self.sxx, self.sxy = self.n + 1, self.sx + x, self.sy + ms, self.sxx + x * x, self.sxy + x * ms

    def time_model(self):
        """(fixed ms, ms per row) by least squares; None until rounds of two different sizes were seen."""
        den = self.n * self.sxx - self.sx * self.sx
        if self.n < 4 or den <= 1e-9:
            return None
        b = (self.n * self.sxy - self.sx * self.sy) / den
        a = (self.sy - b * self.sx) / self.n
        return max(a, 0.0), max(b, 0.0)

    def choose(self, default: int) -> int:
        tm = self.time_model()
        if tm is None or self.seen[0] < 4:
            # no fit yet: alternate depths so that the fit gets two sizes
            return default if int(self.n) % 2 == 0 else max(1, default - 1)
        a, b = tm
        best, best_rate, exp, alive = 1, -1.0, 1.0, 1.0
        for d in range(1, self.max_depth + 1):
            alive *= self.p[d - 1]
            exp += alive
            rate = exp / max(1e-6, a + b * (d + 1))
            if rate > best_rate:
                best, best_rate = d, rate
        return best
