"""Expert residency tier: hot experts in device slots, cold experts in pinned host memory read in place over PCIe.

Every expert's packed weights and scales always have a pinned host copy; ``hot_slots`` device slots hold the experts that
are routed to most. The mat-vec kernel takes a device table of per-expert base pointers, so residency changes are two
stream-ordered copies (weights into the slot, then the table entries) and CUDA graphs that captured the kernel keep
working. ``rebalance`` folds the router's histogram into a decayed heat and swaps the hottest cold experts with the
coldest hot ones when the heat ratio exceeds a margin.

Reference: inc/engine/modules/expert_tier.h:14-112 (hot slots, mapped cold experts, decayed heat, online rebalancing);
the prefill path of a tiered layer runs the same route-indexed kernel, on cold experts that ``ExpertStager`` copied into
device scratch a layer ahead (src/backend/cuda/modules/expert_tier.cu:126).
"""
from __future__ import annotations

import torch


class ExpertTier:
    NAMES = ("gu_p", "gu_s", "dn_p", "dn_s")

    def __init__(self, bank, hot_slots: int, decay: float = 0.9, margin: float = 1.25, margin_add: float = 0.0):
        E = bank.e_local
        self.bank, self.E = bank, E
        self.hot_slots = max(0, min(hot_slots, E))
        self.decay, self.margin, self.margin_add = decay, margin, margin_add      # swap when up > margin * down + margin_add
        dev = bank.gu_p.device
        self.device = dev
        pin = dev.type == "cuda"
        self.cold = {}
        for n in self.NAMES:
            t = getattr(bank, n).cpu().contiguous()
            self.cold[n] = t.pin_memory() if pin else t
        self.slots = {n: torch.empty((self.hot_slots,) + tuple(self.cold[n].shape[1:]), dtype=self.cold[n].dtype, device=dev)
                      for n in self.NAMES}
        self.slot_of = [-1] * E                    # expert -> device slot, or -1 (cold)
        self.expert_in = [-1] * self.hot_slots     # slot -> expert
        self.tab_gu = torch.zeros(2 * E, dtype=torch.int64, device=dev)
        self.tab_dn = torch.zeros(2 * E, dtype=torch.int64, device=dev)
        self.heat = torch.zeros(E, dtype=torch.float32)
        self._seen = torch.zeros(E, dtype=torch.float32)
        self.swaps = 0
        self.history_pct = 0               # largest share of a swap decision taken from the long-run counts (expert_history_pct)
        self.route_bias = None             # (device tensor [n_experts] the router adds to its selection scores, e0, value)
        for e in range(E):
            self._point_cold(e)
        for s in range(self.hot_slots):
            self._load(s, s)
        # the stacked device bank is no longer read by the mat-vec path
        for n in self.NAMES:
            setattr(bank, n, None)
        bank.gu_sf = bank.dn_sf = None

    # ---- pointer tables -----------------------------------------------------------------------------------------------
    def _set(self, e: int, gu_p: int, gu_s: int, dn_p: int, dn_s: int) -> None:
        self.tab_gu[2 * e:2 * e + 2] = torch.tensor([gu_p, gu_s], dtype=torch.int64).to(self.device, non_blocking=False)
        self.tab_dn[2 * e:2 * e + 2] = torch.tensor([dn_p, dn_s], dtype=torch.int64).to(self.device, non_blocking=False)

    def _point_cold(self, e: int) -> None:
        c = self.cold
        self._set(e, c["gu_p"][e].data_ptr(), c["gu_s"][e].data_ptr(), c["dn_p"][e].data_ptr(), c["dn_s"][e].data_ptr())

    def _load(self, e: int, slot: int) -> None:
        """Expert ``e`` becomes resident in ``slot`` (whose previous occupant turns cold first)."""
        old = self.expert_in[slot]
        if old >= 0:
            self._point_cold(old)
            self.slot_of[old] = -1
        for n in self.NAMES:
            self.slots[n][slot].copy_(self.cold[n][e], non_blocking=True)      # stream-ordered behind the readers of the slot
        s = self.slots
        self._set(e, s["gu_p"][slot].data_ptr(), s["gu_s"][slot].data_ptr(), s["dn_p"][slot].data_ptr(), s["dn_s"][slot].data_ptr())
        self.slot_of[e], self.expert_in[slot] = slot, e

    # ---- policy -------------------------------------------------------------------------------------------------------
    def rebalance(self, counts: torch.Tensor, max_swaps: int = 2) -> int:
        """``counts``: the router's cumulative histogram over this rank's experts. Returns the number of swaps made."""
        c = counts.detach().float().cpu()
        self.heat = self.heat * self.decay + (c - self._seen)
        window = float((c - self._seen).sum())
        self._seen = c.clone()
        if self.hot_slots == 0 or self.hot_slots == self.E:
            return 0
        # the score a swap is decided on: the decayed windows, blended with the long-run counts (which include what a heat
        # file of earlier runs brought in). The long-run share grows with the amount of history relative to a window and is
        # capped at history_pct, so a cold start follows its first windows.
        score = self.heat
        total = float(c.sum())
        if self.history_pct > 0 and total > 0 and float(self.heat.sum()) > 0:
            a = (self.history_pct / 100.0) * total / (total + 16.0 * max(window, 1.0))
            score = (1 - a) * self.heat / float(self.heat.sum()) + a * c / total
            score = score * float(self.heat.sum())              # back in route units: margin_add keeps its meaning
        n = 0
        for _ in range(max_swaps):
            cold = [e for e in range(self.E) if self.slot_of[e] < 0]
            hot = [e for e in range(self.E) if self.slot_of[e] >= 0]
            up = max(cold, key=lambda e: (float(score[e]), -e))
            down = min(hot, key=lambda e: (float(score[e]), e))
            if float(score[up]) <= float(score[down]) * self.margin + self.margin_add or float(score[up]) <= 0:
                break
            self._load(up, self.slot_of[down])
            n += 1
        self.swaps += n
        if n:
            self.sync_route_bias()
        return n

    def set_route_bias(self, bias: torch.Tensor, e0: int, value: float) -> None:
        """``bias`` [n_experts] fp32 on the device is what the router adds to its selection scores (the weights stay the
        raw scores): resident experts of this rank's slice [e0, e0 + E) get ``value`` on top of ``base``, so near ties go
        to experts that are in device memory. Follows the residency after every rebalance."""
        self.route_bias = (bias, e0, float(value), bias[e0:e0 + self.E].clone())
        self.sync_route_bias()

    def sync_route_bias(self) -> None:
        if self.route_bias is None:
            return
        bias, e0, value, base = self.route_bias
        mask = torch.tensor([1.0 if s >= 0 else 0.0 for s in self.slot_of], dtype=torch.float32)
        bias[e0:e0 + self.E].copy_(base + value * mask.to(bias.device))

    def resident(self) -> list[int]:
        return sorted(e for e in range(self.E) if self.slot_of[e] >= 0)

    def device_bytes(self) -> int:
        return sum(t.numel() * t.element_size() for t in self.slots.values())

    def host_bytes(self) -> int:
        return sum(t.numel() * t.element_size() for t in self.cold.values())


class ExpertStager:
    """Prefill staging of cold experts: a chunk of many rows would read a cold expert over PCIe once per route, so the
    cold experts of a layer are copied once into device scratch instead, a layer ahead of the compute, and the route
    kernel reads that copy through a second pointer table.

    Two scratch buffers alternate between consecutive tiered layers. ``acquire(tier)`` makes the launching stream wait
    for the layer's copy (starting it first when nothing staged it), starts the next layer's copy into the other buffer on
    the copy stream, and returns the (gate|up, down) pointer tables to launch with; ``release(tier)`` marks the buffer
    free for the copy two layers on. The tables of a (tier, buffer) pair depend only on the residency, so they are built
    once per residency version and no host memory is rewritten while a copy reads it.
    Reference: src/backend/cuda/modules/expert_tier.cu:126 (stage ahead, two buffers, auto off for trellis experts),
    docs/CONFIG.md:91 (expert_stage).
    """

    def __init__(self, tiers: list, min_rows: int = 17):
        self.tiers = [t for _, t in tiers] if tiers and isinstance(tiers[0], tuple) else list(tiers)
        assert self.tiers, "no tiered layers to stage"
        t0 = self.tiers[0]
        self.device = t0.device
        self.min_rows = min_rows
        self.n_cold = max(t.E - t.hot_slots for t in self.tiers)
        self.order = {id(t): i for i, t in enumerate(self.tiers)}
        self.buf = [{n: torch.empty((self.n_cold,) + tuple(t0.cold[n].shape[1:]), dtype=t0.cold[n].dtype, device=self.device)
                     for n in ExpertTier.NAMES} for _ in range(2)]
        cuda = self.device.type == "cuda"
        self.copy_stream = torch.cuda.Stream(self.device) if cuda else None
        self.ready = [torch.cuda.Event() for _ in range(2)] if cuda else None
        self.free = [torch.cuda.Event() for _ in range(2)] if cuda else None
        self.staged = [None, None]                     # per buffer: (tier index, residency version) of its content
        self.used = [False, False]                     # a release was recorded on the buffer's free event
        self._tabs = {}                                # (tier index, buffer) -> (version, tab_gu, tab_dn)
        self.copies = 0                                # cold-expert copies started (bytes: see ``bytes_staged``)
        self.bytes_staged = 0

    @classmethod
    def scratch_bytes(cls, tiers: list) -> int:
        ts = [t for _, t in tiers] if tiers and isinstance(tiers[0], tuple) else list(tiers)
        per = sum(t.cold[n][0].numel() * t.cold[n].element_size() for t in ts[:1] for n in ExpertTier.NAMES)
        return 2 * per * max((t.E - t.hot_slots for t in ts), default=0)

    def wants(self, tier, rows: int) -> bool:
        return rows >= self.min_rows and id(tier) in self.order and tier.hot_slots < tier.E

    def _tables(self, i: int, b: int):
        """Pointer tables of tier ``i`` whose cold entries point into buffer ``b`` (cold experts in ascending order)."""
        t = self.tiers[i]
        hit = self._tabs.get((i, b))
        if hit is not None and hit[0] == t.swaps:
            return hit[1], hit[2]
        gu, dn = t.tab_gu.clone(), t.tab_dn.clone()
        cold = [e for e in range(t.E) if t.slot_of[e] < 0]
        s = self.buf[b]
        idx = torch.tensor([2 * e + j for e in cold for j in (0, 1)], dtype=torch.int64)
        pg = torch.tensor([p for j in range(len(cold)) for p in (s["gu_p"][j].data_ptr(), s["gu_s"][j].data_ptr())], dtype=torch.int64)
        pd = torch.tensor([p for j in range(len(cold)) for p in (s["dn_p"][j].data_ptr(), s["dn_s"][j].data_ptr())], dtype=torch.int64)
        gu[idx.to(self.device)] = pg.to(self.device)
        dn[idx.to(self.device)] = pd.to(self.device)
        self._tabs[(i, b)] = (t.swaps, gu, dn)
        return gu, dn

    def _stage(self, i: int, b: int) -> None:
        """Start the copy of tier ``i``'s cold experts into buffer ``b`` (runs of consecutive experts as one copy each)."""
        t = self.tiers[i]
        cold = [e for e in range(t.E) if t.slot_of[e] < 0]
        runs, j = [], 0
        while j < len(cold):
            k = j
            while k + 1 < len(cold) and cold[k + 1] == cold[k] + 1:
                k += 1
            runs.append((j, cold[j], k - j + 1))
            j = k + 1

        def copy():
            for pos, e, n in runs:
                for name in ExpertTier.NAMES:
                    src = t.cold[name][e:e + n]
                    self.buf[b][name][pos:pos + n].copy_(src, non_blocking=True)
                    self.bytes_staged += src.numel() * src.element_size()
        if self.copy_stream is None:
            copy()
        else:
            with torch.cuda.stream(self.copy_stream):
                if self.used[b]:
                    self.copy_stream.wait_event(self.free[b])       # the layer that last read this buffer has finished
                copy()
                self.ready[b].record(self.copy_stream)
        self.staged[b] = (i, t.swaps)
        self.copies += 1

    def acquire(self, tier):
        i = self.order[id(tier)]
        b = i & 1
        self._tables(i, b)                                  # built on the launching stream before any copy is queued
        if self.staged[b] != (i, tier.swaps):
            self._stage(i, b)
        if self.copy_stream is not None:
            torch.cuda.current_stream(self.device).wait_event(self.ready[b])
        if i + 1 < len(self.tiers):
            nxt = self.tiers[i + 1]
            if nxt.hot_slots < nxt.E and self.staged[b ^ 1] != (i + 1, nxt.swaps):
                self._tables(i + 1, b ^ 1)
                self._stage(i + 1, b ^ 1)
        return self._tables(i, b)

    def release(self, tier) -> None:
        b = self.order[id(tier)] & 1
        if self.free is not None:
            self.free[b].record(torch.cuda.current_stream(self.device))
        self.used[b] = True
