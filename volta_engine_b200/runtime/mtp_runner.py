"""Speculative decoding with the checkpoint's own MTP head.

Round structure of the reference MtpRunner (src/runtime/mtp_runner.cpp:147-276): (1) catch-up of the head over
rows whose true hidden state is known, (2) a device-side draft chain of the head: its argmax is written into the row
descriptor that the next head step and the verify step read, with no read by the host in between, (3) ONE batched
verify forward of ``[anchor, drafts...]`` through the target model, (4) longest-prefix acceptance (greedy equality)
counted on the device; chain, verify step and count replay as one CUDA graph and the host reads one result vector, (5) the cache needs no repair: rejected positions are overwritten later.
The head keeps its own cache layer; position p of that layer holds the head's state for (hidden_p, token_{p+1}).
"""
from __future__ import annotations

import torch

from ..ops import kernels as K
from .batch import BatchRows, LOGITS_ALL, MAX_GRAPH_ROWS


class MtpRunner:
    def __init__(self, engine, depth: int = 3):
        self.e, self.depth = engine, depth
        self.model = engine.model
        assert getattr(self.model, "mtp", None) is not None, "model has no MTP head"
        self.hidden: dict[int, torch.Tensor] = {}      # slot -> residual-stream state of the last verified row
        self.stats = {"rounds": 0, "proposed": 0, "accepted": 0}
        self.cond = [1.0] * max(1, depth)              # survival averages, see round_depth
        self.adaptive = False                          # True: the depth of a round follows the survival estimate
        self.last_depth = depth
        self._sts: dict = {}

    def _rows(self, ids, pos, slot, prefill: bool) -> BatchRows:
        G = 1
        n = len(ids)
        return BatchRows.make(ids, pos, [slot] * n, self.e.device, LOGITS_ALL, G, prefill=prefill and n > MAX_GRAPH_ROWS,
                              nsplit=self.e._nsplit(n))

    def _full_rows(self, h: torch.Tensor, n: int) -> torch.Tensor:
        """Residual rows of the last forward, gathered when the chunk ran sequence-parallel."""
        comm = self.e.comm
        if h.shape[0] == n:
            return h
        return comm.all_gather_rows(h)[:n]

    # ---- prefill: run the target chunk, then the head over every row whose next token is known
    def prefill_rows(self, slot: int, prompt: list[int], start: int, end: int, want_token: bool) -> int:
        e = self.e
        tok = e.prefill_rows(slot, prompt[start:end], start, want_token)
        h = self._full_rows(self.model.last_residual, end - start)
        n_known = end - start if end < len(prompt) else end - start - 1
        if n_known > 0:
            nxt = torch.tensor(prompt[start + 1:start + 1 + n_known], dtype=torch.int32).to(e.device)
            b = self._rows(prompt[start:start + n_known], list(range(start, start + n_known)), slot, True)
            self.model.mtp_forward(nxt, h[:n_known].contiguous(), b, e.kv)
        if end == len(prompt):
            self.hidden[slot] = h[end - start - 1:end - start].clone()
        return tok

    # ---- speculative rounds on the device
    MIN_SURVIVAL = 0.3            # stop chaining once the chance that the block is still alive drops below this
    EMA = 0.1

    def round_depth(self) -> int:
        """Drafts of the next round: the head chains on its own output while the estimated chance that every earlier
        draft was accepted stays above ``MIN_SURVIVAL``. The estimate is an average over past rounds (``cond[k]``: how
        often draft k was accepted when drafts < k were), not a function of the drafted tokens, so the length of a round
        is known before its first step and the whole round can run on the device.
        Reference: src/runtime/mtp_runner.cpp:158-168."""
        if not self.adaptive:
            return self.depth
        alive, d = 1.0, 1
        for k in range(1, self.depth):
            alive *= self.cond[k - 1]
            if alive < self.MIN_SURVIVAL:
                break
            d += 1
        return d

    def _observe(self, drafted: int, acc: int) -> None:
        for k in range(min(drafted, acc + 1)):                  # draft k was judged only if every earlier one was accepted
            hit = 1.0 if k < acc else 0.0
            self.cond[k] += self.EMA * (hit - self.cond[k])

    def _static(self, k: int, d: int):
        """Device-resident state of a round over ``k`` slots with ``d`` drafts each: the chain, the verify step and the
        acceptance counts read and write these tensors only, so a round is a fixed sequence of launches (captured once
        per (k, d) into a CUDA graph) and the host reads one small result at its end."""
        st = self._sts.get((k, d))
        if st is None:
            e = self.e
            dev = e.device
            H = self.model.cfg.hidden
            z = lambda *n, dt=torch.int32: torch.zeros(*n, dtype=dt, device=dev)
            st = self._sts[(k, d)] = {
                "anchor": z(k), "pos": z(k), "slot": z(k), "hid": torch.zeros(k, H, dtype=torch.bfloat16, device=dev),
                "rows": z(k, d + 1),         # per slot [anchor, draft_1 .. draft_d]: the verify step's input rows
                "rows_pos": z(k, d + 1), "head_pos": z(d, k), "slots": z(k, d + 1), "val": z(k * (d + 1), dt=torch.float32),
                "draft": z(d, k), "target": z(k * (d + 1)),
                "result": z(k, 2 * d + 2),   # per slot [accepted count, target tokens (d + 1), drafts (d)]
                "ar": torch.arange(d + 1, dtype=torch.int32, device=dev), "graph": None, "calls": 0,
                "h_in": torch.zeros(3, k, dtype=torch.int32, pin_memory=e.cuda),
                "h_out": torch.zeros(k, 2 * d + 2, dtype=torch.int32, pin_memory=e.cuda),
            }
        return st

    def _round_body(self, st, k: int, d: int):
        e, m = self.e, self.model
        st["rows_pos"].copy_(st["pos"][:, None] + st["ar"][None, :])
        st["head_pos"].copy_(st["pos"][None, :] - 1 + st["ar"][:d, None])
        st["slots"].copy_(st["slot"][:, None].expand(k, d + 1))
        st["rows"][:, 0].copy_(st["anchor"])
        hid, nxt = st["hid"], st["anchor"]
        nsk = e._nsplit(k)
        journal = hasattr(m, "rollback_state")             # recurrent state: the verify block runs journalled
        if journal:
            m.begin_journal(False)
        for i in range(d):                                # head position pos-1+i consumes (hidden, next token)
            b = BatchRows(st["anchor"], st["head_pos"][i], st["slot"], k, LOGITS_ALL, None, nsk)
            logits, hid = m.mtp_forward(nxt, hid, b, e.kv)
            nxt = st["draft"][i]                          # the head's argmax lands in the buffer the next step reads
            e._sample_greedy(logits, nxt, st["val"][:k], k)
            st["rows"][:, i + 1].copy_(nxt)
        n = k * (d + 1)
        b = BatchRows(st["rows"].view(n), st["rows_pos"].view(n), st["slots"].view(n), n, LOGITS_ALL, None, e._nsplit(n))
        if journal:
            m.begin_journal(True, ("mtp", k, d))
        logits = m.forward(b, e.kv)
        if journal:
            m.journal_on = False
        e._sample_greedy(logits, st["target"], st["val"], n)
        tgt = st["target"].view(k, d + 1)
        ok = (tgt[:, :d] == st["rows"][:, 1:]).to(torch.int32)
        st["result"][:, 0].copy_(torch.cumprod(ok, 1).sum(1))
        st["result"][:, 1:d + 2].copy_(tgt)
        st["result"][:, d + 2:].copy_(st["rows"][:, 1:])

    def _device_round_ok(self, k: int = 1) -> bool:
        e = self.e
        if k > 1 and hasattr(self.model, "rollback_state"):
            return False                                   # a journalled verify block holds the rows of one slot
        return (e.cuda and hasattr(e, "_nsplit") and not getattr(e, "mrope", False)
                and k * (self.depth + 1) <= MAX_GRAPH_ROWS)

    def round(self, slot: int, anchor: int, pos: int) -> list[int]:
        if not self._device_round_ok():
            self.e.kv.reserve(slot, pos + self.depth + 3)
            return self._round_host(slot, anchor, pos)
        return self.round_joint([slot], [anchor], [pos])[0]

    def round_joint(self, slots: list[int], anchors: list[int], poss: list[int]) -> list[list[int]]:
        """One round for several slots at once: their head steps run as one batch and their verify rows as one block
        (``len(slots) * (depth + 1)`` rows; the depth is shared: the survival estimate does not depend on the slot).
        Returns the new tokens of every slot. Reference: src/runtime/mtp_runner.cpp:256-409 (``speculate_joint``)."""
        e, m = self.e, self.model
        k, d = len(slots), self.round_depth()
        assert self._device_round_ok(k), "joint round does not fit the decode graphs"
        for s, p in zip(slots, poss):
            e.kv.reserve(s, p + d + 3)
        st = self._static(k, d)
        for j in range(k):
            st["h_in"][0, j], st["h_in"][1, j], st["h_in"][2, j] = anchors[j], poss[j], slots[j]
        st["anchor"].copy_(st["h_in"][0], non_blocking=True)
        st["pos"].copy_(st["h_in"][1], non_blocking=True)
        st["slot"].copy_(st["h_in"][2], non_blocking=True)
        for j, s in enumerate(slots):
            st["hid"][j:j + 1].copy_(self.hidden[s])
        st["calls"] += 1
        if st["graph"] is not None:
            st["graph"].replay()
        elif st["calls"] < 2 or not e.use_graphs:
            self._round_body(st, k, d)
        else:
            torch.cuda.synchronize()
            g = torch.cuda.CUDAGraph()
            with torch.cuda.graph(g):
                self._round_body(st, k, d)
            st["graph"] = g
            g.replay()
        st["h_out"].copy_(st["result"], non_blocking=True)          # the round's only read by the host
        torch.cuda.current_stream().synchronize()
        res = st["h_out"].tolist()
        h = m.last_residual
        out = []
        for j, (slot, anchor, pos) in enumerate(zip(slots, anchors, poss)):
            acc, toks, drafts = res[j][0], res[j][1:d + 2], res[j][d + 2:]
            rows = [anchor] + drafts
            new = drafts[:acc] + [toks[acc]]
            base = j * (d + 1)
            if acc < d and hasattr(m, "rollback_state"):
                m._jlast = ("mtp", k, d)
                m.rollback_state(slot, acc + 1)           # as if only the accepted rows had run
            if acc > 0:                                    # catch-up with the true hidden states of accepted rows
                b = self._rows(rows[:acc], [pos + i for i in range(acc)], slot, False)
                nx = torch.tensor(new[:acc], dtype=torch.int32).to(e.device)
                m.mtp_forward(nx, h[base:base + acc].clone(), b, e.kv)
            self.hidden[slot] = h[base + acc:base + acc + 1].clone()
            self.stats["rounds"] += 1
            self.stats["proposed"] += d
            self.stats["accepted"] += acc
            self._observe(d, acc)
            out.append(new)
        self.last_depth = d
        return out

    def _round_host(self, slot: int, anchor: int, pos: int) -> list[int]:
        """The same round driven from the host (CPU model, engines that relay steps to other ranks): the chain feeds
        device tensors from step to step, and the host reads drafts and target tokens once, after the verify step."""
        e, m = self.e, self.model
        hid = self.hidden[slot]
        nxt = torch.tensor([anchor], dtype=torch.int32).to(e.device)
        depth = self.round_depth()
        dev_drafts = torch.zeros(depth, dtype=torch.int32, device=e.device)
        val_buf = torch.zeros(1, dtype=torch.float32, device=e.device)
        for i in range(depth):                            # head position pos-1+i consumes (hidden, next token)
            b = self._rows([0], [pos - 1 + i], slot, False)
            logits, hid = m.mtp_forward(nxt, hid, b, e.kv)
            nxt = dev_drafts[i:i + 1]
            e._sample_greedy(logits, nxt, val_buf, 1)
        drafts = dev_drafts.tolist()
        rows = [anchor] + drafts
        jn = {"journal": True} if getattr(e, "supports_journal", False) else {}
        toks = e.step(rows, [pos + i for i in range(len(rows))], [slot] * len(rows), **jn)
        acc = 0
        while acc < len(drafts) and toks[acc] == drafts[acc]:
            acc += 1
        if jn and acc < len(drafts):
            e.rollback(slot, acc + 1)
        new = drafts[:acc] + [toks[acc]]
        h = m.last_residual
        if acc > 0:                                        # catch-up with the true hidden states of accepted rows
            b = self._rows(rows[:acc], [pos + i for i in range(acc)], slot, False)
            nx = torch.tensor(new[:acc], dtype=torch.int32).to(e.device)
            m.mtp_forward(nx, h[:acc].clone(), b, e.kv)
        self.hidden[slot] = h[acc:acc + 1].clone()
        self.stats["rounds"] += 1
        self.stats["proposed"] += len(drafts)
        self.stats["accepted"] += acc
        self._observe(len(drafts), acc)
        self.last_depth = len(drafts)
        return new

    def after_plain_step(self, slot: int, fed_tok: int, pos: int, new_tok: int):
        """Keep the head's cache and hidden state current when a plain (non-speculative) step was taken."""
        e, m = self.e, self.model
        prev = self.hidden.get(slot)
        if prev is not None:
            b = self._rows([0], [pos - 1], slot, False)
            m.mtp_forward(torch.tensor([fed_tok], dtype=torch.int32).to(e.device), prev, b, e.kv)
        self.hidden[slot] = m.last_residual[:1].clone()

    def release(self, slot: int):
        self.hidden.pop(slot, None)
