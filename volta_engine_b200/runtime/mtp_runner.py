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

    # ---- one speculative round; returns the newly produced tokens (accepted drafts + the target's own token)
    def _static(self):
        """Device-resident state of a round: the chain, the verify step and the acceptance count read and write these
        tensors only, so a round is a fixed sequence of launches (captured once into a CUDA graph) and the host reads
        one small result at its end."""
        st = getattr(self, "_st", None)
        if st is None:
            e, d = self.e, self.depth
            dev = e.device
            H = self.model.cfg.hidden
            z = lambda n, dt=torch.int32: torch.zeros(n, dtype=dt, device=dev)
            st = self._st = {
                "anchor": z(1), "pos": z(1), "slot": z(1), "hid": torch.zeros(1, H, dtype=torch.bfloat16, device=dev),
                "rows": z(d + 1),            # [anchor, draft_1 .. draft_d]: the verify step's input rows
                "rows_pos": z(d + 1), "head_pos": z(d), "slots": z(d + 1), "val": z(d + 1, torch.float32),
                "target": z(d + 1),          # the target model's greedy token after each row
                "result": z(2 * d + 2),      # [accepted count, target tokens (d + 1), drafts (d)] read by the host
                "ar": torch.arange(d + 1, dtype=torch.int32, device=dev), "graph": None, "calls": 0,
                "h_in": torch.zeros(3, dtype=torch.int32, pin_memory=e.cuda),
                "h_out": torch.zeros(2 * d + 2, dtype=torch.int32, pin_memory=e.cuda),
            }
        return st

    def _round_body(self):
        e, m, st, d = self.e, self.model, self._st, self.depth
        st["rows_pos"].copy_(st["pos"] + st["ar"])
        st["head_pos"].copy_(st["pos"] - 1 + st["ar"][:d])
        st["slots"].copy_(st["slot"].expand(d + 1))
        st["rows"][:1].copy_(st["anchor"])
        hid, nxt = st["hid"], st["anchor"]
        ns1 = e._nsplit(1)
        for i in range(d):                                # head position pos-1+i consumes (hidden, next token)
            b = BatchRows(st["rows"][:1], st["head_pos"][i:i + 1], st["slot"], 1, LOGITS_ALL, None, ns1)
            logits, hid = m.mtp_forward(nxt, hid, b, e.kv)
            nxt = st["rows"][i + 1:i + 2]                 # the head's argmax lands in the row the next step reads
            e._sample_greedy(logits, nxt, st["val"][i + 1:i + 2], 1)
        b = BatchRows(st["rows"], st["rows_pos"], st["slots"], d + 1, LOGITS_ALL, None, e._nsplit(d + 1))
        logits = m.forward(b, e.kv)
        e._sample_greedy(logits, st["target"], st["val"], d + 1)
        ok = (st["target"][:d] == st["rows"][1:]).to(torch.int32)
        st["result"][:1].copy_(torch.cumprod(ok, 0).sum(0, keepdim=True))
        st["result"][1:d + 2].copy_(st["target"])
        st["result"][d + 2:].copy_(st["rows"][1:])

    def _device_round_ok(self) -> bool:
        e = self.e
        return e.cuda and hasattr(e, "_nsplit") and not getattr(e, "mrope", False) and self.depth + 1 <= MAX_GRAPH_ROWS

    def round(self, slot: int, anchor: int, pos: int) -> list[int]:
        e, m = self.e, self.model
        e.kv.reserve(slot, pos + self.depth + 3)
        if not self._device_round_ok():
            return self._round_host(slot, anchor, pos)
        st, d = self._static(), self.depth
        st["h_in"][0], st["h_in"][1], st["h_in"][2] = anchor, pos, slot
        st["anchor"].copy_(st["h_in"][0:1], non_blocking=True)
        st["pos"].copy_(st["h_in"][1:2], non_blocking=True)
        st["slot"].copy_(st["h_in"][2:3], non_blocking=True)
        st["hid"].copy_(self.hidden[slot])
        st["calls"] += 1
        if st["graph"] is not None:
            st["graph"].replay()
        elif st["calls"] < 2 or not e.use_graphs:
            self._round_body()
        else:
            torch.cuda.synchronize()
            g = torch.cuda.CUDAGraph()
            with torch.cuda.graph(g):
                self._round_body()
            st["graph"] = g
            g.replay()
        st["h_out"].copy_(st["result"], non_blocking=True)          # the round's only read by the host
        torch.cuda.current_stream().synchronize()
        res = st["h_out"].tolist()
        acc, toks, drafts = res[0], res[1:d + 2], res[d + 2:]
        rows = [anchor] + drafts
        new = drafts[:acc] + [toks[acc]]
        h = m.last_residual
        if acc > 0:                                        # catch-up with the true hidden states of accepted rows
            b = self._rows(rows[:acc], [pos + i for i in range(acc)], slot, False)
            nx = torch.tensor(new[:acc], dtype=torch.int32).to(e.device)
            m.mtp_forward(nx, h[:acc].clone(), b, e.kv)
        self.hidden[slot] = h[acc:acc + 1].clone()
        self.stats["rounds"] += 1
        self.stats["proposed"] += d
        self.stats["accepted"] += acc
        return new

    def _round_host(self, slot: int, anchor: int, pos: int) -> list[int]:
        """The same round driven from the host (CPU model, engines that relay steps to other ranks): the chain feeds
        device tensors from step to step, and the host reads drafts and target tokens once, after the verify step."""
        e, m = self.e, self.model
        hid = self.hidden[slot]
        nxt = torch.tensor([anchor], dtype=torch.int32).to(e.device)
        dev_drafts = torch.zeros(self.depth, dtype=torch.int32, device=e.device)
        val_buf = torch.zeros(1, dtype=torch.float32, device=e.device)
        for i in range(self.depth):                       # head position pos-1+i consumes (hidden, next token)
            b = self._rows([0], [pos - 1 + i], slot, False)
            logits, hid = m.mtp_forward(nxt, hid, b, e.kv)
            nxt = dev_drafts[i:i + 1]
            e._sample_greedy(logits, nxt, val_buf, 1)
        drafts = dev_drafts.tolist()
        rows = [anchor] + drafts
        toks = e.step(rows, [pos + i for i in range(len(rows))], [slot] * len(rows))
        acc = 0
        while acc < len(drafts) and toks[acc] == drafts[acc]:
            acc += 1
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
