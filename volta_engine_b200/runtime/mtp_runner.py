"""Speculative decoding with the checkpoint's own MTP head.

Round structure of the reference MtpRunner (src/runtime/mtp_runner.cpp:147-276): (1) catch-up of the head over
rows whose true hidden state is known, (2) a device-side draft chain of the head fed with its own previous
argmax, (3) ONE batched verify forward of ``[anchor, drafts...]`` through the target model, (4) longest-prefix
acceptance (greedy equality), (5) the cache needs no repair: rejected positions are overwritten later.
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
    def round(self, slot: int, anchor: int, pos: int) -> list[int]:
        e, m = self.e, self.model
        e.kv.reserve(slot, pos + self.depth + 3)
        hid = self.hidden[slot]
        nxt = torch.tensor([anchor], dtype=torch.int32).to(e.device)
        drafts = []
        tok_buf = torch.zeros(1, dtype=torch.int32, device=e.device)
        val_buf = torch.zeros(1, dtype=torch.float32, device=e.device)
        for i in range(self.depth):                       # head position pos-1+i consumes (hidden, next token)
            b = self._rows([0], [pos - 1 + i], slot, False)
            logits, hid = m.mtp_forward(nxt, hid, b, e.kv)
            e._sample_greedy(logits, tok_buf, val_buf, 1)
            nxt = tok_buf.clone()
            drafts.append(int(tok_buf[0].item()))
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
