"""Single-rank execution engine: chunked prefill, CUDA-graph decode, greedy sampling on the device.

Plays the role of the reference's ``ModelCluster::forward / prefill / sample`` for one rank
(src/runtime/cluster.cpp:328-337,498-556,610-646) with its ``GraphCache`` policy
(inc/engine/core/graph_cache.h:21-89): the first call of a row count runs eagerly, the second is
captured, later calls replay. Row ids / positions / slots live in static device buffers, so a replay
never depends on host arguments; attention grids are position independent.
"""
from __future__ import annotations

import os

import time
from dataclasses import dataclass

import torch

from ..ops import kernels as K
from .batch import BatchRows, LOGITS_ALL, LOGITS_LAST, LOGITS_NONE, MAX_GRAPH_ROWS
from .kv_cache import PagedKVCache


@dataclass
class GenStats:
    prompt_tokens: int = 0
    new_tokens: int = 0
    prefill_ms: float = 0.0
    decode_ms: float = 0.0

    @property
    def prefill_tok_s(self):
        return self.prompt_tokens / (self.prefill_ms / 1e3) if self.prefill_ms > 0 else 0.0

    @property
    def decode_tok_s(self):
        return self.new_tokens / (self.decode_ms / 1e3) if self.decode_ms > 0 else 0.0


class _Graph:
    __slots__ = ("graph", "calls", "tokens", "logits")

    def __init__(self):
        self.graph = None
        self.calls = 0
        self.tokens = None
        self.logits = None


class Engine:
    def __init__(self, model, kv: PagedKVCache, *, use_graphs: bool = True, prefill_chunk: int = 2048,
                 feedback: bool = True):
        self.model, self.kv = model, kv
        self.device = model.device
        self.cuda = self.device.type == "cuda"
        self.use_graphs = use_graphs and self.cuda
        self.prefill_chunk = prefill_chunk
        cap = getattr(getattr(model, "comm", None), "chunk_rows", None)
        if cap:                                    # the communicator's reduce-scatter buffers hold one chunk
            self.prefill_chunk = min(self.prefill_chunk, int(cap))
        self.feedback = feedback
        self.comm = model.comm
        if self.cuda and hasattr(model, "link_prefetch"):
            model.link_prefetch()
        dev = self.device
        R = MAX_GRAPH_ROWS
        # static step descriptor (device) + pinned host staging
        self.s_ids = torch.zeros(R, dtype=torch.int32, device=dev)
        self.s_pos = torch.zeros(R, dtype=torch.int32, device=dev)
        self.s_slot = torch.full((R,), -1, dtype=torch.int32, device=dev)
        self.s_tok = torch.zeros(R, dtype=torch.int32, device=dev)
        self.s_val = torch.zeros(R, dtype=torch.float32, device=dev)
        pin = self.cuda
        self.h_in = torch.zeros(3, R, dtype=torch.int32, pin_memory=pin)
        self.h_tok = torch.zeros(R, dtype=torch.int32, pin_memory=pin)
        from .sampling import NUM_CANDIDATES
        self.s_cand_ids = torch.zeros(R, NUM_CANDIDATES, dtype=torch.int32, device=dev)
        self.s_cand_vals = torch.zeros(R, NUM_CANDIDATES, dtype=torch.float32, device=dev)
        self.s_cand_lse = torch.zeros(R, dtype=torch.float32, device=dev)
        # multimodal rotary positions: per-slot offset of the rotary position against the sequence index
        self.mrope = bool(getattr(getattr(model, "cfg", None), "mrope_sections", ()))
        self.h_delta = [0] * kv.max_slots
        self.s_delta = torch.zeros(kv.max_slots, dtype=torch.int32, device=dev)
        self.s_pos3 = torch.zeros(3 * R, dtype=torch.int32, device=dev)
        self.graphs: dict[tuple, _Graph] = {}
        self.nsplit_cap = int(os.environ.get("VOLTA_NSPLIT_CAP", "32"))   # most key splits of a decode row
        if self.cuda:
            model.ensure_workspace(R, self.nsplit_cap)

    # ------------------------------------------------------------------------------------------ helpers
    def _nsplit(self, rows: int) -> int:
        if not self.cuda:
            return 1
        per = 148 * 3 // max(1, rows * self.model.nkv)
        return max(1, min(self.nsplit_cap, per))

    def _sample_greedy(self, logits: torch.Tensor, out_tok: torch.Tensor, out_val: torch.Tensor, rows: int):
        off = self.comm.rank * self.model.vocab_local
        K.argmax(logits, off, out_tok[:rows], out_val[:rows])
        if self.comm.size > 1:
            merged = self.comm.merge_argmax(out_tok[:rows], out_val[:rows])
            out_tok[:rows].copy_(merged)

    # ------------------------------------------------------------------------------------------ prefill
    def prefill(self, slot: int, tokens: list[int], start_pos: int = 0, mm=None) -> int:
        """Run the prompt rows [start_pos, start_pos + len(tokens)) of ``slot`` through the model in chunks
        and return the greedy next token (host int)."""
        n = len(tokens)
        self.kv.reserve(slot, start_pos + n + 1)
        G = self.model.nq // self.model.nkv
        done = 0
        tok = -1
        if hasattr(self.model, "set_prefill_end"):          # models that run only the tail of a prompt through their late layers
            self.model.set_prefill_end(start_pos + n)
        while done < n:
            c = min(self.prefill_chunk, n - done)
            last = done + c == n
            ids = tokens[done:done + c]
            pos = list(range(start_pos + done, start_pos + done + c))
            if c <= MAX_GRAPH_ROWS:
                b = BatchRows.make(ids, pos, [slot] * c, self.device, LOGITS_ALL if last else LOGITS_NONE, G,
                                   prefill=False, nsplit=self._nsplit(c))
            else:
                b = BatchRows.make(ids, pos, [slot] * c, self.device, LOGITS_LAST if last else LOGITS_NONE, G,
                                   prefill=True)
            self._mm_rows(b, slot, start_pos + done, c, mm)
            logits = self.model.forward(b, self.kv)
            if last:
                rows = logits.shape[0]
                self._sample_greedy(logits, self.s_tok, self.s_val, rows)
                tok = int(self.s_tok[rows - 1].item())
            done += c
        if hasattr(self.model, "set_prefill_end"):
            self.model.set_prefill_end(-1)
        return tok

    # ------------------------------------------------------------------------------------------ decode
    def _forward_static(self, rows: int, nsplit: int, topk: bool = False) -> torch.Tensor:
        b = BatchRows(self.s_ids[:rows], self.s_pos[:rows], self.s_slot[:rows], rows, LOGITS_ALL, None, nsplit)
        if self.mrope:
            # rotary position = sequence index + the slot's offset left by its multimodal prompt (all three axes alike)
            d = self.s_delta[self.s_slot[:rows].clamp(min=0).long()]
            b.pos3 = self.s_pos3[:3 * rows].view(3, rows)
            b.pos3.copy_((self.s_pos[:rows] + d).unsqueeze(0).expand(3, rows))
        logits = self.model.forward(b, self.kv)
        self._sample_greedy(logits, self.s_tok, self.s_val, rows)
        if topk:
            from .sampling import NUM_CANDIDATES
            off = self.comm.rank * self.model.vocab_local
            ids, vals, lse = K.topk(logits, NUM_CANDIDATES, off)
            self.s_cand_ids[:rows].copy_(ids)
            self.s_cand_vals[:rows].copy_(vals)
            self.s_cand_lse[:rows].copy_(lse)
        if self.feedback and not topk:
            # feed the sampled token back and advance positions on the device: replays chain with no host work
            self.s_ids[:rows].copy_(self.s_tok[:rows])
            self.s_pos[:rows].add_(1)
        return logits

    def _run_rows(self, rows: int, topk: bool = False, journal: bool = False):
        nsplit = self._nsplit(rows)
        journal = journal and self.supports_journal
        if self.supports_journal:
            self.model.begin_journal(journal, rows)
        key = (rows, nsplit, self.feedback, topk, journal)
        if not self.use_graphs or rows > MAX_GRAPH_ROWS:
            self._forward_static(rows, nsplit, topk)
            return
        g = self.graphs.get(key)
        if g is None:
            g = self.graphs[key] = _Graph()
        g.calls += 1
        if g.graph is not None:
            g.graph.replay()
        elif g.calls == 1:
            self._forward_static(rows, nsplit, topk)
        else:
            torch.cuda.synchronize()
            graph = torch.cuda.CUDAGraph()
            with torch.cuda.graph(graph):
                self._forward_static(rows, nsplit, topk)
            g.graph = graph
            graph.replay()

    def set_rows(self, ids: list[int], pos: list[int], slots: list[int]):
        """Upload one step's row descriptor from pinned host memory (async on the current stream)."""
        n = len(ids)
        self.h_in[0, :n] = torch.tensor(ids, dtype=torch.int32)
        self.h_in[1, :n] = torch.tensor(pos, dtype=torch.int32)
        self.h_in[2, :n] = torch.tensor(slots, dtype=torch.int32)
        self.s_ids[:n].copy_(self.h_in[0, :n], non_blocking=True)
        self.s_pos[:n].copy_(self.h_in[1, :n], non_blocking=True)
        self.s_slot[:n].copy_(self.h_in[2, :n], non_blocking=True)

    @property
    def supports_journal(self) -> bool:
        """Models with recurrent state record verify blocks so that rejected rows can be taken back (``rollback``)."""
        return hasattr(self.model, "rollback_state")

    def rollback(self, slot: int, keep_rows: int) -> None:
        """After ``step(..., journal=True)`` over rows of ``slot``: keep the effect of the first ``keep_rows`` rows on the
        model's per-slot state (no-op for models whose only state is the KV pool)."""
        if self.supports_journal:
            self.model.rollback_state(slot, keep_rows)

    def step(self, ids: list[int], pos: list[int], slots: list[int], journal: bool = False) -> list[int]:
        """One batched decode / verify step with host round trip: H2D rows, forward, D2H tokens. ``journal``: the rows
        are a speculative block of one slot, part of which may be taken back with :meth:`rollback`."""
        n = len(ids)
        for s, p in zip(slots, pos):
            self.kv.reserve(s, p + 2)
        self.set_rows(ids, pos, slots)
        self._run_rows(n, journal=journal)
        self.h_tok[:n].copy_(self.s_tok[:n], non_blocking=True)
        if self.cuda:
            torch.cuda.current_stream().synchronize()
        return self.h_tok[:n].tolist()

    # ------------------------------------------------------------------------------------------ tree verification
    @property
    def supports_tree(self) -> bool:
        """Tree rows need a model whose only per-sequence state is the paged cache and whose attention takes the tree
        mask: the dense GQA family with plain residuals on one rank's rows (every rank runs the same rows under TP)."""
        m = self.model
        return (type(m).__name__ == "DenseModel" and getattr(m.cfg, "residual", "plain") == "plain"
                and not getattr(m.cfg, "mrope_sections", ()) and not getattr(m.cfg, "sliding_window", 0)
                and not getattr(m.cfg, "sandwich_norm", False))

    @property
    def max_tree_nodes(self) -> int:
        return min(64, int(self.s_tok.numel()))

    def step_tree(self, slot: int, pos0: int, tree) -> list[int]:
        """One forward over all nodes of ``tree`` (runtime.spec_tree.TokenTree) hanging off position ``pos0`` of
        ``slot``; returns the target's greedy token after every node. ``commit_tree`` keeps one branch afterwards."""
        n = len(tree)
        dev = self.device
        assert n <= self.max_tree_nodes, "the tree is larger than the engine's row buffers"
        self.kv.reserve(slot, pos0 + n + 1)
        b = BatchRows.make(tree.tokens, [pos0 + i for i in range(n)], [slot] * n, dev, LOGITS_ALL, 1, nsplit=self._nsplit(n))
        rope = torch.tensor([pos0 + d for d in tree.depths], dtype=torch.int32)
        b.pos3 = rope.unsqueeze(0).expand(3, n).contiguous().to(dev)
        masks = [m - (1 << 64) if m >= (1 << 63) else m for m in tree.masks]          # two's complement for int64
        b.tree = (torch.full((n,), pos0, dtype=torch.int32).to(dev), torch.tensor(masks, dtype=torch.int64).to(dev))
        logits = self.model.forward(b, self.kv)
        self._sample_greedy(logits, self.s_tok, self.s_val, n)
        self.h_tok[:n].copy_(self.s_tok[:n], non_blocking=True)
        if self.cuda:
            torch.cuda.current_stream().synchronize()
        return self.h_tok[:n].tolist()

    def commit_tree(self, slot: int, pos0: int, path: list[int]) -> None:
        """Keep the accepted branch: node path[d] (stored at pos0 + path[d]) becomes position pos0 + d."""
        self.kv.move_rows(slot, [pos0 + i for i in path], [pos0 + d for d in range(len(path))])

    def step_candidates(self, ids: list[int], pos: list[int], slots: list[int], journal: bool = False):
        """Like :meth:`step` but returns, per row, the merged top-16 candidates (ids, logits, lse) for the
        host sampler instead of the greedy token."""
        from .sampling import Candidates, merge_shards
        n = len(ids)
        for s, p in zip(slots, pos):
            self.kv.reserve(s, p + 2)
        self.set_rows(ids, pos, slots)
        self._run_rows(n, topk=True, journal=journal)
        cid, cval, clse = self.s_cand_ids[:n], self.s_cand_vals[:n], self.s_cand_lse[:n]
        if self.comm.size > 1:
            cid, cval, clse = (self.comm.all_gather_rows(t) for t in (cid, cval, clse))
        cid, cval, clse = cid.cpu(), cval.cpu(), clse.cpu()
        shards = max(1, self.comm.size)
        out = []
        for r in range(n):
            parts = [Candidates(cid[sh * n + r].tolist(), cval[sh * n + r].tolist(), float(clse[sh * n + r]))
                     for sh in range(shards)]
            out.append(merge_shards(parts))
        return out

    def set_rope_delta(self, slot: int, delta: int) -> None:
        """Rotary offset of a slot's decode rows (multimodal prompts advance the rotary position by less than their token
        count); 0 for text."""
        if self.mrope and self.h_delta[slot] != delta:
            self.h_delta[slot] = delta
            self.s_delta[slot] = delta

    def _mm_rows(self, b: BatchRows, slot: int, start_pos: int, c: int, mm) -> None:
        if not self.mrope:
            return
        if mm is not None:
            b.pos3, b.embeds, b.embed_mask = mm.chunk(start_pos, start_pos + c, self.device, self.model.cfg.hidden)
            self.set_rope_delta(slot, mm.delta)
        else:
            p = torch.arange(start_pos + self.h_delta[slot], start_pos + self.h_delta[slot] + c, dtype=torch.int32)
            b.pos3 = p.unsqueeze(0).expand(3, c).contiguous().to(self.device)

    def prefill_rows(self, slot: int, tokens: list[int], start_pos: int, want_token: bool, mm=None) -> int:
        """One prefill forward over ``tokens`` (<= prefill_chunk rows) of ``slot``; returns the greedy next
        token when ``want_token`` (else -1). Used by the scheduler to interleave prefill with decode steps."""
        c = len(tokens)
        self.kv.reserve(slot, start_pos + c + 1)
        G = self.model.nq // self.model.nkv
        pos = list(range(start_pos, start_pos + c))
        if c <= MAX_GRAPH_ROWS:
            b = BatchRows.make(tokens, pos, [slot] * c, self.device, LOGITS_ALL if want_token else LOGITS_NONE, G,
                               prefill=False, nsplit=self._nsplit(c))
        else:
            b = BatchRows.make(tokens, pos, [slot] * c, self.device, LOGITS_LAST if want_token else LOGITS_NONE, G,
                               prefill=True)
        self._mm_rows(b, slot, start_pos, c, mm)
        logits = self.model.forward(b, self.kv)
        if not want_token:
            return -1
        rows = logits.shape[0]
        self._sample_greedy(logits, self.s_tok, self.s_val, rows)
        return int(self.s_tok[rows - 1].item())

    def decode_chain(self, first_ids: list[int], pos: list[int], slots: list[int], steps: int) -> torch.Tensor:
        """``steps`` greedy steps for the given rows with the token fed back on the device (no host sync
        between steps). Returns the generated tokens [steps, rows] (device tensor)."""
        assert self.feedback
        n = len(first_ids)
        for s, p in zip(slots, pos):
            self.kv.reserve(s, p + steps + 2)
        self.set_rows(first_ids, pos, slots)
        out = torch.empty(steps, n, dtype=torch.int32, device=self.device)
        for i in range(steps):
            self._run_rows(n)
            out[i].copy_(self.s_tok[:n])
        return out

    # ------------------------------------------------------------------------------------------ generate
    def generate(self, prompt: list[int], max_new: int, slot: int = 0, eos: int | None = None):
        """Greedy generation for one sequence. Returns (tokens, GenStats)."""
        st = GenStats(prompt_tokens=len(prompt))
        t0 = time.perf_counter()
        tok = self.prefill(slot, prompt)
        if self.cuda:
            torch.cuda.synchronize()
        st.prefill_ms = (time.perf_counter() - t0) * 1e3
        out = [tok]
        pos = len(prompt)
        t1 = time.perf_counter()
        while len(out) < max_new and (eos is None or out[-1] != eos):
            tok = self.step([out[-1]], [pos], [slot])[0]
            out.append(tok)
            pos += 1
        st.decode_ms = (time.perf_counter() - t1) * 1e3
        st.new_tokens = len(out)
        return out, st
