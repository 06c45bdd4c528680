"""Request scheduler: slots, priority admission, interleaved chunked prefill, batched decode, speculative
rounds, sampling, stop conditions, prefix-cache resume and metrics.

Counterpart of the reference ``Generator`` (src/runtime/generator.cpp:117-205 admission and loop,
:213-349 emission rules, :576-717 prefill with prefix-cache resume, :948-1182 step selection) run on top
of :class:`~volta_engine_b200.runtime.engine.Engine`. One scheduler thread owns the engine; HTTP handlers
only enqueue requests and receive callbacks.
"""
from __future__ import annotations

import heapq
import itertools
import logging
import threading
import time
from collections import deque
from dataclasses import dataclass, field

from .loop_detect import LoopDetector
from .sampling import SamplingParams, TokenCounts, Xoshiro256pp, logprob_of, penalize, sample_token, spec_step
from .spec_controller import SpecController
from .suffix_index import SuffixIndex


log = logging.getLogger("volta.generator")

@dataclass
class Request:
    prompt: list[int]
    max_tokens: int = 256
    params: SamplingParams = field(default_factory=SamplingParams)
    stop: list[str] = field(default_factory=list)
    stop_token_ids: list[int] = field(default_factory=list)
    priority: int = 0
    on_text: object = None        # callable(text: str, token_ids: list[int], logprobs: list | None)
    on_finish: object = None      # callable(reason: str, usage: dict)
    on_wait: object = None        # callable() keep-alive while queued
    cache_prefix: bool = True
    checkpoints: list[int] = field(default_factory=list)   # extra snapshot positions (system prompt / turn ends)
    ignore_eos: bool = False
    # reasoning block control: the request starts inside an open block when the template opened it; after
    # ``thinking_budget`` reasoning tokens the closing sequence ``think_close`` is forced (soft close)
    think_open: bool = False
    think_end_id: int = -1        # id of the token that closes the block
    think_close: list[int] = field(default_factory=list)
    thinking_budget: int = 0      # 0 = unlimited
    mm: object = None             # runtime.multimodal.MmPrompt: rotary positions + image embedding rows of ``prompt``
    cache_key: list | None = None # prompt as the prefix cache sees it (image tokens replaced by content-derived ids)
    steer: object = None          # runtime.steering.SteerFile applied to this request's slot
    steer_scale: float = 1.0
    steer_scope: int | None = None
    steer_probe: bool = False     # probe this prompt with the forced openings and clamp the declining direction (runtime.steer_probe)
    think_penalty: float = 0.0    # logit taken from the first tokens of reflection markers inside the reasoning block
    id: int = 0
    cancelled: bool = False
    t_submit: float = 0.0


@dataclass
class SlotState:
    idx: int
    req: Request | None = None
    phase: str = "idle"           # idle | prefill | decode
    pos: int = 0                  # tokens whose KV is in the cache
    cursor: int = 0               # next prompt index to prefill
    cached_tokens: int = 0
    out: list[int] = field(default_factory=list)
    next_tok: int = -1            # sampled but not yet fed token
    counts: TokenCounts = field(default_factory=TokenCounts)
    rng: Xoshiro256pp | None = None
    loop: LoopDetector | None = None
    suffix: SuffixIndex | None = None
    ctrl: SpecController | None = None
    pending_bytes: bytes = b""    # undecodable UTF-8 tail
    held: str = ""                # text held back because it may be the start of a stop string
    t_start: float = 0.0
    t_first: float = 0.0
    t_prefill_ms: float = 0.0
    t_restore_ms: float = 0.0
    t_store_ms: float = 0.0
    last_emit: float = 0.0
    think_open: bool = False      # currently inside the reasoning block
    think_count: int = 0          # reasoning tokens produced so far
    last_char: str = ""           # last character of the previous reasoning token (soft close: "3." is not a sentence end)
    depth_rate: object = None     # DepthByRate of the slot's request (spec_depth_rate)
    probe_scores: dict | None = None   # what the request-time probe measured (reported in the usage)
    probe_file_scores: dict | None = None   # scores of the launch option's probe files at the prompt's last token
    forced: list = field(default_factory=list)   # tokens that replace the next sampled ones


class Metrics:
    def __init__(self):
        self.t0 = time.time()
        self.requests = self.completed = self.tokens_out = self.tokens_prefilled = 0
        self.prompt_tokens = self.cached_tokens = 0
        self.finished = {"stop": 0, "length": 0, "stop_string": 0, "cancelled": 0, "loop": 0}
        self.ttft_ms = deque(maxlen=512)
        self.gaps_ms = deque(maxlen=8192)
        self.recent = deque(maxlen=40)
        self.history = deque(maxlen=900)     # (t, decode tok/s, prefill tok/s, active)
        self.spec = {"rounds": 0, "proposed": 0, "accepted": 0, "suffix_rounds": 0, "steps": []}
        self._win = [time.time(), 0, 0]

    def tick(self, decoded: int, prefilled: int, active: int):
        self._win[1] += decoded
        self._win[2] += prefilled
        now = time.time()
        if now - self._win[0] >= 1.0:
            dt = now - self._win[0]
            self.history.append((now - self.t0, self._win[1] / dt, self._win[2] / dt, active))
            self._win = [now, 0, 0]

    @staticmethod
    def _pct(values, qs):
        v = sorted(values)
        if not v:
            return [0.0] * len(qs)
        return [v[min(len(v) - 1, int(q * len(v)))] for q in qs]

    def snapshot(self) -> dict:
        gaps = list(self.gaps_ms)
        hist = [0] * 12
        for g in gaps:
            b = 0
            while b < 11 and g >= (1 << b):
                b += 1
            hist[b] += 1
        n = max(1, self.completed)
        return {
            "totals": {"requests": self.requests, "completed": self.completed, "tokens_out": self.tokens_out,
                       "tokens_prefilled": self.tokens_prefilled, "prompt_tokens": self.prompt_tokens,
                       "cached_tokens": self.cached_tokens, "finished": dict(self.finished)},
            "averages": {"ttft_ms": sum(self.ttft_ms) / max(1, len(self.ttft_ms)),
                         "prefill_tok_s": sum(r["prefill_tok_s"] for r in self.recent) / max(1, len(self.recent)),
                         "decode_tok_s": sum(r["decode_tok_s"] for r in self.recent) / max(1, len(self.recent))},
            "latency": {"gap_ms": self._pct(gaps, (0.5, 0.9, 0.99, 0.999, 1.0)), "gap_samples": len(gaps),
                        "ttft_ms": self._pct(self.ttft_ms, (0.5, 0.9, 0.99)), "gap_hist": hist},
            "speculation": {"rounds": self.spec["rounds"], "proposed": self.spec["proposed"],
                            "accepted": self.spec["accepted"],
                            "accept_rate": self.spec["accepted"] / max(1, self.spec["proposed"]),
                            "tokens_per_round": (self.spec["accepted"] + self.spec["rounds"]) / max(1, self.spec["rounds"]),
                            "suffix": {"rounds": self.spec["suffix_rounds"], "proposed": self.spec["proposed"],
                                       "accepted": self.spec["accepted"]},
                            "steps": self.spec["steps"]},
            "recent": list(self.recent),
            "history": {"t": [h[0] for h in self.history], "decode": [h[1] for h in self.history],
                        "prefill": [h[2] for h in self.history], "active": [h[3] for h in self.history]},
            "uptime_s": time.time() - self.t0, "_n": n,
        }


class Generator:
    def __init__(self, engine, tokenizer, options=None, prefix_cache=None, eos_ids=None):
        self.engine, self.tok, self.opt, self.cache = engine, tokenizer, options, prefix_cache
        mdl = getattr(engine, "model", None)
        self._state_snaps = mdl is not None and getattr(mdl, "prefix_resume", "kv") == "kv+state"
        if self.cache is not None and mdl is not None and getattr(mdl, "prefix_resume", "kv") not in ("kv", "kv+state"):
            # snapshots hold KV pages only; this model keeps state elsewhere, and resuming would continue from whatever
            # the slot's previous request left there
            from ..utils import log
            log.warn("prefix cache disabled: %s keeps per-slot state outside the paged KV pool", type(mdl).__name__)
            self.cache = None
        self.max_slots = min(getattr(options, "max_slots", engine.kv.max_slots), engine.kv.max_slots) if options else engine.kv.max_slots
        self.slots = [SlotState(i) for i in range(self.max_slots)]
        self.eos_ids = set(eos_ids if eos_ids is not None else getattr(tokenizer, "eos_ids", []) or [])
        self.pending: list = []
        self._seq = itertools.count()
        self._ids = itertools.count(1)
        self.cv = threading.Condition()
        self.metrics = Metrics()
        self.running = False
        self.thread = None
        self.speculator = getattr(options, "speculator", "none") if options else "none"
        self.spec_depth = getattr(options, "spec_depth", 3) if options else 3
        self.use_ctrl = getattr(options, "spec_ctrl", True) if options else True
        self.loop_detect = getattr(options, "loop_detect", True) if options else True
        self.prefix_interval = getattr(options, "prefix_interval", 16384) if options else 16384
        self.budget_ms = getattr(options, "prefill_budget_ms", 50.0) if options else 50.0
        # extra decode steps that run between two prompt pieces while other slots decode (0 = a piece every step)
        self.prefill_cooldown = max(0, getattr(options, "prefill_cooldown", 0)) if options else 0
        self._since_prefill = 1 << 30
        self.cache_reply = getattr(options, "prefix_cache_reply", True) if options else True
        self.drafter = None                    # block drafter (speculator "dflash"): object with draft(slot, anchor, pos, depth)
        self.mtp = None
        if self.speculator == "mtp":
            from .mtp_runner import MtpRunner
            self.mtp = MtpRunner(engine, self.spec_depth)
            self.mtp.adaptive = self.use_ctrl               # the depth of a round follows the survival estimate
            # several decoding slots: one joint round (one draft chain, one verify block) for up to spec_joint_max of them
            self.mtp_joint = int(getattr(options, "spec_joint", -1)) == 1 if options else False
            self.mtp_joint_max = max(2, int(getattr(options, "spec_joint_max", 2))) if options else 2

    # ------------------------------------------------------------------------------------------ API
    def submit(self, req: Request) -> int:
        req.id = next(self._ids)
        req.t_submit = time.time()
        with self.cv:
            heapq.heappush(self.pending, (-req.priority, next(self._seq), req))
            self.metrics.requests += 1
            self.cv.notify()
        return req.id

    def cancel(self, req_id: int):
        with self.cv:
            for _, _, r in self.pending:
                if r.id == req_id:
                    r.cancelled = True
            for s in self.slots:
                if s.req is not None and s.req.id == req_id:
                    s.req.cancelled = True
            self.cv.notify()

    def start(self):
        self.running = True
        self.thread = threading.Thread(target=self._loop, name="volta-scheduler", daemon=True)
        self.thread.start()

    def stop(self):
        with self.cv:
            self.running = False
            self.cv.notify()
        if self.thread:
            self.thread.join(timeout=30)

    def generate(self, req: Request) -> dict:
        """Blocking helper: run one request to completion on the calling thread's behalf."""
        done = threading.Event()
        result = {"text": "", "tokens": [], "reason": None, "usage": None}

        def on_text(t, ids, lp):
            result["text"] += t
            result["tokens"].extend(ids)

        def on_finish(reason, usage):
            result["reason"], result["usage"] = reason, usage
            done.set()
        req.on_text, req.on_finish = on_text, on_finish
        self.submit(req)
        if self.thread is None:
            while not done.is_set():
                self.step()
        else:
            done.wait()
        return result

    # ------------------------------------------------------------------------------------------ loop
    def _loop(self):
        while True:
            with self.cv:
                while self.running and not self.pending and not any(s.phase != "idle" for s in self.slots):
                    self.cv.wait(timeout=0.5)
                if not self.running:
                    return
            try:
                self.step()
            except Exception as ex:   # fail the active requests, keep serving
                for s in self.slots:
                    if s.req is not None:
                        self._finish(s, "error", error=str(ex))
                if not self.running:
                    return

    def step(self):
        """One scheduler iteration: admit, one prefill slice, one decode / speculative step."""
        self._admit()
        prefilled = self._prefill_slice()
        decoded = self._decode_step()
        active = sum(1 for s in self.slots if s.phase != "idle")
        self.metrics.tick(decoded, prefilled, active)

    def _admit(self):
        with self.cv:
            while self.pending:
                free = next((s for s in self.slots if s.phase == "idle"), None)
                if free is None:
                    break
                _, _, req = heapq.heappop(self.pending)
                if req.cancelled:
                    if req.on_finish:
                        req.on_finish("cancelled", self._usage(req, 0, 0))
                    self.metrics.finished["cancelled"] += 1
                    continue
                need = len(req.prompt) + req.max_tokens + 1
                if not self.engine.kv.can_reserve(free.idx, min(need, self.engine.kv.max_pages * 64)):
                    heapq.heappush(self.pending, (-req.priority, next(self._seq), req))
                    break
                self._start(free, req)

    def _start(self, s: SlotState, req: Request):
        s.req, s.phase, s.pos, s.cursor, s.out, s.next_tok = req, "prefill", 0, 0, [], -1
        s.counts = TokenCounts()
        s.rng = None if req.params.greedy else Xoshiro256pp(req.params.seed if req.params.seed is not None else req.id)
        s.loop = LoopDetector() if self.loop_detect else None
        s.suffix = SuffixIndex(min_k=getattr(self.opt, "spec_suffix_min", 2) if self.opt else 2) if self.speculator == "suffix" else None
        s.ctrl = SpecController() if (self.speculator != "none" and self.use_ctrl) else None
        if s.ctrl is not None and self.opt is not None and getattr(self.opt, "spec_ctrl_log", False):
            s.ctrl.log_decisions = True
        s.pending_bytes, s.held = b"", ""
        s.t_start, s.t_first, s.t_prefill_ms, s.t_restore_ms, s.t_store_ms = time.time(), 0.0, 0.0, 0.0, 0.0
        s.cached_tokens = 0
        s.think_open, s.think_count, s.forced = req.think_open, 0, []
        s.depth_rate = None
        steer = getattr(getattr(self.engine, "model", None), "steer", None)
        if steer is not None:
            pen_ids = getattr(getattr(self, "steer_cfg", None), "penalty_ids", [])
            if req.steer is not None or (req.think_penalty > 0 and pen_ids):
                steer.set_slot(s.idx, req.steer, prompt_len=len(req.prompt), scale=req.steer_scale, scope=req.steer_scope,
                               penalty_ids=pen_ids if req.think_penalty > 0 else (), penalty=req.think_penalty)
            else:
                steer.clear_slot(s.idx)
        if len(req.prompt) == 0:
            req.prompt = [0]
        if getattr(self.engine, "mrope", False):
            self.engine.set_rope_delta(s.idx, req.mm.delta if req.mm is not None else 0)
        if self.cache is not None and req.cache_prefix:
            t0 = time.time()
            chain = self.cache.find(req.cache_key if req.cache_key is not None else req.prompt)
            snaps = []
            for node in chain:
                snap = self.cache.load(node)
                if snap is None:
                    break
                snaps.append((node, snap))
            if self._state_snaps:
                # the recurrent state is that of the last node of the chain: resume at the deepest node that holds one
                while snaps and "gdn_rec" not in snaps[-1][1]:
                    snaps.pop()
            for node, snap in snaps:
                self.engine.kv.load_rows(s.idx, snap)
                s.pos = s.cursor = node.end
            if self._state_snaps and snaps:
                self.engine.model.unpack_state(s.idx, snaps[-1][1], self.engine.kv)
            s.cached_tokens = s.pos
            s.t_restore_ms = (time.time() - t0) * 1e3
        if s.suffix is not None:
            s.suffix.extend(req.prompt)
        self.metrics.prompt_tokens += len(req.prompt)
        self.metrics.cached_tokens += s.cached_tokens

    # ------------------------------------------------------------------------------------------ prefill
    def _snapshot_points(self, s: SlotState) -> list[int]:
        n = len(s.req.prompt)
        pts = set(p for p in s.req.checkpoints if 0 < p < n)
        if self.prefix_interval > 0:
            pts.update(range(self.prefix_interval, n, self.prefix_interval))
        return sorted(pts)

    def _prefill_slice(self) -> int:
        s = next((x for x in self.slots if x.phase == "prefill"), None)
        if s is None:
            return 0
        if s.req.cancelled:
            self._finish(s, "cancelled")
            return 0
        decoding = any(x.phase == "decode" for x in self.slots)
        if decoding and self._since_prefill < self.prefill_cooldown:
            self._since_prefill += 1
            return 0
        self._since_prefill = 0
        chunk = self.engine.prefill_chunk
        done_rows, t0 = 0, time.time()
        prompt = s.req.prompt
        while s.cursor < len(prompt):
            end = min(len(prompt), s.cursor + chunk)
            for p in self._snapshot_points(s):          # stop at snapshot positions so they can be stored
                if s.cursor < p < end:
                    end = p
                    break
            last = end == len(prompt)
            if self.mtp is not None:
                tok = self.mtp.prefill_rows(s.idx, prompt, s.cursor, end, last)
            else:
                tok = self.engine.prefill_rows(s.idx, prompt[s.cursor:end], s.cursor, last, **({"mm": s.req.mm} if s.req.mm is not None else {}))
            done_rows += end - s.cursor
            s.cursor = s.pos = end
            if self.cache is not None and s.req.cache_prefix and (end in self._snapshot_points(s)):
                self._store_prefix(s, end)
            if last:
                if getattr(self, "probe_files", None):
                    tables = getattr(getattr(self.engine, "model", None), "steer", None)
                    if tables is not None:
                        from .steer_probe import score_probe_files
                        s.probe_file_scores = score_probe_files(self.engine, tables, s.idx, prompt, self.probe_files)
                if s.req.steer_probe and getattr(self, "probe_cfg", None) is not None:
                    tok = self._probe_steer(s, tok)
                s.next_tok = tok
                s.phase = "decode"
                s.t_prefill_ms += (time.time() - t0) * 1e3
                if not s.req.params.greedy:
                    # re-run the last row through the candidate path so the first token is sampled, not argmax
                    s.pos -= 1
                    cand = self.engine.step_candidates([prompt[-1]], [s.pos], [s.idx])[0]
                    s.pos += 1
                    cand = penalize(cand, s.req.params, s.counts.counts)
                    s.next_tok = sample_token(cand, s.req.params, s.rng)
                self.metrics.tokens_prefilled += done_rows
                self._emit(s, [s.next_tok])
                return done_rows
            if decoding and (time.time() - t0) * 1e3 >= self.budget_ms:
                break
        s.t_prefill_ms += (time.time() - t0) * 1e3
        self.metrics.tokens_prefilled += done_rows
        return done_rows

    def _store_prefix(self, s: SlotState, upto: int, pinned: bool = False):
        t0 = time.time()
        toks = ((s.req.cache_key if s.req.cache_key is not None else s.req.prompt) + s.out)[:upto]
        if self._state_snaps and upto != s.pos:
            return                 # the recurrent state belongs to position s.pos: no snapshot of an earlier point exists

        def snap(a, b):
            d = self.engine.kv.save_rows(s.idx, a, b)
            if self._state_snaps:
                d.update(self.engine.model.pack_state(s.idx))
            return d
        self.cache.insert(toks, upto, snap, pinned=pinned)
        s.t_store_ms += (time.time() - t0) * 1e3

    # ------------------------------------------------------------------------------------------ decode
    def _decode_step(self) -> int:
        act = [s for s in self.slots if s.phase == "decode"]
        for s in list(act):
            if s.req.cancelled:
                self._finish(s, "cancelled")
                act.remove(s)
        if not act:
            return 0
        # speculative round for one slot at a time when it is the only decoder (single-stream latency mode)
        budgeted = any(s.think_open and s.req.thinking_budget > 0 or s.forced for s in act)   # plain steps while a budget runs
        if not budgeted and self.speculator == "suffix" and len(act) == 1 and not act[0].req.params.logprobs:
            s = act[0]
            if s.ctrl is None or s.ctrl.use_speculation():
                n = self._suffix_round(s)
                if n:
                    return n
        if not budgeted and self.drafter is not None and len(act) == 1 and not act[0].req.params.logprobs:
            s = act[0]
            if s.ctrl is None or s.ctrl.use_speculation():
                depth = s.ctrl.depth(self.spec_depth) if s.ctrl else self.spec_depth
                if self.opt is not None and getattr(self.opt, "spec_depth_rate", False):
                    from .spec_controller import DepthByRate
                    if getattr(s, "depth_rate", None) is None:
                        s.depth_rate = DepthByRate(self.spec_depth)
                    depth = s.depth_rate.choose(self.spec_depth)
                n = self._verify_round(s, self.drafter.draft(s.idx, s.next_tok, s.pos, depth), "drafter")
                if n:
                    return n
        if not budgeted and self.mtp is not None and len(act) == 1 and act[0].req.params.greedy and act[0].idx in self.mtp.hidden:
            s = act[0]
            if s.ctrl is None or s.ctrl.use_speculation():
                return self._mtp_round(s)
        if (not budgeted and self.mtp is not None and getattr(self, "mtp_joint", False) and 2 <= len(act) <= self.mtp_joint_max
                and all(s.req.params.greedy and s.idx in self.mtp.hidden for s in act) and self.mtp._device_round_ok(len(act))):
            return self._mtp_round_joint(act)
        t0 = time.time()
        ids = [s.next_tok for s in act]
        pos = [s.pos for s in act]
        slots = [s.idx for s in act]
        greedy = all(s.req.params.greedy and not s.req.params.logprobs for s in act)
        if greedy:
            toks = self.engine.step(ids, pos, slots)
            cands = [None] * len(act)
        else:
            cands = self.engine.step_candidates(ids, pos, slots)
            toks = []
            for s, c in zip(act, cands):
                c2 = penalize(c, s.req.params, s.counts.counts)
                toks.append(sample_token(c2, s.req.params, s.rng))
        ms = (time.time() - t0) * 1e3
        if self.mtp is not None:
            if len(act) == 1:
                self.mtp.after_plain_step(act[0].idx, ids[0], pos[0], toks[0])
            else:
                for s in act:            # batched plain steps do not maintain the head: drop its state
                    self.mtp.release(s.idx)
        self._decode_steps = getattr(self, "_decode_steps", 0) + 1
        mdl = getattr(self.engine, "model", None)
        every = getattr(mdl, "expert_adapt_every", 0) if mdl is not None else 0
        if every and self._decode_steps % every == 0:
            swaps = mdl.rebalance_experts(getattr(mdl, "expert_max_swaps", 2))      # expert residency follows the routing heat
            if self.opt is not None and getattr(self.opt, "expert_log", False):
                log.info("expert tier: step %d, %s swaps this rebalance", self._decode_steps, swaps)
        for s, t, c in zip(act, toks, cands):
            t = self._think_gate(s, t)
            s.pos += 1
            s.next_tok = t
            if s.ctrl is not None:
                s.ctrl.record_plain(ms)
            lp = None
            if c is not None and s.req.params.logprobs:
                lp = [{"token": t, "logprob": logprob_of(c, t),
                       "top": [(i, l - c.lse) for i, l in list(zip(c.ids, c.logits))[: s.req.params.logprobs]]}]
            self._emit(s, [t], lp)
        return len(act)

    def _think_gate(self, s: SlotState, t: int) -> int:
        """Reasoning budget: counts tokens inside the open block and, once the budget is spent, replaces the sampled
        tokens by the closing sequence (the model then continues with its answer)."""
        req = s.req
        if s.forced:
            t = s.forced.pop(0)
        elif s.think_open and req.thinking_budget > 0 and req.think_close:
            if t != req.think_end_id and s.think_count + 1 >= req.thinking_budget:
                # The budget is spent. Soft close (reference: docs/CONFIG.md:122, thinking_soft_close): the block closes
                # after the next token that ends a sentence (. ! ?, not a "." behind a digit) or a line, at most
                # ``soft_close`` tokens later; 0 closes right here.
                over = s.think_count + 1 - req.thinking_budget
                soft = int(getattr(self.opt, "thinking_soft_close", 0) or 0) if self.opt is not None else 0
                if over >= soft or self._ends_sentence(s, t):
                    if over >= soft:
                        s.forced = list(req.think_close)
                        t = s.forced.pop(0)
                    else:
                        s.forced = list(req.think_close)      # this token ends the sentence: it stays, the close follows
        if s.think_open:
            if t == req.think_end_id:
                s.think_open = False
                steer = getattr(getattr(self.engine, "model", None), "steer", None)
                if steer is not None and req.steer is not None:
                    steer.set_think_end(s.idx, s.pos + 1)
            else:
                s.think_count += 1
                if req.thinking_budget > 0 and s.think_count + 2 >= req.thinking_budget:
                    try:                      # only near and past the budget: the soft close looks one character back
                        piece = self.tok.decode_bytes([t]).decode("utf-8", "ignore")
                        s.last_char = piece[-1:] if piece else s.last_char
                    except Exception:
                        pass
        return t

    def _probe_steer(self, s: SlotState, tok: int) -> int:
        """Request-time probe (runtime.steer_probe): the forced openings run behind the prompt, the clamps they call for are
        installed beside the request's control vectors, and the prompt's last row runs again so that the first token
        already comes from the edited stream. Returns that token."""
        from .steer_probe import probe_request
        from .steering import SteerFile
        tables = getattr(getattr(self.engine, "model", None), "steer", None)
        req = s.req
        if tables is None or len(req.prompt) < 1:
            return tok
        edits, scores = probe_request(self.engine, tables, self.tok, s.idx, req.prompt, self.probe_cfg)
        s.probe_scores = scores
        if edits is None:
            return tok
        base = req.steer
        merged = SteerFile(hidden=edits.hidden, layers=edits.layers, scope=edits.scope, scale=base.scale if base is not None else 1.0,
                           entries=(list(base.entries) if base is not None else []) + list(edits.entries))
        pen_ids = getattr(getattr(self, "steer_cfg", None), "penalty_ids", [])
        try:
            tables.set_slot(s.idx, merged, prompt_len=len(req.prompt), scale=req.steer_scale, scope=edits.scope,
                            penalty_ids=pen_ids if req.think_penalty > 0 else (), penalty=req.think_penalty)
        except ValueError:                         # more than four edits on a layer: the probe's edits give way
            scores["edits"] = 0
            return tok
        if req.steer is None:
            req.steer = merged                     # the slot is steered from here on (think-end tracking, clear at finish)
        return self.engine.step([req.prompt[-1]], [len(req.prompt) - 1], [s.idx])[0]

    def _ends_sentence(self, s: SlotState, t: int) -> bool:
        try:
            piece = self.tok.decode_bytes([t]).decode("utf-8", "ignore").rstrip(" ")
        except Exception:
            return False
        if not piece:
            return False
        if piece.endswith("\n"):
            return True
        if piece[-1] in "!?":
            return True
        if piece[-1] == ".":
            before = piece[-2] if len(piece) > 1 else s.last_char
            return not before.isdigit()
        return False

    def _mtp_round(self, s: SlotState) -> int:
        t0 = time.time()
        new = self.mtp.round(s.idx, s.next_tok, s.pos)
        return self._mtp_account(s, new, (time.time() - t0) * 1e3)

    def _mtp_round_joint(self, act: list) -> int:
        t0 = time.time()
        news = self.mtp.round_joint([s.idx for s in act], [s.next_tok for s in act], [s.pos for s in act])
        ms = (time.time() - t0) * 1e3
        return sum(self._mtp_account(s, new, ms / len(act)) for s, new in zip(act, news))

    def _mtp_account(self, s: SlotState, new: list[int], ms: float) -> int:
        depth = self.mtp.last_depth
        acc = len(new) - 1
        s.pos += acc + 1
        s.next_tok = new[-1]
        m = self.metrics.spec
        m["rounds"] += 1
        m["proposed"] += depth
        m["accepted"] += acc
        while len(m["steps"]) < depth:
            m["steps"].append({"attempts": 0, "hits": 0})
        for i in range(depth):
            m["steps"][i]["attempts"] += 1
            m["steps"][i]["hits"] += 1 if i < acc else 0
        if s.ctrl:
            s.ctrl.record_round(len(new), depth, acc, ms)
        self._emit(s, new)
        return len(new)

    def _suffix_round(self, s: SlotState) -> int:
        depth = s.ctrl.depth(self.spec_depth) if s.ctrl else self.spec_depth
        width = int(getattr(self.opt, "spec_tree", 0) or 0) if self.opt is not None else 0
        if width > 1 and s.req.params.greedy and getattr(self.engine, "supports_tree", False):
            # several earlier occurrences of the suffix continue differently: verify them as one tree
            from .spec_tree import TokenTree
            paths = s.suffix.draft_paths(depth, width)
            if len(paths) > 1:
                return self._tree_round(s, TokenTree.from_paths(s.next_tok, paths, self.engine.max_tree_nodes), "suffix")
            return self._verify_round(s, paths[0] if paths else [], "suffix")
        return self._verify_round(s, s.suffix.draft(depth), "suffix")

    def _tree_round(self, s: SlotState, tree, kind: str) -> int:
        """One target forward over every node of the tree; the branch the target agrees with is kept (its cache rows
        moved to consecutive positions), the target's token after its last node is the bonus token."""
        t0 = time.time()
        targets = self.engine.step_tree(s.idx, s.pos, tree)
        path, new = tree.accept(targets)
        self.engine.commit_tree(s.idx, s.pos, path)
        acc = len(path) - 1
        ms = (time.time() - t0) * 1e3
        s.pos += acc + 1
        s.next_tok = new[-1]
        m = self.metrics.spec
        m["rounds"] += 1
        m["tree_rounds"] = m.get("tree_rounds", 0) + 1
        m["tree_nodes"] = m.get("tree_nodes", 0) + len(tree) - 1
        m["suffix_rounds"] += 1 if kind == "suffix" else 0
        deepest = max(tree.depths)
        m["proposed"] += deepest
        m["accepted"] += acc
        if s.ctrl:
            s.ctrl.record_round(len(new), deepest, acc, ms)
        self._emit(s, new)
        return len(new)

    def _verify_round(self, s: SlotState, drafts: list[int], kind: str) -> int:
        """One target forward over [next token, drafts...]; keeps the longest prefix the target agrees with."""
        if not drafts:
            return 0
        t0 = time.time()
        rows = [s.next_tok] + drafts
        pos = [s.pos + i for i in range(len(rows))]
        params = s.req.params
        jn = {"journal": True} if getattr(self.engine, "supports_journal", False) else {}
        spool = getattr(self, "target_spool", None)
        if params.greedy and spool is not None and spool.on() and kind == "drafter":
            # the tap spool wants the target's candidates at the emitted positions: the same step with its top-16 read back
            cands = self.engine.step_candidates(rows, pos, [s.idx] * len(rows), **jn)
            toks = [c.ids[max(range(len(c.ids)), key=lambda i: (c.logits[i], -c.ids[i]))] for c in cands]
            acc = 0
            while acc < len(drafts) and toks[acc] == drafts[acc]:
                acc += 1
            new = drafts[:acc] + [toks[acc]]
            for i in range(acc + 1):
                spool.add(s.idx, pos[i] + 1, cands[i].logits, cands[i].ids)
        elif params.greedy:
            toks = self.engine.step(rows, pos, [s.idx] * len(rows), **jn)
            # longest accepted prefix: draft i is accepted when the model's token after row i equals it
            acc = 0
            while acc < len(drafts) and toks[acc] == drafts[acc]:
                acc += 1
            new = drafts[:acc] + [toks[acc]]
        else:
            # sampled requests: exact speculative sampling against the point-mass proposal of each draft. Row i is
            # judged with the penalties of everything committed before it (the drafts accepted so far included), so the
            # tokens are distributed exactly as one-row sampling steps would give them.
            cands = self.engine.step_candidates(rows, pos, [s.idx] * len(rows), **jn)
            counts = dict(s.counts.counts)
            new, acc = [], 0
            for i in range(len(rows)):
                c = penalize(cands[i], params, counts)
                if i == len(drafts):
                    new.append(sample_token(c, params, s.rng))
                    break
                ok, t = spec_step(c, params, drafts[i], s.rng)
                new.append(t)
                counts[t] = counts.get(t, 0) + 1
                if not ok:
                    break
                acc += 1
            toks = new + [new[-1]] * (len(rows) - len(new))
        if jn and acc < len(drafts):
            self.engine.rollback(s.idx, acc + 1)          # recurrent state: as if only the accepted rows had run
        ms = (time.time() - t0) * 1e3
        s.pos += acc + 1
        s.next_tok = new[-1]
        m = self.metrics.spec
        m["rounds"] += 1
        m["suffix_rounds"] += 1 if kind == "suffix" else 0
        m["proposed"] += len(drafts)
        m["accepted"] += acc
        while len(m["steps"]) < len(drafts):
            m["steps"].append({"attempts": 0, "hits": 0})
        for i in range(len(drafts)):
            m["steps"][i]["attempts"] += 1
            m["steps"][i]["hits"] += 1 if i < acc else 0
        if s.ctrl:
            s.ctrl.record_round(len(new), len(drafts), acc, ms)
        if kind == "drafter" and getattr(s, "depth_rate", None) is not None:
            s.depth_rate.record(len(drafts), acc, ms)
        if kind == "drafter" and self.drafter is not None and hasattr(self.drafter, "observe_commit"):
            self.drafter.observe_commit(new)                       # sparse-head evidence, hits and misses
            if self.drafter.sparse_policy is not None:
                self.drafter.sparse_policy.round_time(ms, len(drafts))
        log = getattr(self, "cand_log", None)
        if log is not None and log.on() and kind == "drafter":
            log.round(s.idx, s.pos - acc - 1, rows[0], len(drafts),
                      [(drafts[i], toks[i], [0.0], [drafts[i]]) for i in range(min(acc + 1, len(drafts)))])
        self._emit(s, new)
        return len(new)

    # ------------------------------------------------------------------------------------------ emission
    def _emit(self, s: SlotState, toks: list[int], logprobs=None):
        """Deliver newly sampled tokens: EOS / stop ids, length, stop strings with hold-back, UTF-8 boundary,
        loop detection. The last token of ``toks`` is the next one to feed."""
        req = s.req
        now = time.time()
        if not s.out:
            s.t_first = now
            self.metrics.ttft_ms.append((now - req.t_submit) * 1e3)
        elif s.last_emit:
            self.metrics.gaps_ms.append((now - s.last_emit) * 1e3 / max(1, len(toks)))
        s.last_emit = now
        for i, t in enumerate(toks):
            if (t in self.eos_ids or t in req.stop_token_ids) and not req.ignore_eos:
                self._flush_text(s, final=True)
                self._finish(s, "stop")
                return
            s.out.append(t)
            s.counts.add(t)
            if s.suffix is not None:
                s.suffix.push(t)
            self.metrics.tokens_out += 1
            piece = s.pending_bytes + self.tok.decode_bytes([t])
            text, s.pending_bytes = _utf8_split(piece)
            if text or True:
                hit = self._deliver(s, text, [t], logprobs if i == len(toks) - 1 else None)
                if hit:
                    self._finish(s, "stop_string")
                    return
            if len(s.out) >= req.max_tokens:
                self._flush_text(s, final=True)
                self._finish(s, "length")
                return
            if s.pos + 2 >= self.engine.kv.max_pages * 64:
                self._flush_text(s, final=True)
                self._finish(s, "length")
                return
            if s.loop is not None and s.loop.push(t):
                self._flush_text(s, final=True)
                self._finish(s, "loop")
                return

    def _deliver(self, s: SlotState, text: str, ids: list[int], logprobs) -> bool:
        """Stop-string handling: text that could be the beginning of a stop string is held back."""
        req = s.req
        if not req.stop:
            if req.on_text and (text or ids):
                req.on_text(text, ids, logprobs)
            return False
        buf = s.held + text
        for st in req.stop:
            k = buf.find(st)
            if k >= 0:
                if req.on_text and buf[:k]:
                    req.on_text(buf[:k], ids, logprobs)
                s.held = ""
                return True
        hold = 0
        for st in req.stop:
            for k in range(min(len(st) - 1, len(buf)), 0, -1):
                if buf.endswith(st[:k]):
                    hold = max(hold, k)
                    break
        out, s.held = (buf[:-hold], buf[-hold:]) if hold else (buf, "")
        if req.on_text and (out or ids):
            req.on_text(out, ids, logprobs)
        return False

    def _flush_text(self, s: SlotState, final: bool):
        if s.held and s.req.on_text:
            s.req.on_text(s.held, [], None)
        s.held = ""
        if final and s.pending_bytes and s.req.on_text:
            s.req.on_text(s.pending_bytes.decode("utf-8", errors="replace"), [], None)
        s.pending_bytes = b""

    def _usage(self, req: Request, generated: int, cached: int) -> dict:
        return {"prompt_tokens": len(req.prompt), "completion_tokens": generated, "cached_tokens": cached,
                "total_tokens": len(req.prompt) + generated}

    def _finish(self, s: SlotState, reason: str, error: str | None = None):
        req = s.req
        now = time.time()
        if self.cache is not None and self.cache_reply and req.cache_prefix and reason in ("stop", "length", "stop_string") and s.pos > 0:
            try:                                   # reply snapshot: the next turn resumes after this answer
                self._store_prefix(s, min(s.pos, len(req.prompt) + len(s.out)))
            except Exception:
                pass
        dec_s = max(1e-6, now - (s.t_first or now))
        rec = {"req_id": req.id, "age_s": 0.0, "prompt_tokens": len(req.prompt), "cached_tokens": s.cached_tokens,
               "generated": len(s.out), "queue_ms": (s.t_start - req.t_submit) * 1e3,
               "ttft_ms": ((s.t_first or now) - req.t_submit) * 1e3, "restore_ms": s.t_restore_ms,
               "prefill_ms": s.t_prefill_ms, "store_ms": s.t_store_ms, "total_ms": (now - req.t_submit) * 1e3,
               "decode_tok_s": max(0, len(s.out) - 1) / dec_s,
               "prefill_tok_s": (len(req.prompt) - s.cached_tokens) / max(1e-6, s.t_prefill_ms / 1e3), "reason": reason}
        self.metrics.recent.append(rec)
        self.metrics.completed += 1
        if reason in self.metrics.finished:
            self.metrics.finished[reason] += 1
        usage = self._usage(req, len(s.out), s.cached_tokens)
        if getattr(s, "probe_scores", None):
            usage["steer_probe"] = s.probe_scores
            s.probe_scores = None
        if getattr(s, "probe_file_scores", None):
            usage["probes"] = s.probe_file_scores
            s.probe_file_scores = None
        if error:
            usage["error"] = error
        tap_file = getattr(self, "tap_spool", None)
        if tap_file is not None and self.drafter is not None and getattr(self.drafter, "ring", None) is not None:
            try:                                   # offline drafter training: tokens, last taps, the target's candidates
                end = min(s.pos, len(req.prompt) + len(s.out))
                lo = max(0, end - min(tap_file.window, self.drafter.ring.cap))
                tgt = self.target_spool.take(s.idx) if getattr(self, "target_spool", None) is not None else []
                tap_file.write(list(req.prompt) + list(s.out), self.drafter.ring.rows(s.idx, lo, end) if end > lo else None, lo, tgt)
            except Exception as e:
                log.warning("tap spool: %s", e)
        self.engine.kv.release(s.idx)
        if self.mtp is not None:
            self.mtp.release(s.idx)
        if self.drafter is not None:
            self.drafter.release(s.idx)
        steer = getattr(getattr(self.engine, "model", None), "steer", None)
        if steer is not None and req.steer is not None:
            steer.clear_slot(s.idx)
        s.req, s.phase = None, "idle"
        if req.on_finish:
            req.on_finish(reason, usage)

    # ------------------------------------------------------------------------------------------ monitor
    def slot_views(self) -> list[dict]:
        now = time.time()
        out = []
        for s in self.slots:
            r = s.req
            out.append({"slot": s.idx, "active": r is not None, "phase": s.phase, "req_id": r.id if r else 0,
                        "pos": s.pos, "prompt_tokens": len(r.prompt) if r else 0, "cached_tokens": s.cached_tokens,
                        "generated": len(s.out), "max_tokens": r.max_tokens if r else 0,
                        "age_s": now - s.t_start if r else 0.0,
                        "decode_tok_s": (len(s.out) / max(1e-6, now - s.t_first)) if (r and s.t_first) else 0.0})
        return out

    def queued(self) -> int:
        return len(self.pending)


def _utf8_split(b: bytes) -> tuple[str, bytes]:
    """Decode the longest prefix of ``b`` that ends on a code-point boundary; return (text, remaining tail)."""
    n = len(b)
    cut = n
    for back in range(1, min(4, n) + 1):
        c = b[n - back]
        if c & 0xC0 == 0x80:
            continue
        need = 1 if c < 0x80 else 2 if c >> 5 == 6 else 3 if c >> 4 == 14 else 4 if c >> 3 == 30 else 1
        if need > back:
            cut = n - back
        break
    return b[:cut].decode("utf-8", errors="replace"), b[cut:]
