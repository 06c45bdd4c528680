"""Block drafter speculation (DFlash): a small decoder that reads tapped hidden states of the target model and proposes a
whole block of tokens in one forward.

Round (reference: inc/engine/runtime/dflash2_runner.h:26-60, inc/engine/spec/dflash.h:20-62, src/spec/tap_ring.cu):
  * the target publishes the output of ``target_layer_ids`` for every row it forwards into a per-slot position ring
    (``TapRing``; slot and position come from device memory, so the launch replays in CUDA graphs);
  * the drafter projects the concatenated taps of every known position through ``fc`` + RMSNorm into its context and
    stores that context's keys and values, layer by layer, in its own paged cache;
  * a block of ``block_size`` rows (the anchor token followed by mask tokens) runs through the drafter with attention over
    the context and, bidirectionally, over the block itself; row i of the block proposes the token at position pos + i
    (version 1: the head's argmax per row; version 2: every sub-layer of the drafter is wrapped in a pair of grouped
    dynamic convolutions over the block's rows whose per-row kernels are a projection of the normed input, the residual
    stream is fp32, and the tokens are chosen by a chained walk over the top-16 candidates of every row with a low-rank
    pairwise term between the previous choice and each candidate; ``_forward_v2`` / ``walk_candidates``,
    reference: src/spec/dflash_backbone.cu:186-350, inc/engine/spec/dflash.h:96-140);
  * the target verifies ``[anchor, drafts...]`` in ONE forward and keeps the longest agreeing prefix (generator).
The drafter shares the target's embedding and LM head. Drafter context belongs to a slot; every slot has its own ring.
"""
from __future__ import annotations

from dataclasses import dataclass, field

import torch

from .._lib import call, ptr
from ..models.dense import DenseConfig, DenseModel
from ..ops import kernels as K
from ..ops.linear import LinearBF16
from .batch import BatchRows, LOGITS_ALL, LOGITS_NONE
from .kv_cache import PagedKVCache


@dataclass
class DFlashConfig:
    block_size: int = 8
    n_layers: int = 5
    hidden: int = 5120
    n_q: int = 32
    n_kv: int = 8
    head_dim: int = 128
    ffn: int = 17408
    target_layer_ids: tuple = (5, 19, 33, 47, 61)
    sliding_window: int = 2048
    rope_theta: float = 1.0e7
    rms_eps: float = 1e-6
    mask_token_id: int = 0
    tap_cap: int = 2048
    version: int = 1
    quant: str = "bf16"
    conv_kernel_size: int = 2      # version 2: taps of the dynamic convolutions
    conv_group_size: int = 16      # channels that share one dynamic coefficient
    selector_rank: int = 256       # width of the pairwise term of the candidate walk
    selector_top_k: int = 16       # candidates per block row


class TapRing:
    """[slots, cap, n_taps * H] bf16: tap t of position p of a slot lives in row p % cap."""

    def __init__(self, slots: int, cap: int, layer_ids, hidden: int, device):
        self.layer_ids = tuple(layer_ids)
        self.index = {l: i for i, l in enumerate(self.layer_ids)}
        self.cap, self.H, self.n = cap, hidden, len(self.layer_ids)
        self.taps = torch.zeros(slots, cap, self.n * hidden, dtype=torch.bfloat16, device=device)

    def publish(self, li: int, h: torch.Tensor, pos: torch.Tensor, slot: torch.Tensor, rows: int):
        t = self.index.get(li)
        if t is None:
            return
        if not h.is_cuda:
            for r in range(rows):
                s, p = int(slot[r]), int(pos[r])
                if s >= 0 and p >= 0:
                    self.taps[s, p % self.cap, t * self.H:(t + 1) * self.H] = h[r].to(torch.bfloat16)
            return
        call("publish_taps", "pplippp" + "iiiili", ptr(self.taps), ptr(h), h.stride(0), 1 if h.dtype == torch.float32 else 0,
             ptr(slot), ptr(pos), 0, rows, t, self.H, self.cap, self.taps.stride(0), self.n)

    def rows(self, slot: int, p0: int, p1: int) -> torch.Tensor:
        idx = torch.arange(p0, p1, device=self.taps.device) % self.cap
        return self.taps[slot, idx]


class DFlashRunner:
    def __init__(self, engine, cfg: DFlashConfig, seed: int = 11):
        self.e, self.cfg = engine, cfg
        tgt = engine.model
        dev = engine.device
        tc = tgt.cfg
        assert cfg.hidden == tc.hidden, "the drafter works at the target's hidden size"
        self.ring = TapRing(engine.kv.max_slots, cfg.tap_cap, cfg.target_layer_ids, cfg.hidden, dev)
        tgt.tap_ring = self.ring
        dcfg = DenseConfig(n_layers=cfg.n_layers, hidden=cfg.hidden, n_q=cfg.n_q, n_kv=cfg.n_kv, head_dim=cfg.head_dim, ffn=cfg.ffn,
                           vocab=tc.vocab, rope_theta=cfg.rope_theta, rms_eps=cfg.rms_eps, qk_norm=True,
                           sliding_window=cfg.sliding_window, quant=cfg.quant)
        # tensor parallel like the target: heads and MLP columns split over the ranks, every rank runs the same calls
        comm = getattr(tgt, "comm", None)
        self.model = DenseModel(dcfg, dev, comm if (comm is not None and getattr(comm, "size", 1) > 1) else None).init_random(seed=seed)
        self.model.embed, self.model.lm_head = tgt.embed, tgt.lm_head            # shared with the target
        self.model.vocab_local = tgt.vocab_local
        g = torch.Generator(device=dev).manual_seed(seed + 1)
        self.fc = LinearBF16((torch.randn(cfg.hidden, self.ring.n * cfg.hidden, generator=g, device=dev) * 0.02).to(torch.bfloat16))
        self.hidden_norm = torch.ones(cfg.hidden, dtype=torch.bfloat16, device=dev)
        span = max(cfg.tap_cap, cfg.sliding_window) + 2 * cfg.block_size
        pages = engine.kv.max_slots * (PagedKVCache.pages_for(span) + 3) + 1
        self.kv = PagedKVCache(cfg.n_layers, self.model.nkv, cfg.head_dim, pages, engine.kv.max_slots,
                               engine.kv.max_pages * 64, dev)
        self.ctx_len = [0] * engine.kv.max_slots
        self.model.ensure_workspace(max(64, cfg.block_size), 8)
        self.stats = {"rounds": 0, "proposed": 0, "accepted": 0}
        self.v2 = None
        if cfg.version == 2:
            self._init_v2(g, tc.vocab)
        self.last_conf = None
        self.sparse_policy = None            # host policy of the sparse drafter head (enable_sparse_head)
        self.sparse_head = None
        self.sparse_state_path = None

    # ---- weights of a trained drafter: same tensor names as a dense decoder plus ``fc`` and ``hidden_norm``
    def load(self, src) -> None:
        from ..models.factory import load_dense_weights
        keep = self.model.embed, self.model.lm_head
        load_dense_weights(self.model, src)
        self.model.embed, self.model.lm_head = keep
        self.fc = LinearBF16(src.tensor("fc.weight", self.e.device, torch.bfloat16))
        self.hidden_norm = src.tensor("hidden_norm.weight", self.e.device, torch.bfloat16)
        if self.v2 is not None:
            # version-2 tensors (names of the reference's loader, src/spec/dflash_speculator.cu:363-454): per layer the two
            # convolution pairs' static kernels and coefficient projections, then the candidate selector
            dev, bf = self.e.device, torch.bfloat16

            def get(name):
                return src.tensor(name if src.has(name) else name + ".weight", dev, bf)
            for i, V in enumerate(self.v2["layers"]):
                for ours, theirs in (("attn", "attention_conv"), ("mlp", "mlp_conv")):
                    V[ours + "_base"] = get(f"layers.{i}.{theirs}.base_kernel").reshape(2 * self.cfg.conv_kernel_size, self.cfg.hidden).contiguous()
                    V[ours + "_proj"] = LinearBF16(get(f"layers.{i}.{theirs}.kernel_projection"))
            self.v2["gate"] = LinearBF16(get("candidate_selector.hidden_projection"))
            self.v2["pred"] = get("candidate_selector.predecessor_codebook")
            self.v2["succ"] = get("candidate_selector.successor_codebook")

    def release(self, slot: int) -> None:
        self.ctx_len[slot] = 0
        self.kv.release(slot)

    # ---- launch option spec_profile: wall time of a round's stages, the device drained at every stage boundary
    def enable_profile(self) -> None:
        self.profile = {"rounds": 0, "ingest_ms": 0.0, "backbone_ms": 0.0, "select_ms": 0.0}

    def _mark(self, key: str, t0: float) -> float:
        import time
        if self.e.cuda:
            torch.cuda.synchronize(self.e.device)
        t1 = time.perf_counter()
        self.profile[key] += (t1 - t0) * 1e3
        return t1

    def profile_report(self) -> dict:
        pr = getattr(self, "profile", None)
        if not pr or not pr["rounds"]:
            return {}
        return {k: (round(v / pr["rounds"], 4) if k != "rounds" else v) for k, v in pr.items()}

    # ---- version 2: dynamic convolutions around every sub-layer, candidate selector
    def _init_v2(self, g, vocab: int) -> None:
        """Random weights of the version-2 parts. Per layer and sub-layer (attention, MLP): ``proj`` [2 * taps * groups,
        H] emits the coefficients of both convolutions of the pair (side 0: in front of the sub-layer, side 1: behind
        it; within a side [tap][group]) and ``base`` [2 * taps, H] holds the static kernels of the two sides. Selector:
        ``gate`` [rank, H] projects a block row's hidden state, ``pred`` / ``succ`` [vocab, rank] are the codebooks of
        the previous token and of a candidate."""
        cfg, dev, bf = self.cfg, self.e.device, torch.bfloat16
        H, taps, G = cfg.hidden, cfg.conv_kernel_size, cfg.hidden // cfg.conv_group_size
        assert H % cfg.conv_group_size == 0

        def rnd(*shape, std):
            return (torch.randn(*shape, generator=g, device=dev) * std).to(bf)

        def base():
            b = rnd(2 * taps, H, std=0.02)
            b[0] += 1.0                          # tap 0 of both sides starts as the identity: a fresh drafter is a v1 drafter
            b[taps] += 1.0
            return b.contiguous()
        self.v2 = {"layers": [{"attn_proj": LinearBF16(rnd(2 * taps * G, H, std=0.02)), "attn_base": base(),
                               "mlp_proj": LinearBF16(rnd(2 * taps * G, H, std=0.02)), "mlp_base": base()}
                              for _ in range(cfg.n_layers)],
                   "gate": LinearBF16(rnd(cfg.selector_rank, H, std=0.05)),
                   "pred": rnd(vocab, cfg.selector_rank, std=0.3), "succ": rnd(vocab, cfg.selector_rank, std=0.3)}

    @staticmethod
    def _norm_f32(res: torch.Tensor, w: torch.Tensor, eps: float) -> torch.Tensor:
        """RMSNorm of the fp32 residual stream, rounded to bf16 for the projections that follow."""
        y = res * torch.rsqrt((res * res).mean(-1, keepdim=True) + eps) * w.float()
        return y.to(torch.bfloat16)

    def _forward_v2(self, b: BatchRows) -> torch.Tensor:
        """The version-2 drafter over one block: returns the final-normed hidden rows [block, H] (bf16). Per layer:
        residual split + norm -> conv (side 0) -> attention -> conv (side 1) -> residual split + norm -> conv (side 0) ->
        gated MLP -> conv (side 1); the stream ends in norm(last output + residual)."""
        cfg, m = self.cfg, self.model
        taps, gs = cfg.conv_kernel_size, cfg.conv_group_size
        G = cfg.hidden // gs
        n = b.n
        x = K.embed(b.ids, m.embed, scale=m.cfg.embed_scale).float()
        res = torch.zeros_like(x)
        for li, L in enumerate(m.layers):
            V = self.v2["layers"][li]
            res = res + x
            normed = self._norm_f32(res, L.attn_norm, cfg.rms_eps)
            dyn = V["attn_proj"].forward(normed).reshape(n, 2, taps, G)
            stage = dynconv(normed.float(), dyn[:, 0].contiguous(), V["attn_base"][:taps], gs).to(torch.bfloat16)
            o = m.attn_block(li, L, stage, b, self.kv, None)
            x = dynconv(o.float(), dyn[:, 1].contiguous(), V["attn_base"][taps:], gs)
            res = res + x
            normed = self._norm_f32(res, L.ffn_norm, cfg.rms_eps)
            dyn = V["mlp_proj"].forward(normed).reshape(n, 2, taps, G)
            stage = dynconv(normed.float(), dyn[:, 0].contiguous(), V["mlp_base"][:taps], gs).to(torch.bfloat16)
            d = m.ffn_block(li, L, stage, b, None)
            x = dynconv(d.float(), dyn[:, 1].contiguous(), V["mlp_base"][taps:], gs)
        return self._norm_f32(res + x, m.final_norm, cfg.rms_eps)

    def _select_v2(self, hidden: torch.Tensor, anchor: int) -> list[int]:
        """Candidates of block rows 1.. through the (sharded) target head, then the chained walk."""
        cfg, m, e = self.cfg, self.model, self.e
        rows = hidden[1:].contiguous()
        logits = m.lm_head.forward(rows, out_f32=True)
        ids, vals, lse = K.topk(logits, cfg.selector_top_k, e.comm.rank * m.vocab_local)
        vals = vals - lse[:, None]
        if e.comm.size > 1:                      # every rank's shard candidates, merged to the best k of the union
            ids_all, vals_all, lse_all = (e.comm.all_gather_rows(t) for t in (ids, vals + lse[:, None], lse))
            r = rows.shape[0]
            ids_all = ids_all.reshape(e.comm.size, r, -1).permute(1, 0, 2).reshape(r, -1)
            vals_all = vals_all.reshape(e.comm.size, r, -1).permute(1, 0, 2).reshape(r, -1)
            total = torch.logsumexp(lse_all.reshape(e.comm.size, r), dim=0)
            top = torch.topk(vals_all, cfg.selector_top_k, dim=1)
            ids, vals = torch.gather(ids_all, 1, top.indices).int().contiguous(), (top.values - total[:, None]).contiguous()
        gate = self.v2["gate"].forward(rows)
        anc = torch.tensor([anchor], dtype=torch.int32, device=rows.device)
        out, conf = self.walk_candidates(vals.unsqueeze(0).contiguous(), ids.unsqueeze(0).contiguous(),
                                         gate.unsqueeze(0).contiguous(), self.v2["pred"], self.v2["succ"], anc)
        self.last_conf = conf[0, 1:]
        return [int(t) for t in out[0].tolist()]

    # ---- context: keys and values of every layer from the projected taps of positions [ctx_len, upto)
    def ingest(self, slot: int, upto: int) -> int:
        cfg, m = self.cfg, self.model
        lo = max(self.ctx_len[slot], upto - cfg.tap_cap, 0)
        if upto <= lo:
            return 0
        n = upto - lo
        taps = self.ring.rows(slot, lo, upto)
        ctx = K.rmsnorm(self.fc.forward(taps), self.hidden_norm, cfg.rms_eps, 0.0)
        self._reserve(slot, upto + cfg.block_size)
        pos = torch.arange(lo, upto, dtype=torch.int32, device=ctx.device)
        sl = torch.full((n,), slot, dtype=torch.int32, device=ctx.device)
        for li, L in enumerate(m.layers):
            kpool, vpool = self.kv.layer(li)
            qkv = L.qkv.forward(ctx)
            K.rmsnorm_heads_(qkv, L.k_norm, n, m.nkv, m.hd, qkv.stride(0), cfg.rms_eps, 0.0, m.nq * m.hd)
            K.rope_store(qkv, pos, sl, self.kv.page_table, kpool, vpool, m.nq, m.nkv, m.hd, m.rot, cfg.rope_theta, False)
        self.ctx_len[slot] = upto
        return n

    def _reserve(self, slot: int, n_tokens: int) -> None:
        # pages of positions that left the sliding window (and the ring's span) are recycled before new ones are taken
        cfg = self.cfg
        self.kv.release_prefix(slot, n_tokens - max(cfg.tap_cap, cfg.sliding_window) - 2 * cfg.block_size)
        self.kv.reserve(slot, n_tokens)

    # ---- one block: returns block_size - 1 proposed tokens for positions pos + 1 ...
    def draft(self, slot: int, anchor: int, pos: int, depth: int | None = None) -> list[int]:
        cfg, m, e = self.cfg, self.model, self.e
        B = cfg.block_size
        prof = getattr(self, "profile", None)
        if prof is not None:
            import time as _t
            tp = _t.perf_counter()
        self.ingest(slot, pos)
        if prof is not None:
            prof["rounds"] += 1
            tp = self._mark("ingest_ms", tp)
        self._reserve(slot, pos + B + 1)
        ids = [anchor] + [cfg.mask_token_id] * (B - 1)
        b = BatchRows.make(ids, [pos + i for i in range(B)], [slot] * B, e.device, LOGITS_ALL, 1, nsplit=1)
        b.key_end = torch.full((B,), pos + B - 1, dtype=torch.int32, device=e.device)     # the block sees all of itself
        import time
        pol = self.sparse_policy
        sparse = pol is not None and self.sparse_head is not None and pol.use_sparse()
        t0 = time.perf_counter()
        if self.v2 is not None:
            hid = self._forward_v2(b)
            if prof is not None:
                tp = self._mark("backbone_ms", tp)
            toks = self._select_v2(hid, anchor)                      # [anchor, d1 .. d_{B-1}]
            if prof is not None:
                self._mark("select_ms", tp)
            if pol is not None:
                pol.draft_step_time(False, (time.perf_counter() - t0) * 1e3)
            nd = B - 1 if depth is None else max(0, min(B - 1, depth))
            return toks[1:1 + nd]
        if sparse:                               # the block's hidden rows through the subset of head columns only
            b.logits = LOGITS_NONE
            m.forward(b, self.kv)
            logits = self.sparse_head.logits(m.last_hidden)
        else:
            logits = m.forward(b, self.kv)
        if prof is not None:
            tp = self._mark("backbone_ms", tp)
        if logits.is_cuda:
            idx, _ = K.argmax(logits, id_offset=e.comm.rank * m.vocab_local)
            idx = e.comm.merge_argmax(idx, _) if e.comm.size > 1 else idx
        else:
            idx = logits.float().argmax(-1)
        toks = [int(t) for t in idx.tolist()]
        if prof is not None:
            self._mark("select_ms", tp)
        if pol is not None:                      # the token read above waited for the device: wall time is the step time
            pol.draft_step_time(sparse, (time.perf_counter() - t0) * 1e3)
        n = B - 1 if depth is None else max(0, min(B - 1, depth))
        return toks[1:1 + n]

    # ---- sparse drafter head: the policy counts tokens, proposes the column subset and decides per round whether to use it
    def enable_sparse_head(self, params=None, state_path=None):
        from .sparse_head_policy import SparseHeadPolicy
        assert self.e.comm.size == 1, "the sparse drafter head is built for a single rank"
        self.sparse_policy = SparseHeadPolicy(self.e.model.cfg.vocab, params)
        self.sparse_state_path = state_path
        if state_path:
            self.sparse_policy.load(state_path)
        return self.sparse_policy

    def observe_prompt(self, tokens) -> None:
        if self.sparse_policy is not None:
            self.sparse_policy.observe_prompt(tokens)

    def observe_commit(self, tokens) -> None:
        """Committed output tokens: evidence for the subset, hits / misses of the current one; rebuilds when due."""
        pol = self.sparse_policy
        if pol is None:
            return
        for t in tokens:
            pol.observe_generated(int(t))
        if pol.rebuild_due():
            cols = sorted(pol.ranked())
            m = self.model
            self.sparse_head = SparseHead.extract(m.lm_head, self.cfg.hidden, m.vocab_local,
                                                  torch.tensor(cols, dtype=torch.int32, device=self.e.device))
            pol.set_subset(cols)
        if self.sparse_state_path and pol.save_due():
            pol.save(self.sparse_state_path)

    def walk_candidates(self, unary, cands, gate, pred_cb, succ_cb, anchor):
        """Version 2 token choice: chained greedy walk over per-row candidate sets (top-k of the head) with the low-rank
        pairwise term pred_cb[prev] * gate[row] . succ_cb[cand]. Returns (tokens [bsz, rows + 1], confidence)."""
        bsz, rows, k = cands.shape
        rank = gate.shape[-1]
        if not cands.is_cuda:
            out = torch.zeros(bsz, rows + 1, dtype=torch.int32)
            conf = torch.ones(bsz, rows + 1)
            for b_ in range(bsz):
                prev = int(anchor[b_])
                out[b_, 0] = prev
                for i in range(rows):
                    ag = pred_cb[prev].float() * gate[b_, i].float()
                    sc = unary[b_, i] + succ_cb[cands[b_, i].long()].float() @ ag
                    best = int(sc.argmax())
                    prev = int(cands[b_, i, best])
                    out[b_, i + 1] = prev
                    conf[b_, i + 1] = 1.0 / float(torch.exp(sc - sc[best]).sum())
            return out, conf
        out = torch.empty(bsz, rows + 1, dtype=torch.int32, device=cands.device)
        conf = torch.empty(bsz, rows + 1, dtype=torch.float32, device=cands.device)
        call("selector_walk", "ppppppppiiii", ptr(unary), ptr(cands), ptr(gate), ptr(pred_cb), ptr(succ_cb), ptr(anchor), ptr(out),
             ptr(conf), bsz, rows, k, rank)
        return out, conf


def dynconv(x, dyn, base, group_size, out=None, accumulate=False):
    """Grouped dynamic causal convolution inside a block: out[t, c] (+)= sum_k (base[k, c] + dyn[t, k, c // gs]) * x[t - k, c]."""
    T, C = x.shape
    taps = base.shape[0]
    if out is None:
        out = torch.zeros(T, C, dtype=torch.float32, device=x.device)
        accumulate = False
    if not x.is_cuda:
        res = torch.zeros(T, C)
        w = base.float()[None] + dyn.float().repeat_interleave(group_size, dim=-1)          # [T, taps, C]
        for k in range(taps):
            res[k:] += w[k:, k] * x[:T - k].float()
        out.copy_(out + res if accumulate else res)
        return out
    call("dynconv", "ppppiiiii", ptr(x), ptr(dyn), ptr(base), ptr(out), T, C, taps, group_size, 1 if accumulate else 0)
    return out


def reduce_streams(streams, mode=0):
    """fp32 streams [m, hc, H] -> bf16 [m, H]: mode 0 the mean of the streams, mode k the stream k - 1."""
    m, hc, H = streams.shape
    if not streams.is_cuda:
        return (streams.mean(1) if mode == 0 else streams[:, mode - 1]).to(torch.bfloat16)
    out = torch.empty(m, H, dtype=torch.bfloat16, device=streams.device)
    call("reduce_streams", "ppiiii", ptr(streams), ptr(out), m, H, hc, mode)
    return out


@dataclass
class SparseHead:
    """bf16 copy of a subset of the LM head's columns, so a draft step reads a few MB instead of the whole head; its logits
    are scattered into a full-width row whose other columns hold the lowest value, so the shard argmax / top-k that follows
    is unchanged (reference: inc/engine/modules/sparse_head.h:9-33). The subset comes from running the head (any weight
    format) on blocks of identity rows."""
    cols: torch.Tensor                     # int32 [count], shard-local column ids
    w_sub: torch.Tensor                    # bf16 [count, hidden]
    width: int = 0
    counts: dict = field(default_factory=dict)

    @classmethod
    def extract(cls, head, hidden: int, width: int, cols: torch.Tensor, ident_rows: int = 128) -> "SparseHead":
        dev = cols.device
        count = cols.numel()
        w_sub = torch.zeros(count, hidden, dtype=torch.bfloat16, device=dev)
        for k0 in range(0, hidden, ident_rows):
            rows = min(ident_rows, hidden - k0)
            if cols.is_cuda:
                ident = torch.empty(rows, hidden, dtype=torch.bfloat16, device=dev)
                call("identity_rows", "piii", ptr(ident), rows, hidden, k0)
                chunk = head.forward(ident).to(torch.bfloat16).contiguous()
                call("sparse_gather", "pliipipi", ptr(chunk), chunk.stride(0), rows, k0, ptr(cols), count, ptr(w_sub), hidden)
            else:
                ident = torch.zeros(rows, hidden, dtype=torch.bfloat16)
                ident[torch.arange(rows), k0 + torch.arange(rows)] = 1
                chunk = head.forward(ident).to(torch.bfloat16)
                w_sub[:, k0:k0 + rows] = chunk[:, cols.long()].t()
        return cls(cols, w_sub, width)

    def logits(self, x: torch.Tensor) -> torch.Tensor:
        """x [rows, hidden] bf16 -> bf16 logits [rows, width]: the subset's logits in place, every other column lowest."""
        rows = x.shape[0]
        if not x.is_cuda:
            sub = (x.float() @ self.w_sub.float().t()).to(torch.bfloat16)
            out = torch.full((rows, self.width), -3.0e38, dtype=torch.bfloat16)
            out[:, self.cols.long()] = sub
            return out
        sub = K.gemm_bf16(self.w_sub, x) if rows > 16 else K.bf16_gemv_f32(self.w_sub, x).to(torch.bfloat16)
        out = torch.empty(rows, self.width, dtype=torch.bfloat16, device=x.device)
        call("sparse_scatter", "pipplii", ptr(sub), self.cols.numel(), ptr(self.cols), ptr(out), out.stride(0), self.width, rows)
        return out

    @staticmethod
    def choose_columns(token_counts: dict, budget: int, always=()) -> list[int]:
        """Policy: the ``budget`` most frequent token ids of a usage histogram, plus ids that must stay (eos, specials)."""
        keep = list(dict.fromkeys(int(t) for t in always))
        for t, _ in sorted(token_counts.items(), key=lambda kv: (-kv[1], kv[0])):
            if len(keep) >= budget:
                break
            if int(t) not in keep:
                keep.append(int(t))
        return sorted(keep)
