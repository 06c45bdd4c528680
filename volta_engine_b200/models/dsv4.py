"""DeepSeek-V4.1-style decoder: sliding-window + compressed sparse attention and routed experts on four
hyper-connection streams, with Engram n-gram lookups at chosen layers.

Per layer (src/models/deepseek_v41.cpp:2177-2259 in the reference; the arithmetic is DeepSeek's public inference model):
  * the sublayer input is ``sum_h pre[h] * stream[h]`` with the pre-mix of the sublayer BEFORE (lagged; the first one is
    (1, 0, 0, 0)), RMS-normalised; the output goes back as ``stream[h] = post[h] * y + sum_g comb[g][h] * stream[g]``;
  * attention: low-rank queries (wq_a -> norm -> wq_b, 512 per head), one 512-wide KV vector per token shared by all heads
    as key and value, kept in a position ring of the last 128 tokens (MXFP8); layers with a compress ratio also attend to
    at most 512 entries of a compressed KV cache (NVFP4) that a SOURCE layer fills (ratio 1: every token; ratio r: a
    softmax-gated pool of r tokens) and that an INDEX-SOURCE layer's indexer picks per query (32 heads x 128 dims on an
    FP4 grid, optional two-level candidate blocks); the layers in between reuse both. A per-head sink joins the softmax
    denominator; the output is inverse-rotated, put on the FP8 grid and projected by a grouped low-rank pair
    (wo_a per 8 heads -> 1024, wo_b -> hidden);
  * FFN: routed experts chosen by sqrt(softplus) scores + bias, one shared expert;
  * Engram: at its layers the streams receive a gated value looked up by hashed n-grams of the token ids.
All projections of the normalised input (query down-projection, KV, compressor, compressor gate, indexer head weights)
are one stacked linear, as are the two projections of the normalised query latent, so a layer's attention is a handful
of launches. Heads, output groups and experts are split over tensor-parallel ranks; the caches are replicated.
"""
from __future__ import annotations

from dataclasses import dataclass, field

import torch

from ..ops import dsv4 as V
from ..ops import kernels as K
from ..ops import streams as S
from ..ops.linear import LinearBF16
from ..runtime.batch import LOGITS_ALL, LOGITS_LAST, LOGITS_NONE, BatchRows
from .moe import MoEConfig, MoELayer, MoEModel


@dataclass
class DSV4Config(MoEConfig):
    q_lora_rank: int = 1280
    o_groups: int = 8
    o_lora_rank: int = 1024
    compress_ratios: tuple = ()           # per layer: 0 window only, r > 0 compressed attention at ratio r
    kv_sources: tuple = ()                # layers that compress KV (and own the index keys)
    index_sources: tuple = ()             # layers that run an indexer
    candidate_source: int = -1
    candidate_blocks: int = 2048
    candidate_block: int = 8
    compress_rope_theta: float = 160000.0
    rope_original_len: int = 65536
    rope_factor: float = 16.0
    beta_fast: float = 32.0
    beta_slow: float = 1.0
    engram_layers: tuple = ()
    engram_dim: int = 2048                # width of a looked-up row (heads x head dim)
    engram_rows: int = 1 << 16            # rows of the (synthetic) table
    engram_ngram: int = 4
    hc_eps: float = 1e-6
    model_type: str = "deepseek_v41"

    @classmethod
    def baseline_dsv41(cls):
        """DeepSeek-V4.1-Flash shape (40 layers, hidden 5120, 64 heads, 384 experts top-6 + shared, 4 streams)."""
        return cls(n_layers=40, hidden=5120, n_q=64, n_kv=1, head_dim=512, ffn=0, vocab=129280, n_experts=384, top_k=6,
                   expert_ffn=2304, shared_ffn=2304, router="sqrtsoftplus", router_scale=1.5, act_limit=10.0, rms_eps=1e-20,
                   rope_theta=10000.0, residual="hc", hc_sinkhorn=20,
                   compress_ratios=(0, 0) + (2,) * 18 + (1,) * 20, kv_sources=(2, 8, 14, 20),
                   index_sources=(2, 8, 14, 20, 24, 28, 32, 36), candidate_source=20, engram_layers=(1, 14))

    @classmethod
    def tiny_dsv4(cls, **kw):
        c = cls(n_layers=5, hidden=256, n_q=16, n_kv=1, head_dim=512, ffn=0, vocab=1024, n_experts=8, top_k=2, expert_ffn=128,
                shared_ffn=128, router="sqrtsoftplus", router_scale=1.5, act_limit=10.0, rms_eps=1e-6, residual="hc",
                hc_sinkhorn=20, q_lora_rank=128, o_groups=2, o_lora_rank=128, compress_ratios=(0, 2, 2, 1, 1), kv_sources=(1, 3),
                index_sources=(1, 3, 4), candidate_source=3, candidate_blocks=16, rope_original_len=256, engram_layers=(1,),
                engram_dim=64, engram_rows=512)
        for k, v in kw.items():
            setattr(c, k, v)
        return c


class DSV4Layer(MoELayer):
    __slots__ = ("x_proj", "q_proj", "qa_norm", "kv_norm", "sink", "wo_a", "wo_b", "c_norm", "idx_wk", "idx_knorm", "ratio", "kv_src",
                 "is_kv_source", "is_index_source", "cols", "engram")


class DSV4Model(MoEModel):
    prefix_resume = None      # recurrent / ring / indexer state lives outside the paged KV pool
    layer_cls = DSV4Layer

    def __init__(self, cfg: DSV4Config, device, comm=None):
        assert cfg.head_dim == V.HD and len(cfg.compress_ratios) == cfg.n_layers
        assert cfg.n_q % V.GROUP_HEADS == 0 and cfg.n_q // V.GROUP_HEADS == cfg.o_groups
        cfg.residual = "hc"
        super().__init__(cfg, device, comm)
        tp = self.comm.size
        assert cfg.o_groups % tp == 0, "output groups are split over the ranks"
        self.heads = cfg.n_q // tp
        self.groups = cfg.o_groups // tp
        self.nq, self.nkv, self.hd = self.heads, 1, 64           # the paged cache is not used: a token's footprint there is minimal
        self.sources = [(s, cfg.compress_ratios[s]) for s in cfg.kv_sources]
        self.state: V.DSV4State | None = None
        self.rope_plain = self.rope_comp = None
        self.attn_ws2 = None
        self.engram_table = None
        self.prefill_end = -1            # total length of the prompt being prefilled (set_prefill_end), -1 outside a prefill
        self.trunc_layer, self.trunc_keep = -1, 0
        self.set_prefill_truncate(-1)
        self.tap_ring = None             # a block drafter reads the stream mean at the entry of its target layers
        self.block_keys = None           # (key_end [rows], window): a drafter block whose rows all see the whole block

    kv_layers = 1

    # ------------------------------------------------------------------------------------------ weights
    def _init_attention(self, L, rnd, search):
        cfg = self.cfg
        li = len(self.layers)
        r, H, hl, gl = self.comm.rank, cfg.hidden, self.heads, self.groups
        dev, bf = self.device, torch.bfloat16
        L.ratio = cfg.compress_ratios[li]
        L.is_kv_source = li in cfg.kv_sources
        L.is_index_source = li in cfg.index_sources
        L.kv_src = max((i for i, s in enumerate(cfg.kv_sources) if s <= li), default=-1) if L.ratio > 0 else -1
        ql = cfg.q_lora_rank
        # one stacked projection of the normalised input: [wq_a | wkv | c_wkv | c_wgate | idx_wproj], every part drawn whole
        parts = [("q", rnd(ql, H)), ("kv", rnd(V.HD, H))]
        if L.is_kv_source:
            parts.append(("ckv", rnd(V.HD, H)))
            if L.ratio > 1:
                parts.append(("csc", rnd(V.HD, H)))
        if L.is_index_source:
            parts.append(("wi", rnd(V.IDX_HEADS, H) * 4))
        L.cols, at = {}, 0
        for name, w in parts:
            L.cols[name] = (at, at + w.shape[0])
            at += w.shape[0]
        wx = torch.zeros((at + 127) // 128 * 128, H, device=dev)
        wx[:at] = torch.cat([w for _, w in parts], 0)
        L.x_proj = self._make_linear(wx, search)
        ones = torch.ones
        L.qa_norm = ones(ql, device=dev, dtype=bf)
        L.kv_norm = ones(V.HD, device=dev, dtype=bf)
        wqb_all = [rnd(cfg.n_q * V.HD, ql)]
        wqb = wqb_all[0][r * hl * V.HD:(r + 1) * hl * V.HD]
        if L.is_index_source:                                        # the indexer's queries ride on the same launch
            L.cols["qi"] = (hl * V.HD, hl * V.HD + V.IDX_HEADS * V.IDX_DIM)
            wqb_all.append(rnd(V.IDX_HEADS * V.IDX_DIM, ql) * 4)
            wqb = torch.cat([wqb, wqb_all[1]], 0)
        L.q_proj = self._make_linear(wqb.contiguous(), search, whole=wqb_all)
        L.sink = (torch.randn(cfg.n_q, generator=torch.Generator().manual_seed(li + 7)) * 0.5)[r * hl:(r + 1) * hl].to(dev).contiguous()
        woa = rnd(cfg.o_groups * cfg.o_lora_rank, V.GROUP_HEADS * V.HD).reshape(cfg.o_groups, cfg.o_lora_rank, -1)
        L.wo_a = woa[r * gl:(r + 1) * gl].to(bf).contiguous()          # [groups, o_lora, 8 * 512]: block diagonal over the groups
        wob = rnd(H, cfg.o_groups * cfg.o_lora_rank)
        L.wo_b = self._make_linear(wob[:, r * gl * cfg.o_lora_rank:(r + 1) * gl * cfg.o_lora_rank].contiguous(), search, whole=wob)
        L.c_norm = L.idx_wk = L.idx_knorm = None
        if L.is_kv_source:
            L.c_norm = ones(V.HD, device=dev, dtype=bf)
            L.idx_wk = LinearBF16((rnd(V.IDX_DIM, V.HD) * 4).to(bf))
            L.idx_knorm = ones(V.IDX_DIM, device=dev, dtype=bf)
        L.qkv = L.o_proj = None
        L.engram = None
        if li in cfg.engram_layers:
            L.engram = {"wkv": LinearBF16(rnd(5 * H, cfg.engram_dim).to(bf)), "w": torch.ones(4, H, device=dev),
                        "index": cfg.engram_layers.index(li)}

    def _attn_bytes(self, L) -> int:
        return L.x_proj.nbytes() + L.q_proj.nbytes() + L.wo_b.nbytes() + L.wo_a.numel() * 2

    def init_random(self, seed: int = 5, std: float = 0.02, search: bool = False):
        super().init_random(seed, std, search)
        self.init_stream_weights(seed + 9, std)
        cfg = self.cfg
        if cfg.engram_layers:
            g = torch.Generator().manual_seed(seed + 77)
            self.engram_table = (torch.randn(len(cfg.engram_layers), cfg.engram_rows, cfg.engram_dim, generator=g) * 0.5) \
                .to(torch.bfloat16).to(self.device)
        return self

    # ------------------------------------------------------------------------------------------ state
    def _state(self, kv) -> V.DSV4State:
        if self.state is None:
            cfg, dev = self.cfg, self.device
            max_seq = kv.max_pages * 64
            self.state = V.DSV4State(kv.max_slots, cfg.n_layers, self.sources, max_seq, dev)
            self.rope_plain = V.rope_table(max_seq, cfg.rope_theta, device=dev)
            self.rope_comp = V.rope_table(max_seq, cfg.compress_rope_theta, cfg.rope_original_len, cfg.rope_factor, cfg.beta_fast,
                                          cfg.beta_slow, device=dev)
            if dev.type == "cuda":
                self.attn_ws2 = (torch.empty(16 * self.heads * 8 * V.HD, dtype=torch.float32, device=dev),
                                 torch.empty(16 * self.heads * 8, dtype=torch.float32, device=dev))
        return self.state

    def ensure_workspace(self, max_rows: int, max_splits: int):
        return None

    # ------------------------------------------------------------------------------------------ prefill truncation
    def set_prefill_truncate(self, keep: int) -> None:
        """From the first layer that reads a ratio-1 source's compressed KV on, nothing a later row needs comes from an
        earlier row except that source's KV / index keys and each layer's window. So those layers run only the last ``keep``
        rows of a prefill (``keep`` < 0: the exact count, one window further back per layer; 0: off); the earlier rows stop
        at that layer after writing its window entries and source caches. Needs every KV source at or before that layer
        and every engram layer before it. Reference: src/models/deepseek_v41.cpp:576-594, 2060-2071."""
        cfg = self.cfg
        self.trunc_layer, self.trunc_keep = -1, 0
        if keep == 0:
            return
        b = next((l for l, r in enumerate(cfg.compress_ratios) if r == 1), -1)
        ok = b > 0 and b in cfg.kv_sources and all(s <= b for s in cfg.kv_sources) and all(e < b for e in cfg.engram_layers)
        if not ok:
            return
        exact = (cfg.n_layers - b - 1) * (V.WINDOW - 1) + V.WINDOW
        self.trunc_layer, self.trunc_keep = b, exact if keep < 0 else max(keep, V.WINDOW)

    def set_prefill_end(self, end: int) -> None:
        self.prefill_end = end

    def _trunc_rows(self, b: BatchRows) -> int:
        """How many leading rows of this chunk stop at the truncation layer."""
        if self.trunc_layer < 0 or self.prefill_end < 0 or b.n <= 16 or b.logits == LOGITS_ALL or not b.host_pos:
            return 0
        keep_pos = self.prefill_end - self.trunc_keep
        k = 0
        while k < b.n and b.host_pos[k] < keep_pos:
            k += 1
        return k

    def _attention_kv(self, li, L, x, b: BatchRows, kv):
        """What later rows read of this layer from rows that go no further: its window entries and, as a KV source, its
        compressed KV and index keys."""
        cfg, st, eps = self.cfg, self._state(kv), self.cfg.rms_eps
        xp = L.x_proj.forward(x)
        c = L.cols
        kv_n = K.rmsnorm(xp[:, c["kv"][0]:c["kv"][1]], L.kv_norm, eps, cfg.norm_bias)
        rope = self.rope_comp if L.ratio > 0 else self.rope_plain
        V.window_store(st, li, kv_n, rope, b.slot, b.pos)
        if L.is_kv_source:
            csc = xp[:, c["csc"][0]:c["csc"][1]] if L.ratio > 1 else None
            latent = V.compress(st, L.kv_src, xp[:, c["ckv"][0]:c["ckv"][1]], csc, L.c_norm, rope, b.slot, b.pos, eps)
            V.index_key_store(st, L.kv_src, L.idx_wk.forward(latent), L.idx_knorm, rope, b.slot, b.pos, eps)

    # ------------------------------------------------------------------------------------------ forward
    def forward(self, b: BatchRows, kv) -> torch.Tensor | None:
        cfg, comm = self.cfg, self.comm
        assert b.n <= V.RING - V.WINDOW, "a chunk must fit the position rings beside the window"
        st = self._state(kv)
        eps = cfg.rms_eps
        if cfg.engram_layers:
            if getattr(self, "_history", None) is None:
                # token history per slot (one spare row takes the writes of padding rows, slot < 0)
                self._history = torch.zeros(kv.max_slots + 1, kv.max_pages * 64, dtype=torch.int32, device=self.device)
            eids = V.engram_ids(b.ids, b.slot, b.pos, self._history, len(cfg.engram_layers), cfg.engram_rows, cfg.engram_ngram).long()
        xs = S.init_streams(K.embed(b.ids, self.embed, scale=cfg.embed_scale), 4)
        pre = torch.zeros(b.n, 4, dtype=torch.float32, device=self.device)
        pre[:, 0] = 1.0
        k0 = self._trunc_rows(b)
        self.win_floor = 0
        for li, L in enumerate(self.layers):
            if li == self.trunc_layer and k0 > 0:
                # prefill truncation: the rows before the kept tail stop here, after writing what the kept rows read of this layer
                fn, base, scale = L.attn_hc
                head = BatchRows(b.ids[:k0], b.pos[:k0], b.slot[:k0], k0, LOGITS_NONE)
                mixh = S.hc_collapse(xs[:k0].contiguous(), fn, base, scale, 1, cfg.hc_eps, rms_eps=eps, norm_w=L.attn_norm,
                                     norm_eps=eps, norm_bias=cfg.norm_bias, pre_in=pre[:k0].contiguous())
                self._attention_kv(li, L, mixh.collapsed, head, kv)
                if k0 == b.n:
                    return None                                    # nothing of this chunk runs further (it wants no logits)
                xs, pre = xs[k0:].contiguous(), pre[k0:].contiguous()
                b = BatchRows(b.ids[k0:], b.pos[k0:], b.slot[k0:], b.n - k0, b.logits, None, b.nsplit, None,
                              b.host_slots[k0:], b.host_pos[k0:])
                if st.sel is not None and st.sel[0].shape[0] > b.n:
                    st.sel = (st.sel[0][k0:].contiguous(), st.sel[1][k0:].contiguous())
                st.cand = None if st.cand is None else (st.cand[k0:] if isinstance(st.cand, list) else st.cand[k0:].contiguous())
                self.win_floor = self.prefill_end - self.trunc_keep
            if L.engram is not None:
                rows = self.engram_table[L.engram["index"]][eids[:, L.engram["index"]]]
                V.engram_gate(xs, L.engram["wkv"].forward(rows).contiguous(), L.engram["w"], None, eps)
            self._cur_floor = self.win_floor if li > self.trunc_layer >= 0 else 0
            if self.tap_ring is not None and li in self.tap_ring.index:
                self.tap_ring.publish(li, S.head_mean(xs), b.pos, b.slot, b.n)
            fn, base, scale = L.attn_hc
            mix = S.hc_collapse(xs, fn, base, scale, cfg.hc_sinkhorn, cfg.hc_eps, rms_eps=eps, norm_w=L.attn_norm, norm_eps=eps,
                                norm_bias=cfg.norm_bias, pre_in=pre)
            o = self.attn_block(li, L, mix.collapsed, b, kv, None)
            S.hc_update(o, xs, mix.post, mix.comb, comm=comm)
            fn, base, scale = L.mlp_hc
            mix2 = S.hc_collapse(xs, fn, base, scale, cfg.hc_sinkhorn, cfg.hc_eps, rms_eps=eps, norm_w=L.ffn_norm, norm_eps=eps,
                                 norm_bias=cfg.norm_bias, pre_in=mix.pre)
            d = self.ffn_block(li, L, mix2.collapsed, b, None)
            S.hc_update(d, xs, mix2.post, mix2.comb, comm=comm)
            pre = mix2.pre
        fn, base, scale = self.layers[-1].mlp_hc           # only the collapse with the last pre-mix and the final norm are used
        x = S.hc_collapse(xs, fn, base, scale, 1, cfg.hc_eps, rms_eps=eps, norm_w=self.final_norm, norm_eps=eps,
                          norm_bias=cfg.norm_bias, pre_in=pre).collapsed
        self.last_hidden, self.last_residual, self.last_streams, self.last_pre = x, None, xs, pre
        if b.logits == LOGITS_NONE:
            return None
        if b.logits == LOGITS_LAST:
            x = x[b.n - 1: b.n]
        return self.lm_head.forward(x, out_f32=True)

    def attn_block(self, li, L, x, b: BatchRows, kv, pbuf):
        cfg = self.cfg
        st = self._state(kv)
        eps = cfg.rms_eps
        xp = L.x_proj.forward(x)
        c = L.cols
        qr_n = K.rmsnorm(xp[:, c["q"][0]:c["q"][1]], L.qa_norm, eps, cfg.norm_bias)
        qq = L.q_proj.forward(qr_n)
        q = qq[:, : self.heads * V.HD]
        rope = self.rope_comp if L.ratio > 0 else self.rope_plain
        # the KV projection's norm runs inside the ring write
        V.window_store(st, li, xp[:, c["kv"][0]:c["kv"][1]], rope, b.slot, b.pos, norm=(L.kv_norm, eps, cfg.norm_bias))
        src = L.kv_src
        if L.is_kv_source:
            ckv = xp[:, c["ckv"][0]:c["ckv"][1]]
            csc = xp[:, c["csc"][0]:c["csc"][1]] if L.ratio > 1 else None
            latent = V.compress(st, src, ckv, csc, L.c_norm, rope, b.slot, b.pos, eps)
            V.index_key_store(st, src, L.idx_wk.forward(latent), L.idx_knorm, rope, b.slot, b.pos, eps)
        if L.is_index_source:
            qi = V.index_queries(qq[:, c["qi"][0]:c["qi"][1]], rope, b.pos)
            wi = xp[:, c["wi"][0]:c["wi"][1]].float().contiguous()
            mode = 0 if cfg.candidate_source < 0 else 1 if li == cfg.candidate_source else 2 if li > cfg.candidate_source else 0
            V.indexer(st, src, qi, wi, b.slot, b.pos, mode, cfg.candidate_blocks, cfg.candidate_block)
        nsplit = 1 if b.n > 16 else max(1, min(8, b.nsplit))
        ke, win = self.block_keys if self.block_keys is not None else (None, V.WINDOW)
        o = V.attend(st, li, src, q, L.sink, rope, b.slot, b.pos, self.heads, self.attn_ws2, nsplit=nsplit, key_end=ke, window=win,
                     win_floor=getattr(self, "_cur_floor", 0))
        return L.wo_b.forward(V.grouped_out_proj(o, L.wo_a), out=pbuf)
