"""Dense GQA decoder (Llama / Qwen3 / Gemma-style block: RMSNorm -> GQA attention with RoPE -> RMSNorm ->
gated FFN), tensor-parallel over ``comm.size`` GPUs.

Counterpart of the reference's dense pipelines (simplest: src/models/gemma4.cpp:413-521; the plain
hd-128 GQA decoder: src/video/h3_text.cu). TP layout as in the reference (src/models/gemma4.cpp:42-48,
216-270): column-parallel fused qkv and gate/up, row-parallel o_proj / down_proj, residual replicated,
two fused all-reduce + residual + RMSNorm per layer, vocabulary-parallel LM head with shard argmax
merge. KV heads are replicated when there are fewer of them than ranks.
"""
from __future__ import annotations

import math
import os
from dataclasses import dataclass, asdict

import torch

from ..ops import kernels as K
from ..ops import decode_step as PS
from ..ops.streams import sandwich_add_norm
from ..ops.linear import LinearBF16, LinearNVFP4
from ..parallel.comm import LocalComm
from ..runtime.batch import BatchRows, LOGITS_ALL, LOGITS_LAST, LOGITS_NONE


@dataclass
class DenseConfig:
    n_layers: int = 4
    hidden: int = 512
    n_q: int = 8
    n_kv: int = 2
    head_dim: int = 64
    ffn: int = 1408
    vocab: int = 32000
    rope_theta: float = 1e6
    rms_eps: float = 1e-6
    norm_bias: float = 0.0        # 1.0 for "1 + w" style weights
    rot_dim: int = 0              # 0 = full head_dim
    rope_interleaved: bool = False
    qk_norm: bool = False
    act: str = "silu"             # or "gelu_tanh"
    act_limit: float = 0.0
    tie_embeddings: bool = False
    embed_scale: float = 1.0
    sliding_window: int = 0
    window_pattern: int = 0       # > 0: layers with (li + 1) % window_pattern == 0 attend to everything, the others
                                  # only to the last ``sliding_window`` keys; 0: ``sliding_window`` on every layer
    rope_theta_local: float = 0.0 # rotary base of the windowed layers (0 = rope_theta)
    sandwich_norm: bool = False   # extra RMSNorm on the output of the attention and FFN blocks before the residual add
    mrope_sections: tuple = ()    # (time, height) rotary pair counts of multimodal rope; the rest turns with the width axis
    residual: str = "plain"       # plain | gated (fp32 gated residual streams) | hc (4 fp32 hyper-connection streams)
    hc_mult: int = 4              # residual streams of the gated form
    hc_rank: int = 64             # width of the gated residual's low-rank gate
    hc_sinkhorn: int = 20         # Sinkhorn rounds of the hyper-connection mixing matrix
    attn_scale: float = 0.0       # 0 = 1/sqrt(head_dim)
    logit_softcap: float = 0.0
    quant: str = "nvfp4"          # nvfp4 | bf16
    gemm_mode: str = "w4a16"      # prefill arithmetic for nvfp4 weights
    lm_head_quant: str = "auto"   # auto: random-init NVFP4 models quantise the head like every other weight; bf16 keeps it dense
    model_type: str = "dense"

    @classmethod
    def baseline_27b(cls):
        """Dense 27B-class decoder of the NVFP4 benchmark configuration."""
        return cls(n_layers=64, hidden=5120, n_q=40, n_kv=8, head_dim=128, ffn=17408, vocab=151936,
                   rope_theta=1e6)

    @classmethod
    def tiny(cls, **kw):
        c = cls(n_layers=2, hidden=256, n_q=4, n_kv=2, head_dim=64, ffn=512, vocab=1024)
        for k, v in kw.items():
            setattr(c, k, v)
        return c

    def to_dict(self):
        return asdict(self)


# decode: act(gate) * up inside the gate/up linear's epilogue (VOLTA_FUSE_ACT=0 keeps the separate activation kernel)
FUSE_ROPE = os.environ.get("VOLTA_FUSE_ROPE", "1") != "0"   # rotary embedding + KV store in the qkv decode linear's epilogue
FUSE_GATED_ACT = os.environ.get("VOLTA_FUSE_ACT", "1") != "0"
# decode: RMSNorm fused into the linear that consumes it (VOLTA_FUSE_NORM=0 turns it off). By itself it measured neutral on
# the 27B decode (every CTA recomputes the row statistics, which costs what the removed norm kernels saved); together
# with the rotary / cache-write epilogue in the same qkv launch a layer is five launches and the step went from 4.79 to
# 4.69 ms (208.9 -> 213.3 tok/s), so it is the default for decode rows of the plain dense model on one GPU.
FUSE_PRENORM = os.environ.get("VOLTA_FUSE_NORM", "1") != "0"


def _pad_to(n: int, m: int) -> int:
    return (n + m - 1) // m * m


class DenseLayer:
    __slots__ = ("attn_norm", "qkv", "o_proj", "ffn_norm", "gate_up", "down", "q_norm", "k_norm", "post_attn_norm",
                 "post_ffn_norm", "attn_hc", "mlp_hc")


class DenseModel:
    # what a prefix-cache snapshot must hold to resume this model inside a sequence: "kv" = the paged KV rows are the whole
    # per-slot state; None = there is state outside the pool, so the scheduler must not resume from a snapshot
    prefix_resume = "kv"

    def __init__(self, cfg: DenseConfig, device, comm=None):
        self.cfg = cfg
        self.device = torch.device(device)
        self.comm = comm or LocalComm()
        tp = self.comm.size
        assert cfg.n_q % tp == 0 and cfg.ffn % tp == 0
        self.nq = cfg.n_q // tp
        self.nkv = max(1, cfg.n_kv // tp)
        self.kv_rep = max(1, tp // cfg.n_kv)   # ranks sharing one kv head
        self.ffn = cfg.ffn // tp
        self.hd = cfg.head_dim
        self.rot = cfg.rot_dim or cfg.head_dim
        self.scale = cfg.attn_scale or 1.0 / math.sqrt(cfg.head_dim)
        self.vocab_pad = _pad_to(cfg.vocab, 256 * tp)
        self.vocab_local = self.vocab_pad // tp
        self.layers: list[DenseLayer] = []
        self.embed = None
        self.final_norm = None
        self.lm_head = None
        self.attn_ws = None

    # ------------------------------------------------------------------------------------- weights
    def _make_linear(self, w: torch.Tensor, search: bool, whole=None):
        """``whole``: the full matrices this rank's shard ``w`` was cut from (a tensor or several). The NVFP4 tensor
        scale then comes from them, so every rank's shard carries exactly the values of the single-GPU quantisation and
        tensor-parallel results differ from single-GPU ones by summation order only."""
        if self.cfg.quant == "nvfp4":
            gs = None
            if whole is not None and self.comm.size > 1:
                parts = whole if isinstance(whole, (list, tuple)) else [whole]
                gmax = max(float(t.abs().max()) for t in parts)
                gs = gmax / (6.0 * 448.0) if gmax > 0 else 1.0
            return LinearNVFP4.from_dense(w, self.cfg.gemm_mode, search=search, global_scale=gs).prepare()
        if self.cfg.quant.startswith("gguf_"):
            from ..ops.linear_gguf import LinearGGUF
            from ..quant import gguf as gq
            gtype = {"gguf_q8_0": gq.GGML_Q8_0, "gguf_q4_0": gq.GGML_Q4_0, "gguf_q4_k": gq.GGML_Q4_K,
                     "gguf_q6_k": gq.GGML_Q6_K}[self.cfg.quant]
            return LinearGGUF.from_dense(w, gtype, act_q8=self.cfg.gemm_mode == "q8_act")
        return LinearBF16(w.to(torch.bfloat16))

    def init_random(self, seed: int = 1, std: float = 0.02, search: bool = False):
        """Random N(0, std) weights of the full architecture; this rank keeps its TP shard.

        Every rank draws the same full matrices from the same generator state so shards agree.
        """
        cfg, dev = self.cfg, self.device
        r, tp = self.comm.rank, self.comm.size
        gen = torch.Generator(device=dev)
        gen.manual_seed(seed)

        def rnd(n, k):
            return torch.randn(n, k, generator=gen, device=dev, dtype=torch.float32) * std

        H, hd = cfg.hidden, cfg.head_dim
        self.embed = rnd(cfg.vocab, H).to(torch.bfloat16)
        ones = torch.ones(H, device=dev, dtype=torch.bfloat16)
        nw = ones * (1.0 - cfg.norm_bias)
        for _ in range(cfg.n_layers):
            L = DenseLayer()
            wq, wk, wv = rnd(cfg.n_q * hd, H), rnd(cfg.n_kv * hd, H), rnd(cfg.n_kv * hd, H)
            kv0 = (r // self.kv_rep) * self.nkv if cfg.n_kv < tp else r * self.nkv
            wqkv = torch.cat([wq[r * self.nq * hd:(r + 1) * self.nq * hd],
                              wk[kv0 * hd:(kv0 + self.nkv) * hd], wv[kv0 * hd:(kv0 + self.nkv) * hd]], 0)
            L.qkv = self._make_linear(wqkv, search, whole=(wq, wk, wv))
            del wq, wk, wv, wqkv
            wo = rnd(H, cfg.n_q * hd)
            L.o_proj = self._make_linear(wo[:, r * self.nq * hd:(r + 1) * self.nq * hd].contiguous(), search, whole=wo)
            del wo
            wg, wu = rnd(cfg.ffn, H), rnd(cfg.ffn, H)
            L.gate_up = self._make_linear(torch.cat([wg[r * self.ffn:(r + 1) * self.ffn],
                                                     wu[r * self.ffn:(r + 1) * self.ffn]], 0), search, whole=(wg, wu))
            if isinstance(L.gate_up, LinearNVFP4) and FUSE_GATED_ACT:
                L.gate_up.interleave_gated()
            del wg, wu
            wd = rnd(H, cfg.ffn)
            L.down = self._make_linear(wd[:, r * self.ffn:(r + 1) * self.ffn].contiguous(), search, whole=wd)
            del wd
            L.attn_norm, L.ffn_norm = nw.clone(), nw.clone()
            L.post_attn_norm = L.post_ffn_norm = None
            if cfg.sandwich_norm:
                L.post_attn_norm, L.post_ffn_norm = nw.clone(), nw.clone()
            L.q_norm = L.k_norm = None
            if cfg.qk_norm:
                L.q_norm = torch.ones(hd, device=dev, dtype=torch.bfloat16) * (1.0 - cfg.norm_bias)
                L.k_norm = L.q_norm.clone()
            self.layers.append(L)
        self.final_norm = nw.clone()
        if cfg.tie_embeddings:
            full = self.embed
        else:
            full = rnd(cfg.vocab, H).to(torch.bfloat16)
        head = torch.zeros(self.vocab_local, H, device=dev, dtype=torch.bfloat16)
        lo = r * self.vocab_local
        hi = min(cfg.vocab, lo + self.vocab_local)
        if hi > lo:
            head[: hi - lo] = full[lo:hi]
        quant_head = cfg.quant.startswith("gguf_") or (cfg.quant == "nvfp4" and cfg.lm_head_quant != "bf16"
                                                          and cfg.hidden % 256 == 0)
        self.lm_head = self._make_linear(head.float(), search, whole=full) if quant_head else LinearBF16(head)
        return self

    # ------------------------------------------------------------------------------------------ MTP head
    mtp = None

    def _init_random_with_mtp(self, base_init, seed: int, std: float, search: bool):
        """Random weights plus the checkpoint-style MTP head when ``cfg.mtp_layers``: the head's block is built like one
        more decoder layer (it gets cache layer ``n_layers``), plus the projection of [norm(embedding) | norm(hidden)]
        and three norms. ``base_init`` is the family's own ``init_random``."""
        cfg = self.cfg
        if getattr(self, "_mtp_init_active", False):       # a family composed of two others: the outer call adds the head
            return base_init(seed, std, search)
        n_main = cfg.n_layers
        extra = int(getattr(cfg, "mtp_layers", 0) or 0)
        cfg.n_layers = n_main + extra
        self._mtp_init_active = True
        try:
            base_init(seed, std, search)
        finally:
            cfg.n_layers = n_main
            self._mtp_init_active = False
        if extra:
            gen = torch.Generator(device=self.device)
            gen.manual_seed(seed + 1000)
            H = cfg.hidden
            block = self.layers.pop()
            fc = torch.randn(H, 2 * H, generator=gen, device=self.device) * std
            ones = torch.ones(H, device=self.device, dtype=torch.bfloat16)
            self.mtp = {"layer": block, "fc": self._make_linear(fc, search), "norm_e": ones.clone(),
                        "norm_h": ones.clone(), "norm_out": ones.clone(), "cache_layer": n_main}
        return self

    def mtp_forward(self, next_ids: torch.Tensor, hidden: torch.Tensor, b: BatchRows, kv):
        """One MTP step for the rows of ``b``: ``next_ids[r]`` is the token that follows row r, ``hidden[r]`` the
        residual-stream state of row r. Returns (logits of this rank's vocabulary shard, MTP hidden [n, H])."""
        cfg, m = self.cfg, self.mtp
        e = K.embed(next_ids, self.embed, scale=cfg.embed_scale)
        en = K.rmsnorm(e, m["norm_e"], cfg.rms_eps, cfg.norm_bias)
        hn = K.rmsnorm(hidden, m["norm_h"], cfg.rms_eps, cfg.norm_bias)
        h = m["fc"].forward(torch.cat([en, hn], dim=1).contiguous())
        L = m["layer"]
        comm = self.comm
        x = K.rmsnorm(h, L.attn_norm, cfg.rms_eps, cfg.norm_bias)
        o = self.attn_block(m["cache_layer"], L, x, b, kv, None)
        x = comm.allreduce_add_norm(o, h, L.ffn_norm, cfg.rms_eps, cfg.norm_bias)
        d = self.ffn_block(m["cache_layer"], L, x, b, None)
        x = comm.allreduce_add_norm(d, h, m["norm_out"], cfg.rms_eps, cfg.norm_bias)
        return self.lm_head.forward(x, out_f32=True), h

    def link_prefetch(self) -> None:
        """Tell every decode linear which weights the step reads next (ops.kernels.link_prefetch): qkv -> o_proj ->
        gate / up -> down -> the next layer's qkv, the last down -> the LM head."""
        chain = []
        for L in self.layers:
            chain += [getattr(L, "qkv", None), getattr(L, "o_proj", None), getattr(L, "gate_up", None), getattr(L, "down", None)]
        chain.append(self.lm_head)
        chain = [c for c in chain if c is not None]
        for a, b in zip(chain, chain[1:]):
            K.link_prefetch(a, b)

    def weight_bytes(self) -> int:
        n = self.embed.numel() * 2 + self.lm_head.nbytes()
        for L in self.layers:
            n += L.qkv.nbytes() + L.o_proj.nbytes() + L.gate_up.nbytes() + L.down.nbytes()
        return n

    def decode_bytes_per_token(self) -> int:
        """Weight bytes every decode step must stream from HBM (embedding row excluded)."""
        n = self.lm_head.nbytes()
        for L in self.layers:
            n += L.qkv.nbytes() + L.o_proj.nbytes() + L.gate_up.nbytes() + L.down.nbytes()
        return n

    # ------------------------------------------------------------------------------------- forward
    def forward(self, b: BatchRows, kv) -> torch.Tensor | None:
        """Runs all layers for the rows of ``b``; returns fp32 logits of this rank's vocabulary shard for
        the rows selected by ``b.logits`` (None for LOGITS_NONE)."""
        cfg = self.cfg
        comm = self.comm
        if PS.supported(self, b, kv):
            # decode rows: the whole step is one persistent launch (ops/decode_step.py)
            logits, self.last_hidden, self.last_residual = PS.program_for(self, kv, b.n).run(b.ids, b.pos, b.slot)
            return logits if logits is not None else self.lm_head.forward(self.last_hidden, out_f32=True)
        if cfg.residual != "plain":
            return self._forward_streams(b, kv)
        if self._prenorm_ok(b):
            return self._forward_prenorm(b, kv)
        h = K.embed(b.ids, self.embed, scale=cfg.embed_scale)          # residual stream [n, H] bf16
        if b.embeds is not None:                                        # image tokens: rows of the vision tower
            h = torch.where(b.embed_mask[:, None], b.embeds.to(h.dtype), h)
        L0 = self.layers[0]
        x = K.rmsnorm(h, L0.attn_norm, cfg.rms_eps, cfg.norm_bias)
        # multi-GPU chunks: the residual stream is row-sharded over ranks (sequence-parallel) and the
        # row-parallel GEMMs write straight into the communicator's symmetric input region
        sp = comm.size > 1 and b.n > 16 and not cfg.sandwich_norm
        pbuf = comm.partial_buffer(b.n, cfg.hidden) if sp else None
        if sp:
            h = comm.shard_rows(h)
        for li, L in enumerate(self.layers):
            o = self.attn_block(li, L, x, b, kv, pbuf)
            x = self._add_norm(o, h, getattr(L, "post_attn_norm", None), L.ffn_norm)
            d = self.ffn_block(li, L, x, b, pbuf)
            nxt = self.layers[li + 1].attn_norm if li + 1 < len(self.layers) else self.final_norm
            x = self._add_norm(d, h, getattr(L, "post_ffn_norm", None), nxt)
            tap = getattr(self, "tap_ring", None)
            if tap is not None and li in tap.index:        # a block drafter reads this layer's output (per-slot position ring)
                tap.publish(li, comm.all_gather_rows(h)[:b.n] if sp else h, b.pos, b.slot, b.n)
            steer = getattr(self, "steer", None)
            if steer is not None and not sp and steer.first <= li < steer.first + steer.layers:
                # runtime steering edits the residual after this layer; the next layer's input is re-normalised
                steer.apply(h, b.pos, b.slot, li)
                x = K.rmsnorm(h, nxt, cfg.rms_eps, cfg.norm_bias, out=x)
        self.last_hidden, self.last_residual = x, h
        if getattr(self, "hess", None) is not None:
            self.hess.accumulate(0, 4, x)
        if b.logits == LOGITS_NONE:
            return None
        if b.logits == LOGITS_LAST:
            x = x[b.n - 1: b.n]
        logits = self.lm_head.forward(x, out_f32=True)
        if cfg.logit_softcap > 0:
            if logits.is_cuda:
                from .._lib import call, ptr
                call("softcap", "plf", ptr(logits), logits.numel(), float(cfg.logit_softcap))
            else:
                logits = cfg.logit_softcap * torch.tanh(logits / cfg.logit_softcap)
        steer = getattr(self, "steer", None)
        if steer is not None:
            # reasoning-marker penalty of steered slots (a no-op for slots whose control word holds no penalty ids)
            last = b.logits == LOGITS_LAST
            steer.penalize(logits, b.pos[b.n - 1: b.n] if last else b.pos, b.slot[b.n - 1: b.n] if last else b.slot,
                           self.comm.rank * self.vocab_local)
        return logits

    # ------------------------------------------------------------------------------------- multi-stream residuals
    def init_stream_weights(self, seed: int = 9, std: float = 0.02):
        """Weights of the multi-stream residual forms (``cfg.residual``): per sublayer a gated-residual mixer
        (norm, low-rank gate, inject) or a hyper-connection mixer (24 x 4H projection, base, scale); replicated on
        every rank. Call after the layers exist."""
        from ..ops.streams import GatedResidualWeights
        cfg, dev = self.cfg, self.device
        H, hc, rank = cfg.hidden, (cfg.hc_mult if cfg.residual == "gated" else 4), cfg.hc_rank
        g = torch.Generator(device=dev).manual_seed(seed)

        def rnd(*shape, s=std):
            return torch.randn(*shape, generator=g, device=dev) * s

        def mixer(inject=True):
            if cfg.residual == "gated":
                return GatedResidualWeights(norm=rnd(hc, H, s=0.05).to(torch.bfloat16), down=rnd(rank, hc * H).to(torch.bfloat16),
                                            up=rnd(hc * H, rank, s=0.2).to(torch.bfloat16),
                                            inject=rnd(hc, hc * H).to(torch.bfloat16) if inject else None)
            return (rnd(24, 4 * H, s=0.02).contiguous(), rnd(24, s=0.5).contiguous(),
                    torch.tensor([0.5, 0.5, 0.5], device=dev))
        for L in self.layers:
            L.attn_hc, L.mlp_hc = mixer(), mixer()
        self.final_hc = mixer(inject=False)
        return self

    def _forward_streams(self, b: BatchRows, kv):
        """Forward with fp32 residual streams [n, hc, H]. gated: every sublayer reads mean_s(gate_s * norm(stream_s)) and
        writes stream_s += post_s * y, the update fused with the all-reduce and the next mixer's norm. hc: every sublayer
        reads sum_h pre_h * stream_h (normalised) and writes stream_h = post_h * y + sum_g comb[g][h] * stream_g."""
        from ..ops import streams as S
        cfg, comm = self.cfg, self.comm
        h0 = K.embed(b.ids, self.embed, scale=cfg.embed_scale)
        gated = cfg.residual == "gated"
        xs = S.init_streams(h0, cfg.hc_mult if gated else 4)
        eps = cfg.rms_eps
        if gated:
            normed = S.gr_norm(xs, self.layers[0].attn_hc.norm, eps)
            for li, L in enumerate(self.layers):
                mixed, post = S.gr_mix_prenormed(normed, L.attn_hc)
                o = self.attn_block(li, L, mixed, b, kv, None)
                normed = S.gated_stream_update(o, xs, post, L.mlp_hc.norm, eps, comm=comm)
                mixed, post = S.gr_mix_prenormed(normed, L.mlp_hc)
                d = self.ffn_block(li, L, mixed, b, None)
                nxt = self.layers[li + 1].attn_hc if li + 1 < len(self.layers) else self.final_hc
                normed = S.gated_stream_update(d, xs, post, nxt.norm, eps, comm=comm)
            hid, _ = S.gr_mix_prenormed(normed, self.final_hc)
            x = K.rmsnorm(hid, self.final_norm, eps, cfg.norm_bias)
            pre = hid
        else:
            for li, L in enumerate(self.layers):
                fn, base, scale = L.attn_hc
                mix = S.hc_collapse(xs, fn, base, scale, cfg.hc_sinkhorn, norm_w=L.attn_norm, norm_eps=eps, norm_bias=cfg.norm_bias)
                o = self.attn_block(li, L, mix.collapsed, b, kv, None)
                S.hc_update(o, xs, mix.post, mix.comb, comm=comm)
                fn, base, scale = L.mlp_hc
                mix = S.hc_collapse(xs, fn, base, scale, cfg.hc_sinkhorn, norm_w=L.ffn_norm, norm_eps=eps, norm_bias=cfg.norm_bias)
                d = self.ffn_block(li, L, mix.collapsed, b, None)
                S.hc_update(d, xs, mix.post, mix.comb, comm=comm)
            pre = S.head_mean(xs)
            x = K.rmsnorm(pre, self.final_norm, eps, cfg.norm_bias)
        # (last_residual: the state in front of the final norm, what an MTP head reads; the streams themselves stay fp32)
        self.last_hidden, self.last_residual, self.last_streams = x, pre.to(x.dtype), xs
        if b.logits == LOGITS_NONE:
            return None
        if b.logits == LOGITS_LAST:
            x = x[b.n - 1: b.n]
        return self.lm_head.forward(x, out_f32=True)

    def _prenorm_ok(self, b: BatchRows) -> bool:
        """Decode steps of the plain dense model on one GPU: the two RMSNorms of a layer are computed inside the
        linears that consume them (no norm kernels on the critical path)."""
        if b.n > 4 or not FUSE_PRENORM or type(self) is not DenseModel or self.comm.size != 1 or not self.embed.is_cuda:
            return False
        if getattr(b, "pos3", None) is not None or getattr(b, "tree", None) is not None or getattr(b, "embeds", None) is not None:
            return False                  # rows with their own rotary positions / a tree mask / injected embeddings
        ok = getattr(self, "_prenorm_cached", None)
        if ok is None:
            cfg = self.cfg
            ok = not cfg.sandwich_norm and cfg.hidden % 256 == 0 and all(      # (the norm prologue reads K in 256-wide steps)
                isinstance(L.qkv, LinearNVFP4) and L.qkv.tc_ready() and isinstance(L.gate_up, LinearNVFP4)
                and L.gate_up.tc_ready() and getattr(L.gate_up, "gated", False) for L in self.layers)
            self._prenorm_cached = ok
        return ok and getattr(self, "steer", None) is None

    def _forward_prenorm(self, b: BatchRows, kv):
        cfg = self.cfg
        act = 0 if cfg.act == "silu" else 1
        h = K.embed(b.ids, self.embed, scale=cfg.embed_scale)
        h2 = torch.empty_like(h)
        delta = None
        mark = getattr(self, "_trace_mark", None)          # (push, pop) of utils.trace.enable_layer_trace
        for li, L in enumerate(self.layers):
            if mark is not None:
                if li:
                    mark[1]()
                mark[0](f"L{li}")
            kpool, vpool = kv.layer(li)
            # norm in front and rotation + cache write behind, all inside the projection's launch where the layer allows
            fuse_rope = (FUSE_ROPE and not cfg.qk_norm and not cfg.rope_interleaved and b.pos3 is None
                         and L.qkv.rope_ready(b.n, self.hd) and K.kv_format_of(kpool) < 2)
            rope = (b.pos, b.slot, kv.page_table, kpool, vpool, self.nq, self.nkv, self.rot, self.layer_theta(li)) if fuse_rope else None
            qkv = L.qkv.forward_prenorm(h, delta, L.attn_norm, cfg.rms_eps, cfg.norm_bias, h2 if delta is not None else None,
                                        rope=rope)
            if delta is not None:
                h, h2 = h2, h
            if not fuse_rope:
                if cfg.qk_norm:
                    stride = qkv.stride(0)
                    K.rmsnorm_heads_(qkv, L.q_norm, b.n, self.nq, self.hd, stride, cfg.rms_eps, cfg.norm_bias, 0)
                    K.rmsnorm_heads_(qkv, L.k_norm, b.n, self.nkv, self.hd, stride, cfg.rms_eps, cfg.norm_bias, self.nq * self.hd)
                K.rope_store(qkv, b.pos, b.slot, kv.page_table, kpool, vpool, self.nq, self.nkv, self.hd, self.rot,
                             self.layer_theta(li), cfg.rope_interleaved)
            att = K.attention(qkv, b.pos, b.slot, kv.page_table, kpool, vpool, self.nq, self.nkv, self.hd, self.scale,
                              window=self.layer_window(li), key_end=b.key_end, tiles=b.tiles,
                              nsplit=1 if b.tiles is not None else b.nsplit, ws=self.attn_ws)
            o = L.o_proj.forward(att)
            a = L.gate_up.forward_prenorm(h, o, L.ffn_norm, cfg.rms_eps, cfg.norm_bias, h2, act=act, limit=cfg.act_limit)
            h, h2 = h2, h
            delta = L.down.forward(a)
        if mark is not None:
            mark[1]()
        x = K.rmsnorm(delta, self.final_norm, cfg.rms_eps, cfg.norm_bias, residual=h)
        self.last_hidden, self.last_residual = x, h
        if b.logits == LOGITS_NONE:
            return None
        if b.logits == LOGITS_LAST:
            x = x[b.n - 1: b.n]
        logits = self.lm_head.forward(x, out_f32=True)
        if cfg.logit_softcap > 0:
            from .._lib import call, ptr
            call("softcap", "plf", ptr(logits), logits.numel(), float(cfg.logit_softcap))
        return logits

    def _add_norm(self, part, h, post_norm, next_norm):
        """h += sum over ranks of ``part`` (through ``post_norm`` first for sandwich-norm models); returns the next
        block's input RMSNorm(h)."""
        cfg, comm = self.cfg, self.comm
        if post_norm is None:
            return comm.allreduce_add_norm(part, h, next_norm, cfg.rms_eps, cfg.norm_bias)
        # decode rows: one launch (the all-reduce kernel applies both norms); otherwise all-reduce, then the same epilogue
        return sandwich_add_norm(part, h, post_norm, next_norm, cfg.rms_eps, cfg.norm_bias, 1.0, comm=comm)

    def layer_window(self, li: int) -> int:
        cfg = self.cfg
        if cfg.window_pattern > 0 and (li + 1) % cfg.window_pattern == 0:
            return 0
        return cfg.sliding_window

    def layer_theta(self, li: int) -> float:
        cfg = self.cfg
        return cfg.rope_theta_local if cfg.rope_theta_local > 0 and self.layer_window(li) > 0 else cfg.rope_theta

    def attn_block(self, li, L, x, b: BatchRows, kv, pbuf):
        """Attention sub-layer: returns this rank's partial of the o_proj output [n, H]."""
        cfg = self.cfg
        kpool, vpool = kv.layer(li)
        hs = getattr(self, "hess", None)
        if hs is not None and b.n >= hs.min_rows:      # calibration capture: the unfused path below, with its taps
            return self._attn_block_capture(li, L, x, b, kv, pbuf, hs)
        if (FUSE_ROPE and x.is_cuda and not cfg.qk_norm and not cfg.rope_interleaved and b.pos3 is None and b.tree is None
                and isinstance(L.qkv, LinearNVFP4) and L.qkv.rope_ready(b.n, self.hd) and K.kv_format_of(kpool) < 2):
            # decode rows: rotation and cache write happen in the projection's epilogue (one launch less per layer)
            qkv = L.qkv.forward_rope(x, b.pos, b.slot, kv.page_table, kpool, vpool, self.nq, self.nkv, self.rot,
                                     self.layer_theta(li))
            att = K.attention(qkv, b.pos, b.slot, kv.page_table, kpool, vpool, self.nq, self.nkv, self.hd,
                              self.scale, window=self.layer_window(li), key_end=b.key_end, tiles=b.tiles,
                              nsplit=1 if b.tiles is not None else b.nsplit, ws=self.attn_ws)
            return self._row_parallel(L.o_proj, att, pbuf)
        qkv = L.qkv.forward(x)
        if cfg.qk_norm:
            stride = qkv.stride(0)
            K.rmsnorm_heads_(qkv, L.q_norm, b.n, self.nq, self.hd, stride, cfg.rms_eps, cfg.norm_bias, 0)
            K.rmsnorm_heads_(qkv, L.k_norm, b.n, self.nkv, self.hd, stride, cfg.rms_eps, cfg.norm_bias,
                             self.nq * self.hd)
        # rows with rotary positions of their own (b.pos stays the cache position): the multimodal sections of the model,
        # or, for a model without them (tree verification: position = depth), one section that covers every pair
        mrope = None
        if b.pos3 is not None:
            mrope = (b.pos3, tuple(cfg.mrope_sections) if cfg.mrope_sections else (self.rot // 2, 0))
        K.rope_store(qkv, b.pos, b.slot, kv.page_table, kpool, vpool, self.nq, self.nkv, self.hd, self.rot,
                     self.layer_theta(li), cfg.rope_interleaved, mrope=mrope)
        att = K.attention(qkv, b.pos, b.slot, kv.page_table, kpool, vpool, self.nq, self.nkv, self.hd,
                          self.scale, window=self.layer_window(li), key_end=b.key_end, tiles=b.tiles,
                          nsplit=1 if b.tiles is not None else b.nsplit, ws=self.attn_ws, tree=b.tree)
        return self._row_parallel(L.o_proj, att, pbuf)

    def _attn_block_capture(self, li, L, x, b, kv, pbuf, hs):
        cfg = self.cfg
        kpool, vpool = kv.layer(li)
        hs.accumulate(li, 0, x)
        qkv = L.qkv.forward(x)
        if cfg.qk_norm:
            stride = qkv.stride(0)
            K.rmsnorm_heads_(qkv, L.q_norm, b.n, self.nq, self.hd, stride, cfg.rms_eps, cfg.norm_bias, 0)
            K.rmsnorm_heads_(qkv, L.k_norm, b.n, self.nkv, self.hd, stride, cfg.rms_eps, cfg.norm_bias,
                             self.nq * self.hd)
        mrope = (b.pos3, tuple(cfg.mrope_sections)) if b.pos3 is not None and cfg.mrope_sections else None
        K.rope_store(qkv, b.pos, b.slot, kv.page_table, kpool, vpool, self.nq, self.nkv, self.hd, self.rot,
                     self.layer_theta(li), cfg.rope_interleaved, mrope=mrope)
        att = K.attention(qkv, b.pos, b.slot, kv.page_table, kpool, vpool, self.nq, self.nkv, self.hd,
                          self.scale, window=self.layer_window(li), key_end=b.key_end, tiles=b.tiles,
                          nsplit=1 if b.tiles is not None else b.nsplit, ws=self.attn_ws)
        hs.accumulate(li, 2, att)
        return self._row_parallel(L.o_proj, att, pbuf)

    def enable_hessians(self, layer_range=None, min_rows: int = 17):
        """Calibration capture: x^T x sums at the inputs of the four projections of every layer in ``layer_range``
        and of the head (site numbering of src/models/qwen3_5.cpp:678-906 in the reference: 0 qkv input, 1 gate / up
        input, 2 o_proj input, 3 down input, layer 0 site 4 the head's input). Returns the set; ``dump`` writes it."""
        from ..ops.hessian import HessianSet
        cfg = self.cfg
        hs = HessianSet(cfg.n_layers, 5, min_rows, layer_range)
        for li, L in enumerate(self.layers):
            hs.add(li, 0, cfg.hidden, self.device)
            hs.add(li, 1, cfg.hidden, self.device)
            hs.add(li, 2, self.nq * self.hd, self.device)
            hs.add(li, 3, self.ffn, self.device)
        hs.add(0, 4, cfg.hidden, self.device)
        self.hess = hs
        return hs

    def _row_parallel(self, lin, x, pbuf):
        """Row-parallel projection whose output goes into the layer's all-reduce: on decode rows the NVFP4 decode linear
        sends its result to the peers from its own epilogue (communicators that offer ``push_target``)."""
        if pbuf is None and self.comm.size > 1 and hasattr(self.comm, "push_target") and isinstance(lin, LinearNVFP4):
            return lin.forward(x, push=self.comm)
        return lin.forward(x, out=pbuf)

    def ffn_block(self, li, L, x, b: BatchRows, pbuf):
        """Feed-forward sub-layer: returns this rank's partial of the down projection [n, H]."""
        cfg = self.cfg
        act = 0 if cfg.act == "silu" else 1
        hs = getattr(self, "hess", None)
        if hs is not None:
            hs.accumulate(li, 1, x)
        if getattr(L.gate_up, "gated", False):        # gate / up rows interleaved: activation fused into the decode linear
            a = L.gate_up.forward_gated(x, act, cfg.act_limit)
        else:
            a = K.gated_act(L.gate_up.forward(x), self.ffn, act, cfg.act_limit)
        if hs is not None:
            hs.accumulate(li, 3, a)
        return self._row_parallel(L.down, a, pbuf)

    def ensure_workspace(self, max_rows: int, max_splits: int):
        if self.device.type == "cuda" and (self.attn_ws is None or self.attn_ws.max_splits < max_splits):
            self.attn_ws = K.AttnWorkspace(max_rows, self.nq, self.hd, max_splits, self.device)
