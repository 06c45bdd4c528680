"""Sparse mixture-of-experts decoder: GQA attention (tensor-parallel) + routed experts (expert-parallel) with an
optional always-on shared expert.

Counterpart of the reference's MoE pipelines (Flash-Next: src/models/qwen4_exp.cpp, GLM: src/models/glm5_next.cpp
:1772-1775,2092-2098,2220-2247). Parallel layout as there: hidden state replicated after the attention
all-reduce, every rank routes all rows with a replicated router, runs only its own experts
``[e0, e0 + E/size)`` and contributes a partial row; the tensor-parallel all-reduce (fused with residual add and
RMSNorm) is the combine. Decode rows use route-indexed NVFP4 mat-vecs with the activation fused into the first
projection; prefill chunks sort routes by expert and run the grouped tcgen05 GEMM.
"""
from __future__ import annotations

import contextlib

from dataclasses import dataclass

import torch

from .._lib import call, ptr
from ..ops import kernels as K
from ..ops.linear import LinearBF16
from ..quant import nvfp4 as qn
from ..runtime.batch import BatchRows
from .dense import DenseConfig, DenseLayer, DenseModel


@dataclass
class MoEConfig(DenseConfig):
    n_experts: int = 8
    top_k: int = 2
    expert_ffn: int = 256
    shared_ffn: int = 0            # 0 = no shared expert
    router: str = "softmax"        # softmax | sigmoid
    router_scale: float = 1.0
    n_group: int = 1
    topk_group: int = 1
    first_dense_layers: int = 0    # leading layers with a dense FFN of width cfg.ffn
    router_bias_zipf: float = 0.0  # synthetic skew: expert bias ~ Zipf(s)
    shared_gate: bool = False      # shared expert output scaled by sigmoid(x . w): one more row of the router weight
    mtp_layers: int = 0            # 1: the checkpoint's own multi-token-prediction head (one more decoder block)
    # storage of the routed experts: "nvfp4" (quantised from random dense weights), "nvfp4_random" (codes drawn directly),
    # "exl3_<bits>" (trellis codes drawn directly), or GGUF blocks "gguf_<type>" / "gguf_<gate-up type>+<down type>"
    # (e.g. "gguf_iq2_xxs+q4_k": random block bytes drawn on the device)
    expert_quant: str = "nvfp4"
    model_type: str = "moe"

    @classmethod
    def baseline_moe(cls):
        """512-expert top-10 MoE of the EXL3/EP benchmark configuration (weights held as NVFP4 here)."""
        return cls(n_layers=48, hidden=2048, n_q=16, n_kv=2, head_dim=256, ffn=0, vocab=151936, n_experts=512,
                   top_k=10, expert_ffn=512, shared_ffn=512, router="softmax")

    @classmethod
    def tiny_moe(cls, **kw):
        c = cls(n_layers=2, hidden=256, n_q=4, n_kv=2, head_dim=64, ffn=512, vocab=1024, n_experts=8, top_k=2,
                expert_ffn=128, shared_ffn=128)
        for k, v in kw.items():
            setattr(c, k, v)
        return c


class ExpertBank:
    """Stacked NVFP4 weights of this rank's experts: gate_up [E, 2I, H] and down [E, H, I]."""

    def __init__(self, gu_p, gu_s, gu_g, dn_p, dn_s, dn_g, e0: int, inter: int, hidden: int):
        self.gu_p, self.gu_s, self.gu_g = gu_p, gu_s, gu_g
        self.dn_p, self.dn_s, self.dn_g = dn_p, dn_s, dn_g
        self.e0, self.e_local, self.inter, self.hidden = e0, gu_p.shape[0], inter, hidden
        self.gu_sf = self.dn_sf = None
        if gu_p.is_cuda and (2 * inter) % 128 == 0 and hidden % 128 == 0 and inter % 128 == 0:
            E = self.e_local
            self.gu_sf = qn.scales_blocked_k128(gu_s.reshape(E * 2 * inter, -1))
            self.dn_sf = qn.scales_blocked_k128(dn_s.reshape(E * hidden, -1))

    def nbytes(self):
        return sum(t.numel() * t.element_size() for t in (self.gu_p, self.gu_s, self.dn_p, self.dn_s))

    @classmethod
    def random(cls, E: int, inter: int, hidden: int, e0: int, seed: int, device, std: float = 0.02):
        """Synthetic bank drawn directly in the storage format (uniform E2M1 codes, E4M3 block scales in [0.5, 1.875],
        one tensor scale that puts the weights at about ``std``): a benchmark-sized model initialises in seconds instead
        of quantising tens of thousands of dense matrices."""
        g = torch.Generator(device=device).manual_seed(seed)

        def part(n, k):
            p = torch.randint(0, 256, (E, n, k // 2), dtype=torch.uint8, generator=g, device=device)
            s = torch.randint(0x30, 0x40, (E, n, k // 16), dtype=torch.uint8, generator=g, device=device)
            return p, s
        gp, gs = part(2 * inter, hidden)
        dp, ds = part(hidden, inter)
        scale = torch.full((E,), std / 3.0, dtype=torch.float32, device=device)     # E2M1 codes have an rms of about 3
        return cls(gp, gs, scale, dp, ds, scale.clone(), e0, inter, hidden)

    def dequant(self, which: str, e: int) -> torch.Tensor:
        p, s, g = (self.gu_p, self.gu_s, self.gu_g) if which == "gu" else (self.dn_p, self.dn_s, self.dn_g)
        return qn.dequantize_nvfp4(p[e], s[e], float(g[e]))


def route_reference(logits: torch.Tensor, cfg: MoEConfig, bias: torch.Tensor | None):
    """fp32 statement of the router (see csrc/cuda/moe.cu): -> (ids [rows, k] int32, weights [rows, k] fp32)."""
    lf = logits.float()
    s = torch.sigmoid(lf) if cfg.router == "sigmoid" else torch.nn.functional.softplus(lf).sqrt() if cfg.router == "sqrtsoftplus" else lf
    sel = s + (bias.float() if bias is not None else 0.0)
    rows, E = sel.shape
    if cfg.n_group > 1:
        g = sel.reshape(rows, cfg.n_group, E // cfg.n_group)
        gscore = g.topk(2, dim=-1).values.sum(-1)
        keep = torch.zeros_like(gscore, dtype=torch.bool)
        order = torch.sort(gscore, dim=-1, descending=True, stable=True).indices[:, : cfg.topk_group]
        keep.scatter_(1, order, True)
        sel = torch.where(keep[:, :, None].expand_as(g), g, torch.full_like(g, float("-inf"))).reshape(rows, E)
    order = torch.sort(sel, dim=-1, descending=True, stable=True).indices[:, : cfg.top_k]
    chosen = s.gather(1, order)
    if cfg.router in ("sigmoid", "sqrtsoftplus"):
        w = chosen * cfg.router_scale / (chosen.sum(-1, keepdim=True) + 1e-9)
    else:
        w = torch.softmax(chosen, dim=-1) * cfg.router_scale
    return order.int(), w


class MoELayer(DenseLayer):
    __slots__ = ("router", "router_bias", "bank", "shared_gu", "shared_dn", "dense_ffn", "shared_gated", "tier", "cpu")


class MoEModel(DenseModel):
    layer_cls = MoELayer

    def __init__(self, cfg: MoEConfig, device, comm=None):
        if cfg.ffn == 0:
            cfg.ffn = max(cfg.shared_ffn, 128) * (comm.size if comm else 1)
        super().__init__(cfg, device, comm)
        ep = self.comm.size
        assert cfg.n_experts % ep == 0
        self.e_local = cfg.n_experts // ep
        self.e0 = self.comm.rank * self.e_local
        self.heat = None

    def init_random(self, seed: int = 2, std: float = 0.02, search: bool = False):
        cfg, dev = self.cfg, self.device
        r, tp = self.comm.rank, self.comm.size
        gen = torch.Generator(device=dev)
        gen.manual_seed(seed)

        def rnd(n, k):
            return torch.randn(n, k, generator=gen, device=dev, dtype=torch.float32) * std

        H, hd, I = cfg.hidden, cfg.head_dim, cfg.expert_ffn
        self.embed = rnd(cfg.vocab, H).to(torch.bfloat16)
        nw = torch.ones(H, device=dev, dtype=torch.bfloat16) * (1.0 - cfg.norm_bias)
        self.heat = torch.zeros(cfg.n_layers, cfg.n_experts, dtype=torch.float32, device=dev)
        for li in range(cfg.n_layers):
            L = self.layer_cls()
            self._init_attention(L, rnd, search)
            L.attn_norm, L.ffn_norm = nw.clone(), nw.clone()
            L.q_norm = L.k_norm = None
            L.gate_up = L.down = None
            L.dense_ffn = li < cfg.first_dense_layers
            if L.dense_ffn:
                wg, wu, wd = rnd(cfg.ffn, H), rnd(cfg.ffn, H), rnd(H, cfg.ffn)
                f = cfg.ffn // tp
                L.gate_up = self._make_linear(torch.cat([wg[r * f:(r + 1) * f], wu[r * f:(r + 1) * f]], 0), search, whole=(wg, wu))
                L.down = self._make_linear(wd[:, r * f:(r + 1) * f].contiguous(), search, whole=wd)
                self.layers.append(L)
                continue
            L.shared_gated = bool(cfg.shared_gate and cfg.shared_ffn)
            L.router = LinearBF16(rnd(cfg.n_experts + (1 if L.shared_gated else 0), H).to(torch.bfloat16))
            L.router_bias = None
            if cfg.router_bias_zipf > 0:
                ranks = torch.arange(1, cfg.n_experts + 1, device=dev, dtype=torch.float32)
                perm = torch.randperm(cfg.n_experts, generator=gen, device=dev)
                L.router_bias = (torch.log(ranks.pow(-cfg.router_bias_zipf)))[perm].contiguous()
            if cfg.expert_quant.startswith("gguf_"):
                from ..ops.moe_gguf import GGUFExpertBank, parse_expert_quant
                gt, dt = parse_expert_quant(cfg.expert_quant)
                L.bank = GGUFExpertBank.random(self.e_local, I, H, gt, dt, self.e0, seed=seed * 100003 + li * 4099 + self.e0,
                                               device=dev, amp=std)
            elif cfg.expert_quant.startswith("exl3_"):
                from ..ops.moe_exl3 import EXL3ExpertBank
                L.bank = EXL3ExpertBank.random(self.e_local, I, H, int(cfg.expert_quant[5:]), self.e0,
                                               seed=seed * 100003 + li * 4099 + self.e0, device=dev, std=std)
            elif cfg.expert_quant == "nvfp4_random":
                L.bank = ExpertBank.random(self.e_local, I, H, self.e0, seed * 100003 + li * 4099 + self.e0, dev, std)
            else:
                gp, gs, gg, dp, ds, dg = [], [], [], [], [], []
                for e in range(cfg.n_experts):       # every rank draws all experts so shards agree; keeps its own
                    wgu, wdn = rnd(2 * I, H), rnd(H, I)
                    if self.e0 <= e < self.e0 + self.e_local:
                        p, s, g = qn.quantize_nvfp4(wgu, search=search)
                        gp.append(p), gs.append(s), gg.append(g)
                        p, s, g = qn.quantize_nvfp4(wdn, search=search)
                        dp.append(p), ds.append(s), dg.append(g)
                L.bank = ExpertBank(torch.stack(gp), torch.stack(gs), torch.tensor(gg, device=dev, dtype=torch.float32),
                                    torch.stack(dp), torch.stack(ds), torch.tensor(dg, device=dev, dtype=torch.float32),
                                    self.e0, I, H)
            L.shared_gu = L.shared_dn = None
            if cfg.shared_ffn:
                S = cfg.shared_ffn
                wg, wu, wd = rnd(S, H), rnd(S, H), rnd(H, S)
                f = S // tp if S % tp == 0 and (S // tp) % 128 == 0 else S      # a slice must keep whole 128-wide scale blocks
                self._shared_sliced = f != S
                lo, hi = (r * f, (r + 1) * f) if f != S else (0, S)
                L.shared_gu = self._make_linear(torch.cat([wg[lo:hi], wu[lo:hi]], 0), search, whole=(wg, wu))
                L.shared_dn = self._make_linear(wd[:, lo:hi].contiguous(), search, whole=wd)
            self.layers.append(L)
        self.final_norm = nw.clone()
        full = self.embed if cfg.tie_embeddings else rnd(cfg.vocab, H).to(torch.bfloat16)
        head = torch.zeros(self.vocab_local, H, device=dev, dtype=torch.bfloat16)
        lo = r * self.vocab_local
        hi = min(cfg.vocab, lo + self.vocab_local)
        if hi > lo:
            head[: hi - lo] = full[lo:hi]
        self.lm_head = LinearBF16(head)
        return self

    def _init_attention(self, L, rnd, search):
        """GQA attention weights of one layer (overridden by the latent-attention model)."""
        cfg = self.cfg
        r, tp, H, hd = self.comm.rank, self.comm.size, cfg.hidden, cfg.head_dim
        wq, wk, wv = rnd(cfg.n_q * hd, H), rnd(cfg.n_kv * hd, H), rnd(cfg.n_kv * hd, H)
        kv0 = (r // self.kv_rep) * self.nkv if cfg.n_kv < tp else r * self.nkv
        L.qkv = self._make_linear(torch.cat([wq[r * self.nq * hd:(r + 1) * self.nq * hd],
                                             wk[kv0 * hd:(kv0 + self.nkv) * hd],
                                             wv[kv0 * hd:(kv0 + self.nkv) * hd]], 0), search, whole=(wq, wk, wv))
        wo = rnd(H, cfg.n_q * hd)
        L.o_proj = self._make_linear(wo[:, r * self.nq * hd:(r + 1) * self.nq * hd].contiguous(), search, whole=wo)

    def _attn_bytes(self, L) -> int:
        return L.qkv.nbytes() + L.o_proj.nbytes()

    def decode_bytes_per_token(self) -> int:
        n = self.lm_head.nbytes()
        cfg = self.cfg
        for L in self.layers:
            n += self._attn_bytes(L)
            if L.dense_ffn:
                n += L.gate_up.nbytes() + L.down.nbytes()
            else:
                n += L.router.nbytes() + L.bank.nbytes() * cfg.top_k // max(1, cfg.n_experts)
                if L.shared_gu is not None:
                    n += L.shared_gu.nbytes() + L.shared_dn.nbytes()
        return n

    # ------------------------------------------------------------------------------------------ FFN
    def ffn_block(self, li, L, x, b: BatchRows, pbuf):
        cfg = self.cfg
        if L.dense_ffn:
            return super().ffn_block(li, L, x, b, pbuf)
        act = 0 if cfg.act == "silu" else 1
        rows, H = x.shape
        cpu = getattr(L, "cpu", None) if x.is_cuda else None
        if cpu is not None and rows > 16:
            # host-owned experts answer through a 16-row mailbox: larger chunks go through it piece by piece
            y = pbuf if pbuf is not None else torch.empty(rows, H, dtype=x.dtype, device=x.device)
            for r0 in range(0, rows, 16):
                y[r0:r0 + 16] = self.ffn_block(li, L, x[r0:r0 + 16], b, None)
            return y
        logits = L.router.forward(x, out_f32=True)
        shared = None
        side = None
        if L.shared_gu is not None:
            if getattr(self, "side_streams", False) and x.is_cuda and rows <= 16:
                # the shared expert does not depend on the routing: it runs on a side stream beside the router and the
                # routed experts and joins before the combine (inside a graph capture this becomes a forked branch). Decode
                # rows only: larger chunks are compute-bound and their kernels share workspaces
                side = getattr(self, "_side", None)
                if side is None:
                    side = self._side = torch.cuda.Stream(device=x.device)
                main = torch.cuda.current_stream(x.device)
                side.wait_stream(main)
                x.record_stream(side)
            with (torch.cuda.stream(side) if side is not None else contextlib.nullcontext()):
                sgu = L.shared_gu.forward(x)
                sa = K.gated_act(sgu, sgu.shape[1] // 2, act, cfg.act_limit)
                shared = L.shared_dn.forward(sa)
            if not getattr(self, "_shared_sliced", False) and self.comm.size > 1 and self.comm.rank != 0:
                shared = None            # replicated shared expert: only one rank contributes it to the sum
        if not x.is_cuda:
            if getattr(L, "shared_gated", False) and shared is not None:
                shared = (shared.float() * torch.sigmoid(logits[:, cfg.n_experts:cfg.n_experts + 1])).to(x.dtype)
            return self._ffn_reference(L, x, logits[:, :cfg.n_experts], shared, li)
        bank = L.bank
        k = cfg.top_k
        ids = torch.empty(rows, k, dtype=torch.int32, device=x.device)
        w = torch.empty(rows, k, dtype=torch.float32, device=x.device)
        call("router_select", "pliiiipfiippp", ptr(logits), logits.stride(0), rows, cfg.n_experts, k,
             {"sigmoid": 1, "sqrtsoftplus": 2}.get(cfg.router, 0), ptr(L.router_bias), float(cfg.router_scale), cfg.n_group,
             cfg.topk_group, ptr(ids), ptr(w), self.heat[li].data_ptr() if self.heat is not None else 0)
        routes = rows * k
        rec = getattr(self, "route_recorder", None)
        if rec is not None:
            rec.record(li, x, ids, w)
        if cpu is not None:
            cpu.post(x, ids, w, bank.e0, bank.e_local)          # routes of host-owned experts leave the table (id -1)
        y = pbuf if pbuf is not None else torch.empty(rows, H, dtype=x.dtype, device=x.device)
        I = bank.inter
        tier = getattr(L, "tier", None)
        if hasattr(bank, "routes"):
            # experts held as GGUF blocks: fused dequant mat-vec per route, or per-slab dequantise + grouped GEMM
            d, inv = bank.routes(x, ids, act, cfg.act_limit), None
        elif tier is not None or rows <= 16 or bank.gu_sf is None:
            # tiered residency: per-expert base pointers (device slot or pinned host memory) instead of the stacked bank
            stager = getattr(self, "expert_stager", None)
            staged = None
            if tier is not None and stager is not None and stager.wants(tier, rows) and not torch.cuda.is_current_stream_capturing():
                staged = stager.acquire(tier)                   # cold experts of this layer are in device scratch by now
            tabs = staged if staged is not None else ((tier.tab_gu, tier.tab_dn) if tier is not None else None)
            gu = (tabs[0].data_ptr(), 0) if tier is not None else (ptr(bank.gu_p), ptr(bank.gu_s))
            dn = (tabs[1].data_ptr(), 0) if tier is not None else (ptr(bank.dn_p), ptr(bank.dn_s))
            a = torch.empty(routes, I, dtype=x.dtype, device=x.device)
            call("nvfp4_moe_gemv", "ppppiiplipliiiiif", gu[0], gu[1], ptr(bank.gu_g), ptr(ids), bank.e0,
                 bank.e_local, ptr(x), x.stride(0), k, ptr(a), a.stride(0), routes, 2 * I, H, 1, act, float(cfg.act_limit))
            d = torch.empty(routes, H, dtype=x.dtype, device=x.device)
            call("nvfp4_moe_gemv", "ppppiiplipliiiiif", dn[0], dn[1], ptr(bank.dn_g), ptr(ids), bank.e0,
                 bank.e_local, ptr(a), a.stride(0), 1, ptr(d), d.stride(0), routes, H, I, 0, act, 0.0)
            if staged is not None:
                stager.release(tier)
            inv = None
        else:
            d, inv = self._grouped(bank, x, ids, routes, k, act)
        gate = logits[:, cfg.n_experts:] if getattr(L, "shared_gated", False) else None     # extra router column
        if side is not None:
            main.wait_stream(side)
            if shared is not None:
                shared.record_stream(main)
        call("moe_combine", "plpppiiplplpliii", ptr(d), d.stride(0), ptr(w), ptr(ids), ptr(inv), bank.e0, bank.e_local,
             ptr(shared), shared.stride(0) if shared is not None else 0,
             gate.data_ptr() if gate is not None else 0, logits.stride(0) if gate is not None else 0,
             ptr(y), y.stride(0), rows, k, H)
        if cpu is not None:
            cpu.wait_add(y)                                     # + the host experts' weighted sum, once it is published
        return y

    def _grouped(self, bank, x, ids, routes, k, act):
        """Prefill path: sort local routes by expert, grouped tcgen05 GEMMs, results stay in sorted order."""
        cfg = self.cfg
        H, I = bank.hidden, bank.inter
        bn = 64 if routes // max(1, bank.e_local) < 96 else 128
        max_tiles = routes // bn + bank.e_local + 1
        dev = x.device
        inv = torch.empty(routes, dtype=torch.int32, device=dev)
        srt = torch.empty(routes, dtype=torch.int32, device=dev)
        tab = torch.empty(max_tiles, 4, dtype=torch.int32, device=dev)
        totals = torch.zeros(2, dtype=torch.int32, device=dev)
        call("moe_sort", "piiiipppip", ptr(ids), routes, bank.e0, bank.e_local, bn, ptr(inv), ptr(srt), ptr(tab),
             max_tiles, ptr(totals))
        xs = torch.empty(routes, H, dtype=x.dtype, device=dev)
        call("moe_gather", "plppiplii", ptr(x), x.stride(0), ptr(srt), ptr(totals), k, ptr(xs), xs.stride(0), H, routes)
        gu = torch.empty(routes, 2 * I, dtype=x.dtype, device=dev)
        st = K.status_word(dev)
        call("gemm_grouped_w4a16", "pppplpliiiiipip", ptr(bank.gu_p), ptr(bank.gu_sf), ptr(bank.gu_g), ptr(xs), xs.stride(0),
             ptr(gu), gu.stride(0), routes, bank.e_local, 2 * I, H, bn, ptr(tab), max_tiles, ptr(st))
        a = K.gated_act(gu, I, act, cfg.act_limit)
        d = torch.empty(routes, H, dtype=x.dtype, device=dev)
        call("gemm_grouped_w4a16", "pppplpliiiiipip", ptr(bank.dn_p), ptr(bank.dn_sf), ptr(bank.dn_g), ptr(a), a.stride(0),
             ptr(d), d.stride(0), routes, bank.e_local, H, I, bn, ptr(tab), max_tiles, ptr(st))
        return d, inv

    def _ffn_reference(self, L, x, logits, shared, li=-1):
        """fp32 oracle of the routed FFN (same rounding points as the kernels: bf16 between the stages)."""
        cfg, bank = self.cfg, L.bank
        ids, w = route_reference(logits, cfg, L.router_bias)
        rec = getattr(self, "route_recorder", None)
        if rec is not None and li >= 0:
            rec.record(li, x, ids, w)
        rows, H = x.shape
        y = torch.zeros(rows, H, dtype=torch.float32)
        for t in range(rows):
            for kk in range(cfg.top_k):
                e = int(ids[t, kk]) - bank.e0
                if e < 0 or e >= bank.e_local:
                    continue
                gu = (x[t:t + 1].float() @ bank.dequant("gu", e).t()).to(x.dtype)
                a = K.gated_act(gu, bank.inter, 0 if cfg.act == "silu" else 1, cfg.act_limit)
                d = (a.float() @ bank.dequant("dn", e).t()).to(x.dtype)
                y[t] += float(w[t, kk]) * d[0].float()
        if shared is not None:
            y += shared.float()
        return y.to(x.dtype)

    def enable_expert_tier(self, hot_slots: int, decay: float = 0.9, margin: float = 1.25, margin_add: float = 0.0,
                           history_pct: int = 0, resident_bias: float = 0.0):
        """Keep only ``hot_slots`` experts of every MoE layer in device memory; the rest stay in pinned host memory and are
        read in place by the mat-vec kernel. Returns the tiers (``ExpertTier.rebalance`` moves experts between the two).
        ``history_pct``: largest share of a swap decision taken from the long-run counts; ``resident_bias``: added to the
        router's selection score of resident experts (near ties then avoid host-memory experts)."""
        from ..runtime.expert_tier import ExpertTier
        tiers = []
        for li, L in enumerate(self.layers):
            if getattr(L, "bank", None) is not None and not L.dense_ffn:
                L.tier = ExpertTier(L.bank, hot_slots, decay, margin, margin_add)
                L.tier.history_pct = int(history_pct)
                if resident_bias:
                    if getattr(L, "router_bias", None) is None:
                        L.router_bias = torch.zeros(self.cfg.n_experts, dtype=torch.float32, device=self.device)
                    L.tier.set_route_bias(L.router_bias, self.e0, resident_bias)
                tiers.append((li, L.tier))
        self.tiers = tiers
        self.expert_stager = None
        return tiers

    def enable_expert_staging(self, min_rows: int = 17):
        """Prefill chunks of at least ``min_rows`` rows read a tiered layer's cold experts from device scratch that a copy
        stream fills a layer ahead (two buffers of one layer's cold experts). Returns the stager, or None when the scratch
        does not fit in free device memory."""
        from ..runtime.expert_tier import ExpertStager
        tiers = getattr(self, "tiers", None)
        if not tiers or all(t.hot_slots >= t.E for _, t in tiers):
            return None
        if self.device.type == "cuda":
            free, _ = torch.cuda.mem_get_info(self.device)
            if ExpertStager.scratch_bytes(tiers) + (256 << 20) > free:
                return None
        self.expert_stager = ExpertStager(tiers, min_rows)
        return self.expert_stager

    def rebalance_experts(self, max_swaps: int = 2) -> int:
        """Fold the routing histogram of every tiered layer into its decayed heat and swap experts whose heat says so."""
        n = 0
        for li, tier in getattr(self, "tiers", []):
            n += tier.rebalance(self.heat[li, self.e0:self.e0 + self.e_local], max_swaps)
        return n

    def expert_heat(self) -> dict:
        cfg = self.cfg
        tot = self.heat.flatten().tolist() if self.heat is not None else []
        return {"ranks": self.comm.size, "layers": cfg.n_layers, "experts": cfg.n_experts, "total": tot, "recent": tot}
