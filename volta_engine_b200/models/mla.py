"""MLA (multi-head latent attention) MoE decoder with an optional MTP draft head.

Attention: low-rank query (q_lora) and a latent KV cache row ``[c_kv (512) | k_rope (64)]`` per token shared by all
heads, decoupled RoPE key; decode / verify rows run the absorbed form (csrc/cuda/mla.cu), prefill chunks expand
K / V per head for the chunk's context and reuse the dense paged-attention kernel (head_dim padded to 256).
FFN: routed experts + shared expert from :mod:`.moe`, optional leading dense layers.
MTP head (reference form, src/models/qwen3_5.cpp:929-1006): ``h' = fc([norm_e(embed(tok_{i+1})) | norm_h(hidden_i)])``
-> one decoder layer with its own cache layer -> norm -> shared LM head.

The reference has the rope-free GLM variant of MLA (inc/engine/modules/mla.h:13-49) in src/models/glm5_next.cpp;
heads are split over tensor-parallel ranks, the latent cache is replicated on every rank.
"""
from __future__ import annotations

import math
from dataclasses import dataclass

import torch

from .._lib import call, ptr
from ..ops import kernels as K
from ..ops.linear import LinearBF16
from ..runtime.batch import BatchRows
from .moe import MoEConfig, MoELayer, MoEModel

LAT, ROPE, LAT_ROW = 512, 64, 576


@dataclass
class MLAConfig(MoEConfig):
    q_lora_rank: int = 768
    kv_lora_rank: int = 512
    qk_nope: int = 128
    qk_rope: int = 64
    v_head_dim: int = 128
    mtp_layers: int = 0
    dsa: bool = False              # sparse attention: a pooled-key indexer picks the 2048 tokens a decode row attends to
    model_type: str = "mla_moe"

    @classmethod
    def baseline_mla_mtp(cls):
        """MLA MoE + MTP benchmark configuration (46 layers, hidden 4096, 32 heads, 128 experts top-8 + shared)."""
        return cls(n_layers=46, hidden=4096, n_q=32, n_kv=1, head_dim=576, ffn=0, vocab=151552, n_experts=128, top_k=8,
                   expert_ffn=1408, shared_ffn=1408, router="sigmoid", router_scale=2.5, q_lora_rank=768, mtp_layers=1)

    @classmethod
    def baseline_dsv3(cls):
        """DeepSeek-V3-shaped configuration (61 layers, 3 dense, 256 experts sigmoid top-8, 8 groups / top-4)."""
        return cls(n_layers=61, hidden=7168, n_q=128, n_kv=1, head_dim=576, ffn=18432, vocab=129280, n_experts=256,
                   top_k=8, expert_ffn=2048, shared_ffn=2048, router="sigmoid", router_scale=2.5, n_group=8, topk_group=4,
                   first_dense_layers=3, q_lora_rank=1536)

    @classmethod
    def tiny_mla(cls, **kw):
        c = cls(n_layers=2, hidden=256, n_q=4, n_kv=1, head_dim=576, ffn=512, vocab=1024, n_experts=8, top_k=2,
                expert_ffn=128, shared_ffn=128, q_lora_rank=128, mtp_layers=1)
        for k, v in kw.items():
            setattr(c, k, v)
        return c


class MLALayer(MoELayer):
    __slots__ = ("qkv_a", "q_a_norm", "kv_a_norm", "q_b", "w_uk", "w_uv", "w_ukv", "dsa")


class MLAModel(MoEModel):
    @property
    def prefix_resume(self):
        """The sparse-attention indexer keeps pooled keys outside the paged pool."""
        return None if self.cfg.dsa else "kv"

    layer_cls = MLALayer

    def __init__(self, cfg: MLAConfig, device, comm=None):
        assert cfg.kv_lora_rank == LAT and cfg.qk_rope == ROPE, "latent kernels are built for kv_lora 512 + rope 64"
        super().__init__(cfg, device, comm)
        self.heads = cfg.n_q // self.comm.size
        self.nq, self.nkv, self.hd = self.heads, 1, LAT_ROW      # cache geometry: one latent "kv head" of 576
        self.qd = cfg.qk_nope + cfg.qk_rope
        self.scale = cfg.attn_scale or 1.0 / math.sqrt(self.qd)
        self.a_rows = (cfg.q_lora_rank + LAT + ROPE + 127) // 128 * 128
        self.mtp = None
        self.mla_ws = None
        self.dsa_states: dict = {}
        self.dsa_scratch = None

    # ------------------------------------------------------------------------------------------ weights
    def _init_attention(self, L, rnd, search):
        cfg = self.cfg
        r, H, hl = self.comm.rank, cfg.hidden, self.heads
        wa = torch.zeros(self.a_rows, H, device=self.device)
        wa[: cfg.q_lora_rank + LAT + ROPE] = rnd(cfg.q_lora_rank + LAT + ROPE, H)
        L.qkv_a = self._make_linear(wa, search)
        ones = torch.ones
        L.q_a_norm = ones(cfg.q_lora_rank, device=self.device, dtype=torch.bfloat16)
        L.kv_a_norm = ones(LAT, device=self.device, dtype=torch.bfloat16)
        wqb = rnd(cfg.n_q * self.qd, cfg.q_lora_rank)
        L.q_b = self._make_linear(wqb[r * hl * self.qd:(r + 1) * hl * self.qd].contiguous(), search, whole=wqb)
        wkvb = rnd(cfg.n_q * (cfg.qk_nope + cfg.v_head_dim), LAT).reshape(cfg.n_q, cfg.qk_nope + cfg.v_head_dim, LAT)
        mine = wkvb[r * hl:(r + 1) * hl]
        # W_uk as [head, nope, 512] for q absorption; W_uv [head, v, 512]; stacked [head*(nope+v), 512] for prefill
        L.w_uk = mine[:, : cfg.qk_nope].contiguous().to(torch.bfloat16)
        L.w_uv = mine[:, cfg.qk_nope:].contiguous().to(torch.bfloat16)
        L.w_ukv = LinearBF16(mine.reshape(hl * (cfg.qk_nope + cfg.v_head_dim), LAT).to(torch.bfloat16))
        wo = rnd(H, cfg.n_q * cfg.v_head_dim)
        L.o_proj = self._make_linear(wo[:, r * hl * cfg.v_head_dim:(r + 1) * hl * cfg.v_head_dim].contiguous(), search, whole=wo)
        L.qkv = None
        L.dsa = None
        if cfg.dsa:                                  # indexer weights (replicated on every rank: the list must agree)
            from ..ops import dsa as D
            bf = torch.bfloat16
            L.dsa = D.DSAWeights(proj=LinearBF16(rnd(D.PROJ, H).to(bf) * 8), q_proj=LinearBF16(rnd(D.HEADS * D.DIM, cfg.q_lora_rank).to(bf) * 8),
                                 ln_w=torch.ones(D.DIM, device=self.device, dtype=bf), ln_b=torch.zeros(D.DIM, device=self.device, dtype=bf),
                                 ape=(rnd(D.POOL, D.DIM) * 10).to(bf))

    def _attn_bytes(self, L) -> int:
        return L.qkv_a.nbytes() + L.q_b.nbytes() + L.o_proj.nbytes() + (L.w_uk.numel() + L.w_uv.numel()) * 2

    def init_random(self, seed: int = 3, std: float = 0.02, search: bool = False):
        return self._init_random_with_mtp(super().init_random, seed, std, search)

    def ensure_workspace(self, max_rows: int, max_splits: int):
        if self.device.type == "cuda" and self.mla_ws is None:
            self.mla_ws = (torch.empty(max_rows * self.heads * max_splits * LAT, dtype=torch.float32, device=self.device),
                           torch.empty(max_rows * self.heads * max_splits, dtype=torch.float32, device=self.device),
                           max_splits)
            self.attn_ws = K.AttnWorkspace(1, 1, 64, 1, self.device)

    # ------------------------------------------------------------------------------------------ attention
    def attn_block(self, li, L, x, b: BatchRows, kv, pbuf):
        cfg = self.cfg
        n = x.shape[0]
        pool = kv.k[li]                                            # [pages, 1, 64, 576]
        a = L.qkv_a.forward(x)
        ql = cfg.q_lora_rank
        q_lat = K.rmsnorm(a[:, :ql], L.q_a_norm, cfg.rms_eps, cfg.norm_bias)
        ckv = K.rmsnorm(a[:, ql:ql + LAT], L.kv_a_norm, cfg.rms_eps, cfg.norm_bias)
        krope = a[:, ql + LAT: ql + LAT + ROPE]
        q = L.q_b.forward(q_lat)                                   # [n, heads * 192]
        sel = None
        if getattr(L, "dsa", None) is not None:
            from ..ops import dsa as D
            st = self._dsa_state(li, kv)
            wts = D.update(st, L.dsa, x, b.slot, b.pos)
            if b.tiles is None:                                    # decode / verify rows attend to the indexer's list
                sel = D.select(st, L.dsa.q_proj.forward(q_lat).contiguous(), wts, b.slot, b.pos)
        if not x.is_cuda:
            att = self._attn_reference(L, q, ckv, krope, b, kv, pool, sel)
            return L.o_proj.forward(att, out=pbuf)
        call("mla_rope_store", "pliiplplpppipifi", ptr(q), q.stride(0), self.qd, self.heads, ptr(ckv), ckv.stride(0),
             ptr(krope), krope.stride(0), ptr(b.pos), ptr(b.slot), ptr(kv.page_table), kv.page_table.shape[1], ptr(pool),
             n, float(cfg.rope_theta), 1 if cfg.rope_interleaved else 0)
        vd = cfg.v_head_dim
        if b.tiles is None:                                        # decode / verify rows: absorbed form
            q_abs = torch.empty(n, self.heads, LAT_ROW, dtype=x.dtype, device=x.device)
            call("mla_absorb_q", "pliippii", ptr(q), q.stride(0), self.qd, cfg.qk_nope, ptr(L.w_uk), ptr(q_abs), n, self.heads)
            o_part, lse_part, max_splits = self.mla_ws
            nsplit = max(1, min(max_splits, b.nsplit))
            o_lat = torch.empty(n, self.heads, LAT, dtype=x.dtype, device=x.device)
            a_pos, a_slot, a_table, a_pool = b.pos, b.slot, kv.page_table, pool
            if sel is not None:
                # the listed tokens' latent rows form a short virtual sequence per row in scratch pages
                from ..ops import dsa as D
                idx, nkeys = sel
                if self.dsa_scratch is None or self.dsa_scratch[0].shape[0] < n * D.PAGES_PER_ROW:
                    rows_cap = max(16, n)
                    self.dsa_scratch = (torch.zeros(rows_cap * D.PAGES_PER_ROW, 1, 64, LAT_ROW, dtype=x.dtype, device=x.device),
                                        torch.arange(rows_cap * D.PAGES_PER_ROW, dtype=torch.int32, device=x.device)
                                        .reshape(rows_cap, D.PAGES_PER_ROW).contiguous(),
                                        torch.arange(rows_cap, dtype=torch.int32, device=x.device))
                a_pool, a_table, ar = self.dsa_scratch
                D.gather_rows(pool, kv.page_table, b.slot, idx, nkeys, a_pool)
                a_pos = nkeys - 1
                a_slot = torch.where(b.slot < 0, b.slot, ar[:n])
                nsplit = 1 if nsplit == 1 else min(nsplit, 8)
            call("mla_decode", "pppppppipliiifp", ptr(q_abs), ptr(o_lat), ptr(o_part), ptr(lse_part), ptr(a_pos), ptr(a_slot),
                 ptr(a_table), a_table.shape[1], ptr(a_pool), a_pool.shape[0], n, self.heads, nsplit,
                 float(self.scale), ptr(K.status_word(x.device)))
            att = torch.empty(n, self.heads * vd, dtype=x.dtype, device=x.device)
            call("mla_expand_out", "pppliii", ptr(o_lat), ptr(L.w_uv), ptr(att), att.stride(0), n, self.heads, vd)
        else:
            att = self._attn_prefill_expanded(L, q, b, kv, pool)
        return L.o_proj.forward(att, out=pbuf)

    def _attn_prefill_expanded(self, L, q, b: BatchRows, kv, pool):
        """Expand K / V per head for the context of the chunk's sequence and run the dense paged kernel (hd 256)."""
        cfg = self.cfg
        n, hl, nope, vd = q.shape[0], self.heads, cfg.qk_nope, cfg.v_head_dim
        slot = b.host_slots[0]
        assert all(s == slot for s in b.host_slots), "a prefill chunk holds one sequence"
        ctx = max(b.host_pos) + 1
        npages = (ctx + 63) // 64
        pages = kv.host_table[slot, :npages].long().to(q.device)
        lat = pool[pages, 0].reshape(npages * 64, LAT_ROW)                       # [ctx_pad, 576]
        up = L.w_ukv.forward(lat[:, :LAT].contiguous())                          # [ctx_pad, hl * (nope + vd)]
        up = up.reshape(npages, 64, hl, nope + vd)
        kfull = torch.zeros(npages, hl, 64, 256, dtype=q.dtype, device=q.device)
        vfull = torch.zeros(npages, hl, 64, 256, dtype=q.dtype, device=q.device)
        kfull[..., :nope] = up[..., :nope].permute(0, 2, 1, 3)
        kfull[..., nope:nope + ROPE] = lat[:, LAT:].reshape(npages, 1, 64, ROPE)
        vfull[..., :vd] = up[..., nope:].permute(0, 2, 1, 3)
        q256 = torch.zeros(n, hl, 256, dtype=q.dtype, device=q.device)
        q256[..., : self.qd] = q.reshape(n, hl, self.qd)
        table = torch.arange(npages, dtype=torch.int32, device=q.device).reshape(1, npages)
        slot0 = torch.zeros(n, dtype=torch.int32, device=q.device)
        tiles = K.make_prefill_tiles([0] * n, 1, q.device)
        out = K.attention(q256.reshape(n, hl * 256), b.pos, slot0, table, kfull, vfull, hl, hl, 256, self.scale, tiles=tiles)
        return out.reshape(n, hl, 256)[..., :vd].reshape(n, hl * vd).contiguous()

    def _dsa_state(self, li, kv):
        st = self.dsa_states.get(li)
        if st is None:
            from ..ops import dsa as D
            st = self.dsa_states[li] = D.DSAState(kv.max_slots, kv.max_pages * 64, self.device)
        return st

    def _attn_reference(self, L, q, ckv, krope, b: BatchRows, kv, pool, sel=None):
        """fp32 oracle: rotate, store the latent row, per-row softmax over the expanded keys."""
        from ..ops.reference import rope_rotate
        cfg = self.cfg
        n, hl, nope, vd = q.shape[0], self.heads, cfg.qk_nope, cfg.v_head_dim
        qv = q.reshape(n, hl, self.qd).clone()
        qv[..., nope:] = rope_rotate(qv[..., nope:], b.pos, ROPE, cfg.rope_theta, cfg.rope_interleaved)
        kr = rope_rotate(krope.reshape(n, 1, ROPE).clone(), b.pos, ROPE, cfg.rope_theta, cfg.rope_interleaved)
        for r in range(n):
            s = int(b.slot[r])
            if s < 0:
                continue
            p = int(b.pos[r])
            page = int(kv.page_table[s, p // 64])
            pool[page, 0, p % 64, :LAT] = ckv[r]
            pool[page, 0, p % 64, LAT:] = kr[r, 0]
        out = torch.zeros(n, hl * vd, dtype=q.dtype)
        wuk, wuv = L.w_uk.float(), L.w_uv.float()
        for r in range(n):
            s = int(b.slot[r])
            if s < 0:
                continue
            p = int(b.pos[r])
            pages = kv.page_table[s, : p // 64 + 1].long()
            lat = pool[pages, 0].reshape(-1, LAT_ROW)[: p + 1].float()
            if sel is not None:                                                   # sparse rows: only the listed positions
                lat = lat[sel[0][r, : int(sel[1][r])].long()]
            k_nope = torch.einsum("tc,hdc->htd", lat[:, :LAT], wuk)               # [h, t, nope]
            sc = torch.einsum("hd,htd->ht", qv[r, :, :nope].float(), k_nope)
            sc = sc + qv[r, :, nope:].float() @ lat[:, LAT:].t()
            pr = torch.softmax(sc * self.scale, dim=-1)
            o_lat = (pr @ lat[:, :LAT]).to(q.dtype).float()                       # latent output rounded like the kernel
            out[r] = torch.einsum("hc,hvc->hv", o_lat, wuv).reshape(-1).to(q.dtype)
        return out

