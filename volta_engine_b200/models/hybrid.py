"""Hybrid decoder: Gated-DeltaNet linear-attention layers interleaved with gated full-attention layers (every
``full_interval``-th layer), dense or mixture-of-experts FFN. Covers the Qwen3.5 / Qwen3-Next family shape:
GDN layers keep a convolution state and a recurrent state per slot instead of KV pages; full layers use
q/k RMSNorm, partial rotary embedding and a sigmoid output gate computed from the layer input.

Reference: src/models/qwen3_5.cpp (48 GDN + 16 gated full-attention layers, MTP head), src/models/qwen4exp.cpp
(GDN + sparse attention + routed experts), inc/engine/modules/gdn.h.
"""
from __future__ import annotations

from dataclasses import dataclass

import torch

from ..ops import kernels as K
from ..ops.gdn import GDNJournal, GDNDims, GDNState, KDAWeights, gdn_forward, kda_forward
from ..ops.linear import LinearBF16
from ..runtime.batch import BatchRows
from .moe import MoEConfig, MoELayer, MoEModel


@dataclass
class HybridConfig(MoEConfig):
    full_interval: int = 4         # layers li with (li + 1) % full_interval == 0 are full attention
    gdn_k_heads: int = 16
    gdn_v_heads: int = 32
    gdn_dk: int = 128
    gdn_dv: int = 128
    gdn_conv: int = 4
    attn_gate: bool = True
    linear_mixer: str = "gdn"      # gdn (one decay per head) | kda (Kimi delta attention: one decay per key channel, low-rank gates)
    kda_rank: int = 128            # rank of the KDA decay / output-gate projections
    qsa: bool = False              # block-sparse attention: a 4-head indexer over pooled keys picks a decode row's 2048 tokens
    model_type: str = "hybrid_gdn"

    @classmethod
    def baseline_next80b(cls):
        """80B-A3B-class hybrid MoE: 48 layers (36 GDN + 12 gated attention), hidden 2048, 512 experts top-10."""
        return cls(n_layers=48, hidden=2048, n_q=16, n_kv=2, head_dim=256, ffn=0, vocab=151936, n_experts=512, top_k=10,
                   expert_ffn=512, shared_ffn=512, router="softmax", rot_dim=64, qk_norm=True, norm_bias=1.0,
                   rope_theta=1e7)

    @classmethod
    def dense_27b(cls):
        """27B-class hybrid with a dense FFN: 64 layers (48 GDN + 16 gated attention), hidden 5120, ffn 17408."""
        return cls(n_layers=64, hidden=5120, n_q=24, n_kv=4, head_dim=256, ffn=17408, vocab=151936, n_experts=1, top_k=1,
                   expert_ffn=128, shared_ffn=0, first_dense_layers=64, rot_dim=64, qk_norm=True, gdn_v_heads=48,
                   norm_bias=1.0, rope_theta=1e7)

    @classmethod
    def flash_next(cls):
        """The Flash-Next assembly (reference: src/models/qwen4_exp.cpp, docs/FLASH_NEXT.md:8-45): 48 layers of hidden
        2560, gated delta-net mixers with block-sparse (QSA) full-attention layers of 24 query / 2 KV heads of 256, 512
        routed experts top-10 (softmax) beside a sigmoid-gated shared expert, four gated fp32 residual streams, the
        checkpoint's own MTP head. (The n-gram embedding layer needs its table files and is left to the loader.)"""
        return cls(n_layers=48, hidden=2560, n_q=24, n_kv=2, head_dim=256, ffn=0, vocab=151936, n_experts=512, top_k=10,
                   expert_ffn=512, shared_ffn=512, shared_gate=True, router="softmax", rot_dim=64, qk_norm=True, norm_bias=1.0,
                   rope_theta=1e7, qsa=True, attn_gate=True, residual="gated", mtp_layers=1, gdn_k_heads=16, gdn_v_heads=32)

    @classmethod
    def qwen3_5_27b(cls):
        """The 27B hybrid assembly (reference: src/models/qwen3_5.cpp): ``dense_27b`` plus the checkpoint's MTP head."""
        c = cls.dense_27b()
        c.mtp_layers = 1
        return c

    @classmethod
    def tiny_hybrid(cls, **kw):
        c = cls(n_layers=4, hidden=256, n_q=4, n_kv=2, head_dim=64, ffn=512, vocab=1024, n_experts=8, top_k=2, expert_ffn=128,
                shared_ffn=128, full_interval=2, gdn_k_heads=2, gdn_v_heads=4, gdn_dk=64, gdn_dv=64, rot_dim=32, qk_norm=True)
        for k, v in kw.items():
            setattr(c, k, v)
        return c

    def is_full(self, li: int) -> bool:
        if li >= self.n_layers_main:
            return True                 # the MTP head's block is a full-attention layer
        return (li + 1) % self.full_interval == 0

    @property
    def n_layers_main(self) -> int:
        return getattr(self, "_n_main", None) or self.n_layers


class HybridLayer(MoELayer):
    __slots__ = ("gdn", "gate_proj", "kv_index", "qsa")


class HybridModel(MoEModel):
    @property
    def prefix_resume(self):
        """"kv+state": a sequence snapshot is the KV pages plus the recurrent and convolution state of the slot at the
        snapshot's last position (``snapshot_state`` / ``restore_state``). Models whose attention layers keep indexer
        keys outside the pool have no resumable snapshot."""
        return None if getattr(self.cfg, "qsa", False) else "kv+state"

    layer_cls = HybridLayer

    def __init__(self, cfg: HybridConfig, device, comm=None):
        super().__init__(cfg, device, comm)
        tp = self.comm.size
        # tensor parallel: the key and value heads of the linear-attention mixers are split over the ranks (a value head
        # reads key head h // (n_v / n_k), so contiguous slices stay together); the fused input projection is column
        # parallel per section, the output projection row parallel into the layer's all-reduce, the state is per rank
        assert cfg.gdn_k_heads % tp == 0 and cfg.gdn_v_heads % tp == 0, "linear-attention heads must divide by the rank count"
        assert tp == 1 or not cfg.qsa, "the block-sparse indexer runs on one GPU in this build"
        self.dims_full = GDNDims(cfg.gdn_k_heads, cfg.gdn_v_heads, cfg.gdn_dk, cfg.gdn_dv, cfg.gdn_conv)
        self.dims = GDNDims(cfg.gdn_k_heads // tp, cfg.gdn_v_heads // tp, cfg.gdn_dk, cfg.gdn_dv, cfg.gdn_conv)
        self.n_full = sum(1 for li in range(cfg.n_layers) if cfg.is_full(li))
        self.gdn_states: list[GDNState] | None = None
        self._li = 0
        self._scratch = None

    @property
    def kv_layers(self) -> int:
        """KV-cache layers this model needs (only the full-attention layers hold keys and values; one more for the MTP
        head's block)."""
        return self.n_full + int(getattr(self.cfg, "mtp_layers", 0) or 0)

    def init_random(self, seed: int = 4, std: float = 0.02, search: bool = False):
        self._li = 0
        cfg = self.cfg
        cfg._n_main = cfg.n_layers
        self._init_random_with_mtp(super().init_random, seed, std, search)
        if self.mtp is not None and cfg.qk_norm:
            L = self.mtp["layer"]
            L.q_norm = torch.ones(cfg.head_dim, device=self.device, dtype=torch.bfloat16) * (1.0 - cfg.norm_bias)
            L.k_norm = L.q_norm.clone()
        if cfg.qk_norm:
            for L in self.layers:
                if L.gdn is None:
                    L.q_norm = torch.ones(cfg.head_dim, device=self.device, dtype=torch.bfloat16) * (1.0 - cfg.norm_bias)
                    L.k_norm = L.q_norm.clone()
        return self

    def _init_attention(self, L, rnd, search):
        cfg, d, dev = self.cfg, self.dims, self.device
        li = self._li
        self._li += 1
        L.gdn = L.gate_proj = L.qsa = None
        L.kv_index = -1
        if cfg.is_full(li):
            super()._init_attention(L, rnd, search)
            L.kv_index = sum(1 for j in range(li) if cfg.is_full(j))
            if cfg.attn_gate:
                wg = rnd(cfg.n_q * cfg.head_dim, cfg.hidden)
                q0, q1 = self.comm.rank * self.nq * cfg.head_dim, (self.comm.rank + 1) * self.nq * cfg.head_dim
                L.gate_proj = self._make_linear(wg[q0:q1].contiguous(), search, whole=wg)
            if cfg.qsa:
                from ..ops import dsa as D
                from ..ops.linear import LinearBF16
                z = torch.zeros(D.DIM, device=dev, dtype=torch.bfloat16)
                L.qsa = D.QSAWeights(proj=LinearBF16((rnd(D.QSA_HEADS * D.DIM + D.DIM, cfg.hidden) * 8).to(torch.bfloat16)),
                                     q_norm=z.clone(), k_norm=z.clone(), rot=min(64, D.DIM), theta=cfg.rope_theta, eps=cfg.rms_eps)
            return
        H = cfg.hidden
        r, tp, df = self.comm.rank, self.comm.size, self.dims_full
        real = df.conv_dim + df.n_v * df.dv + 2 * df.n_v
        w_full = rnd(real, H)                                   # [q | k | v | z | b | a] of all heads

        def sections(nk, nv):
            return [nk * d.dk, nk * d.dk, nv * d.dv, nv * d.dv, nv, nv]
        rows, at = [], 0
        for full_n, mine_n in zip(sections(df.n_k, df.n_v), sections(d.n_k, d.n_v)):
            rows.append(torch.arange(at + r * mine_n, at + (r + 1) * mine_n, device=dev))     # this rank's slice of the section
            at += full_n
        rows = torch.cat(rows)
        w_in = torch.zeros(d.proj_out, H, device=dev)
        w_in[:rows.numel()] = w_full[rows]
        conv_full = (rnd(df.conv_dim, d.conv_k) * (0.5 / 0.02)).float()
        v0, v1 = r * d.n_v, (r + 1) * d.n_v
        w_out = rnd(H, df.n_v * d.dv)
        g = {"in_proj": self._make_linear(w_in, search, whole=w_full),
             "conv_w": conv_full[rows[: d.conv_dim]].contiguous(),
             "A_log": torch.log(torch.linspace(1.0, 8.0, df.n_v, device=dev)).float()[v0:v1].contiguous(),
             "dt_bias": torch.linspace(-1.0, 1.0, df.n_v, device=dev).float()[v0:v1].contiguous(),
             "norm_w": torch.ones(d.dv, device=dev, dtype=torch.float32),
             "out_proj": self._make_linear(w_out[:, v0 * d.dv:v1 * d.dv].contiguous(), search, whole=w_out)}
        if cfg.linear_mixer == "kda":
            from ..ops.linear import LinearBF16
            bf, kr = torch.bfloat16, cfg.kda_rank
            assert d.n_k == d.n_v, "KDA has as many key heads as value heads"
            f_b, g_b = (rnd(df.n_v * d.dk, kr) * 10).to(bf), (rnd(df.n_v * d.dv, kr) * 10).to(bf)
            g["kda"] = KDAWeights(f_a=LinearBF16(rnd(kr, H).to(bf)), f_b=LinearBF16(f_b[v0 * d.dk:v1 * d.dk].contiguous()),
                                  g_a=LinearBF16(rnd(kr, H).to(bf)), g_b=LinearBF16(g_b[v0 * d.dv:v1 * d.dv].contiguous()),
                                  A_log=torch.log(torch.linspace(0.5, 2.0, df.n_v, device=dev)).float()[v0:v1].contiguous(),
                                  dt_bias=torch.linspace(-1.0, 1.0, df.n_v * d.dk, device=dev).float()[v0 * d.dk:v1 * d.dk].contiguous(),
                                  norm_w=g["norm_w"])
        L.gdn = g
        L.qkv = L.o_proj = None

    def _attn_bytes(self, L) -> int:
        if L.gdn is not None:
            return L.gdn["in_proj"].nbytes() + L.gdn["out_proj"].nbytes()
        n = L.qkv.nbytes() + L.o_proj.nbytes()
        return n + (L.gate_proj.nbytes() if L.gate_proj is not None else 0)

    def state_bytes_per_slot(self) -> int:
        d = self.dims
        per = ((d.conv_k - 1) * d.conv_dim + d.n_v * d.dk * d.dv) * 4
        return per * (self.cfg.n_layers - self.n_full)

    def _states(self, kv):
        if self.gdn_states is None:
            self.gdn_states = [GDNState(self.dims, kv.max_slots, self.device) if L.gdn is not None else None
                               for L in self.layers]
        return self.gdn_states

    def attn_block(self, li, L, x, b: BatchRows, kv, pbuf):
        cfg = self.cfg
        if L.gdn is not None:
            g = L.gdn
            proj = g["in_proj"].forward(x)
            st = self._states(kv)[li]
            jn = None
            if self.journal_on and b.tiles is None:
                # rows of a speculative verify block (one slot): keep what is needed to take rejected rows back
                js = self._jcur
                jn = js["layers"].get(li)
                if jn is None:
                    sh = self._shadows.get(li)
                    if sh is None:
                        sh = self._shadows[li] = (torch.zeros_like(st.conv[:1]), torch.zeros_like(st.rec[:1]))
                    jn = js["layers"][li] = GDNJournal(st, sh)
                if js["rows"] is None:
                    js["rows"] = (b.pos.clone(), b.slot.clone())      # the engine advances its row descriptor after the step
            jpos, jslot = self._jcur["rows"] if jn is not None else (b.pos, b.slot)
            if "kda" in g:
                y = kda_forward(proj, x, g["kda"], jpos, jslot, st, self.dims, g["conv_w"], cfg.rms_eps, journal=jn)
                return g["out_proj"].forward(y.to(x.dtype), out=pbuf)
            y = gdn_forward(proj, jpos, jslot, st, self.dims, g["conv_w"], g["A_log"], g["dt_bias"],
                            g["norm_w"], cfg.rms_eps, journal=jn)
            return g["out_proj"].forward(y.to(x.dtype), out=pbuf)
        kpool, vpool = kv.layer(L.kv_index)
        qkv = L.qkv.forward(x)
        if cfg.qk_norm:
            stride = qkv.stride(0)
            K.rmsnorm_heads_(qkv, L.q_norm, b.n, self.nq, self.hd, stride, cfg.rms_eps, cfg.norm_bias, 0)
            K.rmsnorm_heads_(qkv, L.k_norm, b.n, self.nkv, self.hd, stride, cfg.rms_eps, cfg.norm_bias, self.nq * self.hd)
        K.rope_store(qkv, b.pos, b.slot, kv.page_table, kpool, vpool, self.nq, self.nkv, self.hd, self.rot,
                     cfg.rope_theta, cfg.rope_interleaved)
        gate = L.gate_proj.forward(x) if L.gate_proj is not None else None
        a_pos, a_slot, a_table, a_k, a_v, nsplit = b.pos, b.slot, kv.page_table, kpool, vpool, b.nsplit
        if getattr(L, "qsa", None) is not None:
            from ..ops import dsa as D
            st = self._qsa_state(li, kv)
            qi = D.qsa_update(st, L.qsa, x, b.slot, b.pos)
            if b.tiles is None and b.key_end is None:
                # decode rows attend to the indexer's list: the listed keys and values form a short virtual sequence per
                # row in scratch pages (prefill chunks attend densely)
                idx, nkeys = D.qsa_select(st, qi, b.slot, b.pos)
                a_k, a_v, a_table, ar = self._qsa_scratch(b.n, kpool)
                D.gather_rows(kpool, kv.page_table, b.slot, idx, nkeys, a_k)
                D.gather_rows(vpool, kv.page_table, b.slot, idx, nkeys, a_v)
                a_pos = nkeys - 1
                a_slot = torch.where(b.slot < 0, b.slot, ar[:b.n])
                nsplit = min(nsplit, 8)
        att = K.attention(qkv, a_pos, a_slot, a_table, a_k, a_v, self.nq, self.nkv, self.hd, self.scale,
                          window=cfg.sliding_window, key_end=b.key_end, gate=gate, tiles=b.tiles,
                          nsplit=1 if b.tiles is not None else nsplit, ws=self.attn_ws)
        return L.o_proj.forward(att, out=pbuf)

    def _qsa_state(self, li, kv):
        if not hasattr(self, "qsa_states"):
            self.qsa_states, self.qsa_scr = {}, None
        st = self.qsa_states.get(li)
        if st is None:
            from ..ops import dsa as D
            st = self.qsa_states[li] = D.QSAState(kv.max_slots, kv.max_pages * 64, self.device)
        return st

    def _qsa_scratch(self, n, kpool):
        from ..ops import dsa as D
        if self.qsa_scr is None or self.qsa_scr[3].numel() < n:
            cap = max(16, n)
            shape = (cap * D.PAGES_PER_ROW,) + tuple(kpool.shape[1:])
            self.qsa_scr = (torch.zeros(shape, dtype=kpool.dtype, device=kpool.device),
                            torch.zeros(shape, dtype=kpool.dtype, device=kpool.device),
                            torch.arange(cap * D.PAGES_PER_ROW, dtype=torch.int32, device=kpool.device)
                            .reshape(cap, D.PAGES_PER_ROW).contiguous(),
                            torch.arange(cap, dtype=torch.int32, device=kpool.device))
        return self.qsa_scr

    # ---- speculative verify blocks: journal and rollback of the recurrent state
    journal_on = False            # set by the engine for a verify step (rows of one slot that may be rejected)

    def begin_journal(self, on: bool, tag=0) -> None:
        """Called before a forward. ``tag`` names the set of operands this forward records into (the engine passes the
        row count: a CUDA graph of that row count keeps writing the tensors its capture pass recorded)."""
        self.journal_on = bool(on)
        if not hasattr(self, "_jsets"):
            self._jsets, self._shadows = {}, {}
        if on:
            self._jcur = self._jsets.setdefault(tag, {"rows": None, "layers": {}})
            self._jcur["rows"] = None
            self._jlast = tag

    def rollback_state(self, slot: int, keep: int) -> None:
        """After a journalled block: leave the slot's recurrent and convolution state as if only the block's first
        ``keep`` rows had run (the KV pool needs nothing: rejected rows are overwritten by the next step)."""
        js = getattr(self, "_jsets", {}).get(getattr(self, "_jlast", None))
        if js is None:
            raise RuntimeError("rollback without a journalled step")
        for li, jn in js["layers"].items():
            jn.replay(self.gdn_states[li], slot, keep)

    # recurrent state travels with sequence snapshots
    def snapshot_state(self, slot: int) -> list:
        return [s.snapshot(slot) if s is not None else None for s in (self.gdn_states or [])]

    def restore_state(self, slot: int, snaps: list):
        for s, snap in zip(self.gdn_states or [], snaps):
            if s is not None and snap is not None:
                s.restore(slot, snap)

    def pack_state(self, slot: int) -> dict:
        """The slot's state of every linear-attention layer as two stacked host tensors (what a prefix snapshot stores)."""
        sts = [s for s in (self.gdn_states or []) if s is not None]
        if not sts:
            return {}
        return {"gdn_conv": torch.stack([s.conv[slot] for s in sts]).cpu(), "gdn_rec": torch.stack([s.rec[slot] for s in sts]).cpu()}

    def unpack_state(self, slot: int, snap: dict, kv) -> None:
        sts = [s for s in self._states(kv) if s is not None]
        for i, s in enumerate(sts):
            s.conv[slot].copy_(snap["gdn_conv"][i])
            s.rec[slot].copy_(snap["gdn_rec"][i])
