"""Gated DeltaNet (linear attention with a gated delta rule) mixer: fp32 oracle and GPU entry points.

Per layer and slot the mixer keeps a short-convolution state (the last ``conv_k - 1`` inputs of every q/k/v channel)
and a recurrent state S [v_heads, dk, dv] in fp32. For each token t (per value head, key heads repeated):

    u   = silu(causal_conv1d([q|k|v])),  q, k = l2norm(u_q), l2norm(u_k),  q *= dk^-0.5
    g_t = -exp(A_log) * softplus(a_t + dt_bias),  beta_t = sigmoid(b_t)
    S   = S * exp(g_t);  delta = (v_t - S^T k_t) * beta_t;  S += k_t (x) delta;  o_t = S^T q_t
    y_t = rmsnorm(o_t) * w * silu(z_t)

A row whose position is 0 starts its slot from a zero state. Rows of one slot inside a batch are consecutive positions.
Reference: inc/engine/modules/gdn.h (``project_gates``, ``causal_conv1d_silu*``, ``l2_norm_heads``,
``recurrent_step[_rows]``, ``gated_rmsnorm``), src/models/qwen3_5.cpp (layer wiring).
"""
from __future__ import annotations

from dataclasses import dataclass

import torch
import torch.nn.functional as F

from .._lib import call, ptr


@dataclass
class GDNDims:
    n_k: int = 16          # key / query heads
    n_v: int = 32          # value heads (multiple of n_k)
    dk: int = 128
    dv: int = 128
    conv_k: int = 4

    @property
    def conv_dim(self) -> int:
        return 2 * self.n_k * self.dk + self.n_v * self.dv

    @property
    def proj_out(self) -> int:
        """Columns of the fused input projection: [q | k | v | z | b | a], padded to a multiple of 128."""
        n = self.conv_dim + self.n_v * self.dv + 2 * self.n_v
        return (n + 127) // 128 * 128


class GDNState:
    """conv [slots, conv_k-1, conv_dim] (oldest first) and rec [slots, n_v, dk, dv] fp32 of one layer."""

    def __init__(self, d: GDNDims, max_slots: int, device):
        self.conv = torch.zeros(max_slots, d.conv_k - 1, d.conv_dim, dtype=torch.float32, device=device)
        self.rec = torch.zeros(max_slots, d.n_v, d.dk, d.dv, dtype=torch.float32, device=device)

    def nbytes(self):
        return (self.conv.numel() + self.rec.numel()) * 4

    def snapshot(self, slot: int) -> dict:
        return {"conv": self.conv[slot].cpu().clone(), "rec": self.rec[slot].cpu().clone()}

    def restore(self, slot: int, snap: dict):
        self.conv[slot].copy_(snap["conv"])
        self.rec[slot].copy_(snap["rec"])


def gdn_reference(proj, pos, slot, st: GDNState, d: GDNDims, conv_w, A_log, dt_bias, norm_w, eps: float) -> torch.Tensor:
    """proj [n, proj_out] (fused projection of the rows) -> y [n, n_v*dv]; updates ``st`` in place."""
    n = proj.shape[0]
    C, nv, nk, dk, dv, kc = d.conv_dim, d.n_v, d.n_k, d.dk, d.dv, d.conv_k
    pf = proj.float()
    raw = pf[:, :C]
    z = pf[:, C:C + nv * dv].reshape(n, nv, dv)
    b = pf[:, C + nv * dv: C + nv * dv + nv]
    a = pf[:, C + nv * dv + nv: C + nv * dv + 2 * nv]
    cw = conv_w.float()                                       # [C, conv_k], tap conv_k-1 multiplies the current input
    y = torch.zeros(n, nv, dv)
    rep = nv // nk
    for i in range(n):
        s, p = int(slot[i]), int(pos[i])
        if s < 0:
            continue
        if p == 0:
            st.conv[s].zero_()
            st.rec[s].zero_()
        hist = torch.cat([st.conv[s], raw[i:i + 1]], 0)      # [conv_k, C]
        u = F.silu((hist * cw.t()).sum(0))
        st.conv[s] = hist[1:]
        q = u[: nk * dk].reshape(nk, dk)
        k = u[nk * dk: 2 * nk * dk].reshape(nk, dk)
        v = u[2 * nk * dk:].reshape(nv, dv)
        q = q / torch.sqrt((q * q).sum(-1, keepdim=True) + 1e-6) * dk ** -0.5
        k = k / torch.sqrt((k * k).sum(-1, keepdim=True) + 1e-6)
        q, k = q.repeat_interleave(rep, 0), k.repeat_interleave(rep, 0)
        g = -torch.exp(A_log.float()) * F.softplus(a[i] + dt_bias.float())
        beta = torch.sigmoid(b[i])
        S = st.rec[s] * torch.exp(g)[:, None, None]
        mem = torch.einsum("hkv,hk->hv", S, k)
        delta = (v - mem) * beta[:, None]
        S = S + k[:, :, None] * delta[:, None, :]
        st.rec[s] = S
        o = torch.einsum("hkv,hk->hv", S, q)
        o = o * torch.rsqrt((o * o).mean(-1, keepdim=True) + eps) * norm_w.float()[None, :]
        y[i] = o * F.silu(z[i])
    return y.reshape(n, nv * dv)


class GDNJournal:
    """What a block of rows did to one layer's state, kept so that a speculative verify step can be taken back: the
    state of the block's slot before the block (``shadow``) and the per-row operands of the recurrence (on the GPU the
    outputs of the prepare kernel: post-convolution q | k | v, decay and beta; on the CPU the projection rows).
    ``replay(keep)`` restores the shadow and applies the first ``keep`` rows again with the same kernel and the same
    operands, so the state equals, bit for bit, the one that stepping only those rows would have left.
    Reference: inc/engine/modules/gdn.h:157-161 (journal + kda_replay). A slot's state of one layer is 2 MB here, so
    the shadow is a device copy inside the verify step's graph rather than a 36 MiB snapshot per row."""

    def __init__(self, st: GDNState, shadow: tuple | None = None):
        """``shadow``: (conv [1, ...], rec [1, ...]) buffers shared by the journals of one layer (one per row count of the
        verify step: each CUDA graph keeps its own operands, and only the last step's shadow is ever needed)."""
        self.shadow_conv, self.shadow_rec = shadow if shadow is not None else (torch.zeros_like(st.conv[:1]),
                                                                               torch.zeros_like(st.rec[:1]))
        self.rows = None          # operands of the last journalled block
        self.fn = None            # callable(keep): applies rows [0, keep) to the state

    def begin(self, st: GDNState, slot: torch.Tensor):
        idx = slot[:1].clamp(min=0).long()
        torch.index_select(st.conv, 0, idx, out=self.shadow_conv)
        torch.index_select(st.rec, 0, idx, out=self.shadow_rec)

    def replay(self, st: GDNState, slot: int, keep: int):
        st.conv[slot].copy_(self.shadow_conv[0])
        st.rec[slot].copy_(self.shadow_rec[0])
        if keep > 0 and self.fn is not None:
            self.fn(keep)


def gdn_forward(proj, pos, slot, st: GDNState, d: GDNDims, conv_w, A_log, dt_bias, norm_w, eps: float, scratch=None,
                journal: GDNJournal | None = None):
    """GPU path: prepare (conv + norms + gates, parallel over rows), recurrence (sequential per slot), gated norm.
    ``journal``: the block's slot state is copied aside first and the operands are kept for ``journal.replay``."""
    if journal is not None:
        journal.begin(st, slot)
    if not proj.is_cuda:
        if journal is not None:
            journal.fn = lambda keep: gdn_reference(proj[:keep], pos[:keep], slot[:keep], st, d, conv_w, A_log, dt_bias,
                                                    norm_w, eps)
        return gdn_reference(proj, pos, slot, st, d, conv_w, A_log, dt_bias, norm_w, eps).to(proj.dtype)
    n = proj.shape[0]
    dev = proj.device
    C, nv = d.conv_dim, d.n_v
    if scratch is None or scratch[0].shape[0] < n:
        scratch = (torch.empty(n, C, dtype=torch.float32, device=dev), torch.empty(n, 2 * nv, dtype=torch.float32, device=dev),
                   torch.empty(n, nv * d.dv, dtype=torch.float32, device=dev))
    u, gb, o = scratch
    out = torch.empty(n, nv * d.dv, dtype=torch.bfloat16, device=dev)
    call("gdn_prepare", "plpppppppp" + "iiiiiii", ptr(proj), proj.stride(0), ptr(pos), ptr(slot), ptr(st.conv), ptr(conv_w),
         ptr(A_log), ptr(dt_bias), ptr(u), ptr(gb), n, d.n_k, d.n_v, d.dk, d.dv, d.conv_k, st.conv.shape[0])
    call("gdn_recurrent", "plpppppppiiiiiii", ptr(proj), proj.stride(0), ptr(pos), ptr(slot), ptr(st.conv), ptr(st.rec),
         ptr(u), ptr(gb), ptr(o), n, d.n_k, d.n_v, d.dk, d.dv, d.conv_k, st.conv.shape[0])
    call("gdn_gated_norm", "pplpp" + "iiiii" + "f", ptr(o), ptr(proj), proj.stride(0), ptr(norm_w), ptr(out), n, d.n_v, d.dv,
         C, d.conv_k, float(eps))
    if journal is not None:
        o2 = torch.empty_like(o)

        def again(keep, proj=proj, pos=pos, slot=slot, u=u, gb=gb):
            call("gdn_recurrent", "plpppppppiiiiiii", ptr(proj), proj.stride(0), ptr(pos), ptr(slot), ptr(st.conv), ptr(st.rec),
                 ptr(u), ptr(gb), ptr(o2), keep, d.n_k, d.n_v, d.dk, d.dv, d.conv_k, st.conv.shape[0])
        journal.fn = again
    return out


# ---------------------------------------------------------------------------------------------- KDA
@dataclass
class KDAWeights:
    """Kimi-delta-attention gates of one layer (heads of 128 x 128, as many key heads as value heads).
    Reference: inc/engine/modules/gdn.h:113-132 (project_kda_gates operands)."""
    f_a: object               # linear hidden -> rank        (decay, low rank)
    f_b: object               # linear rank -> heads * dk
    g_a: object               # linear hidden -> rank        (output gate, low rank)
    g_b: object               # linear rank -> heads * dv
    A_log: torch.Tensor       # [heads] fp32
    dt_bias: torch.Tensor     # [heads * dk] fp32
    norm_w: torch.Tensor      # [dv] fp32


def kda_reference(proj, f, z, pos, slot, st: GDNState, d: GDNDims, conv_w, A_log, dt_bias, norm_w, eps: float) -> torch.Tensor:
    """fp32 statement. proj [n, >= conv_dim + nv*dv + nv] = [q | k | v | (unused z) | b | ...], f [n, nv*dk] decay
    pre-activations, z [n, nv*dv] gate pre-activations. Per row: conv + SiLU, L2 norms and the q scale as the gated delta
    rule; S = diag(exp(g)) S with g = -5 sigmoid(exp(A_log[h]) (f + dt_bias)) per key channel; delta = beta (v - S^T k);
    S += k delta^T; y = rmsnorm(S^T q) * w * sigmoid(z)."""
    n = proj.shape[0]
    C, nv, nk, dk, dv = d.conv_dim, d.n_v, d.n_k, d.dk, d.dv
    assert nk == nv
    pf = proj.float()
    raw = pf[:, :C]
    b = pf[:, C + nv * dv: C + nv * dv + nv]
    cw = conv_w.float()
    y = torch.zeros(n, nv, dv)
    for i in range(n):
        s, p = int(slot[i]), int(pos[i])
        if s < 0:
            continue
        if p == 0:
            st.conv[s].zero_()
            st.rec[s].zero_()
        hist = torch.cat([st.conv[s], raw[i:i + 1]], 0)
        u = F.silu((hist * cw.t()).sum(0))
        st.conv[s] = hist[1:]
        q = u[: nk * dk].reshape(nk, dk)
        k = u[nk * dk: 2 * nk * dk].reshape(nk, dk)
        v = u[2 * nk * dk:].reshape(nv, dv)
        q = q / torch.sqrt((q * q).sum(-1, keepdim=True) + 1e-6) * dk ** -0.5
        k = k / torch.sqrt((k * k).sum(-1, keepdim=True) + 1e-6)
        g = -5.0 * torch.sigmoid(torch.exp(A_log.float())[:, None] * (f[i].float().reshape(nv, dk) + dt_bias.float().reshape(nv, dk)))
        beta = torch.sigmoid(b[i])
        S = st.rec[s] * torch.exp(g)[:, :, None]
        mem = torch.einsum("hkv,hk->hv", S, k)
        delta = (v - mem) * beta[:, None]
        S = S + k[:, :, None] * delta[:, None, :]
        st.rec[s] = S
        o = torch.einsum("hkv,hk->hv", S, q)
        o = o * torch.rsqrt((o * o).mean(-1, keepdim=True) + eps) * norm_w.float()[None, :]
        y[i] = o * torch.sigmoid(z[i].float().reshape(nv, dv))
    return y.reshape(n, nv * dv)


def kda_forward(proj, x, W: KDAWeights, pos, slot, st: GDNState, d: GDNDims, conv_w, eps: float,
                journal: GDNJournal | None = None) -> torch.Tensor:
    """Kimi delta attention over the rows: ``proj`` is the fused [q | k | v | - | b | -] projection of ``x`` (the layout of
    the gated delta rule, its z and a columns unused), the decay and the output gate come from the low-rank pairs in ``W``."""
    f = W.f_b.forward(W.f_a.forward(x))
    z = W.g_b.forward(W.g_a.forward(x))
    if journal is not None:
        journal.begin(st, slot)
    if not proj.is_cuda:
        if journal is not None:
            journal.fn = lambda keep: kda_reference(proj[:keep], f[:keep], z[:keep], pos[:keep], slot[:keep], st, d, conv_w,
                                                    W.A_log, W.dt_bias, W.norm_w, eps)
        return kda_reference(proj, f, z, pos, slot, st, d, conv_w, W.A_log, W.dt_bias, W.norm_w, eps).to(proj.dtype)
    n, dev = proj.shape[0], proj.device
    C, nv = d.conv_dim, d.n_v
    u = torch.empty(n, C, dtype=torch.float32, device=dev)
    gb = torch.empty(n, 2 * nv, dtype=torch.float32, device=dev)
    o = torch.empty(n, nv * d.dv, dtype=torch.float32, device=dev)
    kdec = torch.empty(n, nv * d.dk, dtype=torch.float32, device=dev)
    out = torch.empty(n, nv * d.dv, dtype=torch.bfloat16, device=dev)
    zero = torch.zeros(nv, dtype=torch.float32, device=dev)
    call("gdn_prepare", "plpppppppp" + "iiiiiii", ptr(proj), proj.stride(0), ptr(pos), ptr(slot), ptr(st.conv), ptr(conv_w),
         ptr(zero), ptr(zero), ptr(u), ptr(gb), n, d.n_k, d.n_v, d.dk, d.dv, d.conv_k, st.conv.shape[0])
    call("kda_decay", "plpppiii", ptr(f), f.stride(0), ptr(W.A_log), ptr(W.dt_bias), ptr(kdec), n, nv, d.dk)
    call("kda_recurrent", "plppppppppiiiiiii", ptr(proj), proj.stride(0), ptr(pos), ptr(slot), ptr(st.conv), ptr(st.rec),
         ptr(u), ptr(gb), ptr(o), ptr(kdec), n, d.n_k, d.n_v, d.dk, d.dv, d.conv_k, st.conv.shape[0])
    call("kda_gated_norm", "pplppiiif", ptr(o), ptr(z), z.stride(0), ptr(W.norm_w), ptr(out), n, nv, d.dv, float(eps))
    if journal is not None:
        o2 = torch.empty_like(o)

        def again(keep, proj=proj, pos=pos, slot=slot, u=u, gb=gb, kdec=kdec):
            call("kda_recurrent", "plppppppppiiiiiii", ptr(proj), proj.stride(0), ptr(pos), ptr(slot), ptr(st.conv), ptr(st.rec),
                 ptr(u), ptr(gb), ptr(o2), ptr(kdec), keep, d.n_k, d.n_v, d.dk, d.dv, d.conv_k, st.conv.shape[0])
        journal.fn = again
    return out
