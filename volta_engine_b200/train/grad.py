"""Training primitives (fp32): SwiGLU forward / backward, scaled linear (W = diag(su) T diag(sv)) forward / backward,
row-weighted squared error, Adam (plain, log-scale, additive), row gathers / scatter-adds.

GPU tensors use the kernels of csrc/cuda/train.cu; the two matrix products of the scaled linear are plain library
GEMMs (torch.matmul), as in the reference. CPU tensors run the same arithmetic in PyTorch, which is what the
central-difference gradient checks exercise. Reference: inc/engine/train/grad.h:36-97.
"""
from __future__ import annotations

from dataclasses import dataclass

import torch

from .._lib import call, ptr


def swiglu_forward(g, u, limit: float = 0.0):
    if g.is_cuda:
        a = torch.empty_like(g)
        call("train_swiglu_fwd", "ppplf", ptr(g), ptr(u), ptr(a), g.numel(), float(limit))
        return a
    if limit > 0:
        g, u = g.clamp(max=limit), u.clamp(-limit, limit)
    return g * torch.sigmoid(g) * u


def swiglu_backward(g, u, da, limit: float = 0.0):
    if g.is_cuda:
        dg, du = torch.empty_like(g), torch.empty_like(u)
        call("train_swiglu_bwd", "ppppplf", ptr(g), ptr(u), ptr(da), ptr(dg), ptr(du), g.numel(), float(limit))
        return dg, du
    g_live = torch.ones_like(g, dtype=torch.bool)
    u_live = torch.ones_like(u, dtype=torch.bool)
    if limit > 0:
        g_live, u_live = g < limit, (u > -limit) & (u < limit)
        g, u = g.clamp(max=limit), u.clamp(-limit, limit)
    s = torch.sigmoid(g)
    dact = s * (1 + g * (1 - s))
    return torch.where(g_live, da * u * dact, torch.zeros_like(g)), torch.where(u_live, da * g * s, torch.zeros_like(u))


def scale_rows_(x, s):
    if x.is_cuda:
        call("train_scale_rows", "ppii", ptr(x), ptr(s), x.shape[0], x.shape[1])
        return x
    return x.mul_(s[:, None])


@dataclass
class ScaledLinear:
    """W = diag(su) T diag(sv), T [k, n] frozen (an EXL3 tensor's trellis core between its input and output scales)."""
    T: torch.Tensor
    su: torch.Tensor
    sv: torch.Tensor
    dsu: torch.Tensor | None = None
    dsv: torch.Tensor | None = None


def scaled_linear_forward(l: ScaledLinear, X):
    """-> (Y, Z) with Z = (X diag(su)) T kept for the backward and Y = Z diag(sv)."""
    Z = (X * l.su[None, :]) @ l.T
    return Z * l.sv[None, :], Z


def scaled_linear_backward(l: ScaledLinear, X, Z, dY, want_dx: bool = True):
    """Adds the scale gradients into l.dsu / l.dsv (when present); returns dX (or None)."""
    if l.dsv is not None:
        l.dsv += (dY * Z).sum(0)
    dZ = dY * l.sv[None, :]
    dXs = dZ @ l.T.t()                       # gradient with respect to X diag(su)
    if l.dsu is not None:
        l.dsu += (dXs * X).sum(0)
    return dXs * l.su[None, :] if want_dx else None


def weighted_sq_error(y, t, w=None, want_dy: bool = False, scale: float = 1.0):
    """sum_r w_r |y_r - t_r|^2 (-> python float), and dy = scale * 2 w_r (y - t) when asked for."""
    rows, n = t.shape
    if t.is_cuda:
        part = torch.empty(rows, dtype=torch.float64, device=t.device)
        dy = torch.empty_like(t) if want_dy else None
        call("train_sq_error", "pppiipfp", ptr(y), ptr(t), ptr(w), rows, n, ptr(dy), float(scale), ptr(part))
        return float(part.sum().item()), dy
    d = (y if y is not None else 0.0) - t
    wr = w if w is not None else torch.ones(rows)
    loss = float(((d.double() ** 2).sum(1) * wr.double()).sum())
    return loss, (scale * 2.0 * wr[:, None] * d if want_dy else None)


def weighted_sq_norm(t, w=None) -> float:
    return weighted_sq_error(None, t, w)[0]


@dataclass
class AdamOptions:
    lr: float = 1e-3
    beta1: float = 0.9
    beta2: float = 0.999
    eps: float = 1e-8


def _adam(p, base, derived, g, m, v, step, o: AdamOptions, gscale, mode):
    if p.is_cuda:
        call("train_adam", "pppppplifffffi", ptr(p), ptr(base), ptr(derived), ptr(g), ptr(m), ptr(v), p.numel(), step,
             o.lr, o.beta1, o.beta2, o.eps, float(gscale), mode)
        return
    gi = g * gscale
    if mode == 1:
        gi = gi * derived
    m.mul_(o.beta1).add_(gi, alpha=1 - o.beta1)
    v.mul_(o.beta2).addcmul_(gi, gi, value=1 - o.beta2)
    c1, c2 = 1 - o.beta1 ** step, 1 - o.beta2 ** step
    p.sub_(o.lr * (m / c1) / ((v / c2).sqrt() + o.eps))
    if mode == 1:
        derived.copy_(base * torch.exp(p))
    elif mode == 2:
        derived.copy_(base + p)


def adam_step(p, g, m, v, step: int, o: AdamOptions = AdamOptions()):
    _adam(p, None, None, g, m, v, step, o, 1.0, 0)


def adam_log_scales(s0, a, s, g, m, v, step: int, grad_scale: float = 1.0, o: AdamOptions = AdamOptions()):
    """Parameters s = s0 e^a: Adam on a from g = dL/ds (d/da = s d/ds), then s from the new a."""
    _adam(a, s0, s, g, m, v, step, o, grad_scale, 1)


def adam_deltas(w0, a, w, g, m, v, step: int, grad_scale: float = 1.0, o: AdamOptions = AdamOptions()):
    """Parameters w = w0 + a."""
    _adam(a, w0, w, g, m, v, step, o, grad_scale, 2)


def gather_rows(src, idx, w=None):
    n, cols = idx.numel(), src.shape[1]
    if src.is_cuda:
        dst = torch.empty(n, cols, dtype=torch.float32, device=src.device)
        call("train_gather_rows", "pippiip", ptr(src), 1 if src.dtype == torch.float16 else 0, ptr(idx), ptr(w), n, cols, ptr(dst))
        return dst
    out = src[idx.long()].float()
    return out * w[:, None] if w is not None else out


def scatter_add_rows_(dst, src, idx, w=None):
    """dst[idx[i]] += w[i] * src[i]; idx without repeats within one call."""
    if dst.is_cuda:
        call("train_scatter_add_rows", "pppiip", ptr(src), ptr(idx), ptr(w), idx.numel(), src.shape[1], ptr(dst))
        return dst
    dst.index_add_(0, idx.long(), src * w[:, None] if w is not None else src)
    return dst


def exp_scale(base, a):
    if base.is_cuda:
        out = torch.empty_like(base)
        call("train_exp_scale", "pppl", ptr(base), ptr(a), ptr(out), base.numel())
        return out
    return base * torch.exp(a)
