"""Plain PyTorch fp32 statements of every op: the numerics oracle of the CUDA kernels and the CPU path
used by host-side tests (scheduler, server, loaders run the same model code on CPU tensors).

Definitions follow the reference's portable shader math: RMSNorm with constant weight bias
(inc/engine/modules/norm.h:9-31), RoPE (inc/engine/backend/cuda/rope_math.cuh:9-27), SwiGLU with clamp
(src/backend/cuda/modules/swiglu.cu:10-30), causal softmax attention with sliding window / key_end /
sigmoid gate (src/kernels/slang/ref_attention.slang:1-10,47-50,65-70).
"""
from __future__ import annotations

import math

import torch

PAGE = 64


def rmsnorm(x, w, eps, wbias=0.0, residual=None):
    """Returns (out, new_residual). residual (if given) is updated as residual + x first."""
    xf = x.float()
    if residual is not None:
        if residual.dtype == torch.float32:
            xf = xf + residual
            new_res = xf
        else:
            xf = (xf + residual.float()).to(residual.dtype).float()
            new_res = xf.to(residual.dtype)
    else:
        new_res = None
    inv = torch.rsqrt(xf.pow(2).mean(-1, keepdim=True) + eps)
    out = (xf * inv * (w.float() + wbias)).to(x.dtype)
    return out, new_res


def rmsnorm_heads(x, w, heads, hd, eps, wbias=0.0):
    rows = x.shape[0]
    v = x[:, : heads * hd].reshape(rows, heads, hd).float()
    inv = torch.rsqrt(v.pow(2).mean(-1, keepdim=True) + eps)
    return (v * inv * (w.float() + wbias)).to(x.dtype).reshape(rows, heads * hd)


def rope_rotate(v, pos, rot_dim, theta, interleaved=False, pos_scale=1.0, mrope=None):
    """v [rows, heads, hd] -> rotated copy (fp32 math, rounded to v.dtype). ``mrope`` = (pos3 [3, rows], (s0, s1)):
    rotary pairs [0, s0) turn with pos3[0] (time), [s0, s0+s1) with pos3[1] (height), the rest with pos3[2] (width)."""
    rows, heads, hd = v.shape
    half = rot_dim // 2
    i = torch.arange(half, device=v.device, dtype=torch.float32)
    inv_freq = torch.exp2(-math.log2(theta) * (2.0 * i / rot_dim))
    if mrope is not None:
        pos3, (s0, s1) = mrope
        sec = torch.where(torch.arange(half) < s0, 0, torch.where(torch.arange(half) < s0 + s1, 1, 2))
        pp = pos3.float()[sec].t()                                  # [rows, half]
        ang = pp * pos_scale * inv_freq[None, :]
    else:
        ang = pos.float()[:, None] * pos_scale * inv_freq[None, :]
    cs, sn = ang.cos()[:, None, :], ang.sin()[:, None, :]
    vf = v.float().clone()
    if interleaved:
        a0, a1 = vf[..., 0:rot_dim:2], vf[..., 1:rot_dim:2]
        r0, r1 = a0 * cs - a1 * sn, a1 * cs + a0 * sn
        out = vf.clone()
        out[..., 0:rot_dim:2] = r0
        out[..., 1:rot_dim:2] = r1
    else:
        a0, a1 = vf[..., :half], vf[..., half:rot_dim]
        out = vf.clone()
        out[..., :half] = a0 * cs - a1 * sn
        out[..., half:rot_dim] = a1 * cs + a0 * sn
    return out.to(v.dtype)


def rope_store(qkv, pos, slot, page_table, kpool, vpool, nq, nkv, hd, rot_dim, theta, interleaved=False,
               pos_scale=1.0, mrope=None):
    rows = qkv.shape[0]
    q = qkv[:, : nq * hd].reshape(rows, nq, hd)
    k = qkv[:, nq * hd:(nq + nkv) * hd].reshape(rows, nkv, hd)
    v = qkv[:, (nq + nkv) * hd:].reshape(rows, nkv, hd)
    qr = rope_rotate(q, pos, rot_dim, theta, interleaved, pos_scale, mrope)
    kr = rope_rotate(k, pos, rot_dim, theta, interleaved, pos_scale, mrope)
    qkv[:, : nq * hd] = qr.reshape(rows, -1)
    qkv[:, nq * hd:(nq + nkv) * hd] = kr.reshape(rows, -1)
    for r in range(rows):
        s = int(slot[r]) if slot is not None else 0
        if s < 0:
            continue
        p = int(pos[r])
        page = int(page_table[s, p // PAGE])
        kpool[page, :, p % PAGE, :] = kr[r]
        vpool[page, :, p % PAGE, :] = v[r]


def gated_act(gu, I, act=0, limit=0.0):
    g, u = gu[..., :I].float(), gu[..., I:2 * I].float()
    if limit > 0:
        g = g.clamp(max=limit)
        u = u.clamp(-limit, limit)
    a = torch.nn.functional.silu(g) if act == 0 else torch.nn.functional.gelu(g, approximate="tanh")
    return (a * u).to(gu.dtype)


def attention(q, pos, slot, page_table, kpool, vpool, nq, nkv, hd, scale, window=0, key_end=None, gate=None, tree=None):
    """q [rows, >= nq*hd] (already rotated). Returns [rows, nq*hd]. ``tree`` = (base [rows], mask [rows] int64): keys at
    cache positions >= base[r] are visible to row r only where bit (position - base[r]) of mask[r] is set."""
    rows = q.shape[0]
    G = nq // nkv
    out = torch.zeros(rows, nq * hd, dtype=q.dtype, device=q.device)
    for r in range(rows):
        s = int(slot[r]) if slot is not None else 0
        if s < 0:
            continue
        p = int(pos[r])
        lim = int(key_end[r]) if key_end is not None else p
        lo = max(0, p - window + 1) if window > 0 else 0
        n = lim + 1
        pages = page_table[s, : (n + PAGE - 1) // PAGE].long()
        K = kpool[pages].permute(1, 0, 2, 3).reshape(nkv, -1, hd)[:, lo:n].float()
        V = vpool[pages].permute(1, 0, 2, 3).reshape(nkv, -1, hd)[:, lo:n].float()
        qr = q[r, : nq * hd].reshape(nkv, G, hd).float()
        sc = torch.einsum("hgd,hkd->hgk", qr, K) * scale
        if tree is not None:
            tb, tm = int(tree[0][r]), int(tree[1][r])
            keys = torch.arange(lo, n)
            hide = (keys >= tb) & (((tm >> (keys - tb).clamp(min=0)) & 1) == 0)
            sc = sc.masked_fill(hide[None, None, :], float("-inf"))
        pr = torch.softmax(sc, dim=-1)
        o = torch.einsum("hgk,hkd->hgd", pr, V).reshape(nq * hd)
        if gate is not None:
            o = o * torch.sigmoid(gate[r, : nq * hd].float())
        out[r] = o.to(q.dtype)
    return out


def argmax(logits, id_offset=0):
    v, i = logits.float().max(dim=-1)
    # ties -> lowest id: torch.max returns the first maximal index on CPU; enforce explicitly
    eq = logits.float() == v[:, None]
    first = eq.float().argmax(dim=-1)
    return (first + id_offset).int(), v


def topk(logits, k, id_offset=0):
    lf = logits.float()
    vals, ids = torch.sort(lf, dim=-1, descending=True, stable=True)
    lse = torch.logsumexp(lf, dim=-1)
    return (ids[:, :k] + id_offset).int(), vals[:, :k], lse
