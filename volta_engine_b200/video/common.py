"""Shared pieces of the video pipeline: bidirectional attention over one packed sequence and layer norm helpers.

On a GPU the attention runs on the engine's paged attention kernels (keys and values are laid out as one ad-hoc
sequence of 64-row pages, every row's ``key_end`` is the last row, so nothing is masked): head_dim 128 takes the tcgen05
prefill kernel, head_dim 64 (the VAE decoder) the mma.sync one. The CPU statement is a plain softmax.
Reference: src/kernels/cuda/h3/h3_attn.cu:38 (full and key-range attention for head_dim 128 and 64).
"""
from __future__ import annotations

import math

import torch

from ..ops import kernels as K


def full_attention(q: torch.Tensor, k: torch.Tensor, v: torch.Tensor, heads: int, hd: int, scale: float | None = None) -> torch.Tensor:
    """q, k, v [n, heads * hd] -> [n, heads * hd]; every row attends to every row."""
    n = q.shape[0]
    scale = scale if scale is not None else 1.0 / math.sqrt(hd)
    if not q.is_cuda or hd not in (64, 128, 256):
        qh, kh, vh = (t.float().reshape(n, heads, hd).transpose(0, 1) for t in (q, k, v))
        p = torch.softmax(qh @ kh.transpose(1, 2) * scale, -1)
        return (p @ vh).transpose(0, 1).reshape(n, heads * hd).to(q.dtype)
    dev = q.device
    pages = (n + 63) // 64 + 1
    kpool = torch.zeros(pages, heads, 64, hd, dtype=torch.bfloat16, device=dev)
    vpool = torch.zeros_like(kpool)
    idx = torch.arange(n, device=dev)
    kpool[1 + idx // 64, :, idx % 64] = k.reshape(n, heads, hd).to(torch.bfloat16)
    vpool[1 + idx // 64, :, idx % 64] = v.reshape(n, heads, hd).to(torch.bfloat16)
    table = torch.arange(1, pages, dtype=torch.int32, device=dev)[None].contiguous()
    slot = torch.zeros(n, dtype=torch.int32, device=dev)
    key_end = torch.full((n,), n - 1, dtype=torch.int32, device=dev)
    tiles = K.make_prefill_tiles([0] * n, 1, dev)
    qkv = torch.cat([q, k, v], 1).to(torch.bfloat16).contiguous()
    out = K.attention(qkv, idx.int(), slot, table, kpool, vpool, heads, heads, hd, scale, key_end=key_end, tiles=tiles)
    return out.to(q.dtype)


def layer_norm(x: torch.Tensor, w: torch.Tensor, b: torch.Tensor | None, eps: float = 1e-6) -> torch.Tensor:
    xf = x.float()
    y = (xf - xf.mean(-1, keepdim=True)) * torch.rsqrt(xf.var(-1, unbiased=False, keepdim=True) + eps) * w.float()
    return y + b.float() if b is not None else y
