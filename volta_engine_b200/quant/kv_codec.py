"""KV cache element codecs in PyTorch: the CPU path of the quantised cache formats and the oracle of the store / attention
kernels.

Formats of one cache tensor (reference: inc/engine/core/kv_format.h:9-18, src/backend/cuda/modules/kv_quant.cuh:166-246):
  I8   one byte per element, one fp16 scale per 64 elements (amax / 127), round to nearest, clamp +-127
  Q4   4 bits per element (value + 8 in a nibble, low nibble = even element), one fp16 scale per 64 (amax / 7) taken after
       an orthonormal 64-point Walsh-Hadamard rotation of the 64 elements (its own inverse)
  FP4  E2M1 per element, one E4M3 scale byte per 16 elements (amax / 6)
Whole-cache presets: k8v4 = (I8 keys, Q4 values), nvfp4 = (FP4, FP4).
"""
from __future__ import annotations

import torch

from . import nvfp4 as qn

Q_BF16, Q_E5M2, Q_I8, Q_Q4, Q_FP4 = 0, 1, 2, 3, 4
# cache format code -> (key codec, value codec)
FORMATS = {0: (Q_BF16, Q_BF16), 1: (Q_E5M2, Q_E5M2), 2: (Q_I8, Q_Q4), 3: (Q_FP4, Q_FP4)}
FORMAT_CODES = {"bf16": 0, "fp16": 0, "fp8": 1, "k8v4": 2, "nvfp4": 3}


def data_bytes(q: int, hd: int) -> int:
    return {Q_BF16: 2 * hd, Q_E5M2: hd, Q_I8: hd, Q_Q4: hd // 2, Q_FP4: hd // 2}[q]


def scale_bytes(q: int, hd: int) -> int:
    return {Q_I8: hd // 64 * 2, Q_Q4: hd // 64 * 2, Q_FP4: hd // 16}.get(q, 0)


def fwht64(x: torch.Tensor) -> torch.Tensor:
    """Orthonormal 64-point Walsh-Hadamard transform over the last dimension (length 64)."""
    y = x.float().clone()
    h = 1
    while h < 64:
        y = y.reshape(*y.shape[:-1], 64 // (2 * h), 2, h)
        a, b = y[..., 0, :], y[..., 1, :]
        y = torch.stack([a + b, a - b], dim=-2).reshape(*y.shape[:-3], 64)
        h *= 2
    return y * 0.125


def encode(x: torch.Tensor, q: int):
    """x [..., hd] -> (data uint8 [..., data_bytes], scales uint8 [..., scale_bytes])."""
    hd = x.shape[-1]
    xf = x.float()
    if q in (Q_I8, Q_Q4):
        v = xf.reshape(*x.shape[:-1], hd // 64, 64)
        if q == Q_Q4:
            v = fwht64(v)
        top = 127.0 if q == Q_I8 else 7.0
        sh = (v.abs().amax(-1) / top).to(torch.float16)
        s = sh.float()
        inv = torch.where(s > 0, 1.0 / s, torch.zeros_like(s))
        qv = torch.round(v * inv[..., None])
        scales = sh.contiguous().view(torch.uint8).reshape(*x.shape[:-1], hd // 64 * 2)
        if q == Q_I8:
            return qv.clamp(-127, 127).to(torch.int8).view(torch.uint8).reshape(*x.shape[:-1], hd), scales
        n = (qv.clamp(-8, 7) + 8).to(torch.uint8).reshape(*x.shape[:-1], hd // 2, 2)
        return n[..., 0] | (n[..., 1] << 4), scales
    if q == Q_FP4:
        v = xf.reshape(*x.shape[:-1], hd // 16, 16)
        sb = qn.e4m3_encode(v.abs().amax(-1) / 6.0)
        s = qn.e4m3_decode(sb).float()
        inv = torch.where(s > 0, 1.0 / s, torch.zeros_like(s))
        c = qn.e2m1_encode(v * inv[..., None]).reshape(*x.shape[:-1], hd // 2, 2)
        return c[..., 0] | (c[..., 1] << 4), sb.reshape(*x.shape[:-1], hd // 16)
    raise ValueError(f"codec {q} has no packed form")


def decode(data: torch.Tensor, scales: torch.Tensor, q: int, hd: int) -> torch.Tensor:
    """Inverse of ``encode`` -> fp32 [..., hd]."""
    lead = data.shape[:-1]
    if q == Q_I8:
        s = scales.contiguous().view(torch.float16).float().reshape(*lead, hd // 64)
        return (data.contiguous().view(torch.int8).float().reshape(*lead, hd // 64, 64) * s[..., None]).reshape(*lead, hd)
    if q == Q_Q4:
        s = scales.contiguous().view(torch.float16).float().reshape(*lead, hd // 64)
        n = torch.stack([data & 15, data >> 4], dim=-1).reshape(*lead, hd // 64, 64).float() - 8.0
        return fwht64(n * s[..., None]).reshape(*lead, hd)
    if q == Q_FP4:
        s = qn.e4m3_decode(scales).float().reshape(*lead, hd // 16)
        c = torch.stack([data & 15, data >> 4], dim=-1).reshape(*lead, hd // 16, 16)
        return (qn.e2m1_decode(c).float() * s[..., None]).reshape(*lead, hd)
    raise ValueError(f"codec {q} has no packed form")
