"""GGUF block formats in vectorised PyTorch (CPU or GPU): the oracle of the fused dequant mat-vec kernels,
the quantise-at-write path of the synthetic checkpoint writers, and the CPU linear semantics.

Block layouts are the ggml ones the reference consumes (inc/engine/modules/gguf.h:18-27; vendored codecs under
src/kernels/cpu/gguf/ggml): little-endian, fp16 scales.
  Q8_0  32 values : f16 d, int8 q[32]                                   x = d * q
  Q4_0  32 values : f16 d, 16 bytes (low nibble = first half)            x = d * (q - 8)
  Q4_K 256 values : f16 d, f16 dmin, 12 bytes of 6-bit (scale, min) x 8, 128 bytes   x = d*sc*q - dmin*m
  Q6_K 256 values : 128 bytes low 4 bits, 64 bytes high 2 bits, int8 sc[16], f16 d    x = d * sc * (q - 32)
CPU linear semantics (src/backend/cpu/linear_gguf.cpp:65-113): the activation row is quantised to Q8_0,
each block contributes an integer dot product scaled by both block scales, accumulated in fp32.
"""
from __future__ import annotations

import torch

GGML_F32, GGML_F16, GGML_Q4_0, GGML_Q8_0, GGML_Q4_K, GGML_Q6_K, GGML_BF16 = 0, 1, 2, 8, 12, 14, 30
BLOCK = {GGML_Q4_0: (32, 18), GGML_Q8_0: (32, 34), GGML_Q4_K: (256, 144), GGML_Q6_K: (256, 210),
         GGML_F32: (1, 4), GGML_F16: (1, 2), GGML_BF16: (1, 2)}
NAMES = {GGML_F32: "F32", GGML_F16: "F16", GGML_Q4_0: "Q4_0", GGML_Q8_0: "Q8_0", GGML_Q4_K: "Q4_K",
         GGML_Q6_K: "Q6_K", GGML_BF16: "BF16"}


def _f16(raw: torch.Tensor) -> torch.Tensor:
    """[..., 2] uint8 -> float32 of the little-endian fp16."""
    return raw.contiguous().view(torch.float16).float().squeeze(-1)


def _f16_bytes(x: torch.Tensor) -> torch.Tensor:
    return x.to(torch.float16).contiguous().view(torch.uint8).reshape(*x.shape, 2)


def row_bytes(ggml_type: int, k: int) -> int:
    n, b = BLOCK[ggml_type]
    assert k % n == 0
    return k // n * b


# ------------------------------------------------------------------------------------------------ Q8_0
def quantize_q8_0(x: torch.Tensor) -> torch.Tensor:
    """[rows, K] -> uint8 [rows, K/32*34]"""
    rows, K = x.shape
    xb = x.float().reshape(rows, K // 32, 32)
    d = (xb.abs().amax(-1) / 127.0).to(torch.float16)
    df = d.float()
    inv = torch.where(df > 0, 1.0 / df, torch.zeros_like(df))
    q = torch.round(xb * inv[..., None]).clamp(-127, 127).to(torch.int8)
    out = torch.cat([_f16_bytes(d), q.view(torch.uint8)], dim=-1)
    return out.reshape(rows, -1)


def dequantize_q8_0(raw: torch.Tensor, K: int) -> torch.Tensor:
    rows = raw.shape[0]
    b = raw.reshape(rows, K // 32, 34)
    d = _f16(b[..., :2])
    q = b[..., 2:].contiguous().view(torch.int8).float()
    return (q * d[..., None]).reshape(rows, K)


def split_q8_0(raw: torch.Tensor, K: int):
    """-> (d float32 [rows, K/32], q int8 [rows, K/32, 32])"""
    rows = raw.shape[0]
    b = raw.reshape(rows, K // 32, 34)
    return _f16(b[..., :2]), b[..., 2:].contiguous().view(torch.int8)


# ------------------------------------------------------------------------------------------------ Q4_0
def quantize_q4_0(x: torch.Tensor) -> torch.Tensor:
    rows, K = x.shape
    xb = x.float().reshape(rows, K // 32, 32)
    idx = xb.abs().argmax(-1, keepdim=True)
    mx = xb.gather(-1, idx).squeeze(-1)
    d = (mx / -8.0).to(torch.float16)
    df = d.float()
    inv = torch.where(df != 0, 1.0 / df, torch.zeros_like(df))
    q = (xb * inv[..., None] + 8.5).floor().clamp(0, 15).to(torch.uint8)
    packed = q[..., :16] | (q[..., 16:] << 4)
    return torch.cat([_f16_bytes(d), packed], dim=-1).reshape(rows, -1)


def dequantize_q4_0(raw: torch.Tensor, K: int) -> torch.Tensor:
    rows = raw.shape[0]
    b = raw.reshape(rows, K // 32, 18)
    d = _f16(b[..., :2])
    qs = b[..., 2:]
    q = torch.cat([qs & 15, qs >> 4], dim=-1).float() - 8.0
    return (q * d[..., None]).reshape(rows, K)


# ------------------------------------------------------------------------------------------------ Q4_K
def _unpack_scales_k4(sc: torch.Tensor):
    """sc uint8 [..., 12] -> (scale [..., 8], min [..., 8]) as int64."""
    s = sc.long()
    lo_sc, lo_m = s[..., 0:4] & 63, s[..., 4:8] & 63
    hi_sc = (s[..., 8:12] & 15) | ((s[..., 0:4] >> 6) << 4)
    hi_m = (s[..., 8:12] >> 4) | ((s[..., 4:8] >> 6) << 4)
    return torch.cat([lo_sc, hi_sc], -1), torch.cat([lo_m, hi_m], -1)


def _pack_scales_k4(scale: torch.Tensor, mn: torch.Tensor) -> torch.Tensor:
    s, m = scale.long(), mn.long()
    out = torch.zeros(*s.shape[:-1], 12, dtype=torch.int64, device=s.device)
    out[..., 0:4] = (s[..., 0:4] & 63) | ((s[..., 4:8] >> 4) << 6)
    out[..., 4:8] = (m[..., 0:4] & 63) | ((m[..., 4:8] >> 4) << 6)
    out[..., 8:12] = (s[..., 4:8] & 15) | ((m[..., 4:8] & 15) << 4)
    return out.to(torch.uint8)


def dequantize_q4_k(raw: torch.Tensor, K: int) -> torch.Tensor:
    rows = raw.shape[0]
    b = raw.reshape(rows, K // 256, 144)
    d, dmin = _f16(b[..., 0:2]), _f16(b[..., 2:4])
    sc, mn = _unpack_scales_k4(b[..., 4:16])
    qs = b[..., 16:].reshape(rows, K // 256, 4, 32)           # 4 groups of 32 bytes: low nibble = sub-block 2g
    q = torch.stack([qs & 15, qs >> 4], dim=3).reshape(rows, K // 256, 8, 32).float()
    x = q * (d[..., None] * sc.float())[..., None] - (dmin[..., None] * mn.float())[..., None]
    return x.reshape(rows, K)


def quantize_q4_k(x: torch.Tensor) -> torch.Tensor:
    """Min/max affine quantiser per 32-value sub-block with 6-bit scales and mins (no iterative refinement)."""
    rows, K = x.shape
    xb = x.float().reshape(rows, K // 256, 8, 32)
    mn = (-xb.amin(-1)).clamp(min=0)                          # stored min is subtracted: x = s*q - m
    mx = xb.amax(-1)
    scale = ((mx + mn) / 15.0).clamp(min=0)
    d = (scale.amax(-1) / 63.0).to(torch.float16)
    dmin = (mn.amax(-1) / 63.0).to(torch.float16)
    df, dmf = d.float(), dmin.float()
    sc = torch.where(df[..., None] > 0, torch.round(scale / df[..., None].clamp(min=1e-30)), torch.zeros_like(scale)).clamp(0, 63)
    mq = torch.where(dmf[..., None] > 0, torch.round(mn / dmf[..., None].clamp(min=1e-30)), torch.zeros_like(mn)).clamp(0, 63)
    s_eff, m_eff = df[..., None] * sc, dmf[..., None] * mq
    inv = torch.where(s_eff > 0, 1.0 / s_eff.clamp(min=1e-30), torch.zeros_like(s_eff))
    q = torch.round((xb + m_eff[..., None]) * inv[..., None]).clamp(0, 15).to(torch.uint8)
    q = q.reshape(rows, K // 256, 4, 2, 32)
    packed = (q[:, :, :, 0] | (q[:, :, :, 1] << 4)).reshape(rows, K // 256, 128)
    out = torch.cat([_f16_bytes(d), _f16_bytes(dmin), _pack_scales_k4(sc, mq), packed], dim=-1)
    return out.reshape(rows, -1)


# ------------------------------------------------------------------------------------------------ Q6_K
def dequantize_q6_k(raw: torch.Tensor, K: int) -> torch.Tensor:
    rows = raw.shape[0]
    b = raw.reshape(rows, K // 256, 210)
    ql = b[..., 0:128].reshape(rows, K // 256, 2, 64).long()
    qh = b[..., 128:192].reshape(rows, K // 256, 2, 32).long()
    sc = b[..., 192:208].contiguous().view(torch.int8).reshape(rows, K // 256, 2, 8).float()
    d = _f16(b[..., 208:210])
    q1 = ((ql[..., 0:32] & 15) | (((qh >> 0) & 3) << 4)) - 32
    q2 = ((ql[..., 32:64] & 15) | (((qh >> 2) & 3) << 4)) - 32
    q3 = ((ql[..., 0:32] >> 4) | (((qh >> 4) & 3) << 4)) - 32
    q4 = ((ql[..., 32:64] >> 4) | (((qh >> 6) & 3) << 4)) - 32
    q = torch.stack([q1, q2, q3, q4], dim=3).float()          # [rows, nb, 2 halves, 4 quarters, 32]
    idx = torch.arange(32, device=raw.device) // 16            # scale index inside a quarter
    s = sc.reshape(rows, K // 256, 2, 4, 2)[..., idx]          # sc[is + 2*quarter]
    return (q * s * d[..., None, None, None]).reshape(rows, K)


def quantize_q6_k(x: torch.Tensor) -> torch.Tensor:
    rows, K = x.shape
    xb = x.float().reshape(rows, K // 256, 16, 16)
    amax_idx = xb.abs().argmax(-1, keepdim=True)
    mxv = xb.gather(-1, amax_idx).squeeze(-1)
    scale = mxv / -32.0                                        # per 16 values
    big_idx = scale.abs().argmax(-1, keepdim=True)
    d = (scale.gather(-1, big_idx).squeeze(-1) / -128.0).to(torch.float16)
    df = d.float()
    sc = torch.where(df[..., None] != 0, torch.round(scale / df[..., None]), torch.zeros_like(scale)).clamp(-128, 127)
    eff = df[..., None] * sc
    inv = torch.where(eff != 0, 1.0 / eff, torch.zeros_like(eff))
    q = (torch.round(xb * inv[..., None]).clamp(-32, 31) + 32).long().reshape(rows, K // 256, 2, 4, 32)
    ql = torch.zeros(rows, K // 256, 2, 64, dtype=torch.int64, device=x.device)
    qh = torch.zeros(rows, K // 256, 2, 32, dtype=torch.int64, device=x.device)
    ql[..., 0:32] = (q[..., 0, :] & 15) | ((q[..., 2, :] & 15) << 4)
    ql[..., 32:64] = (q[..., 1, :] & 15) | ((q[..., 3, :] & 15) << 4)
    for j in range(4):
        qh |= (q[..., j, :] >> 4) << (2 * j)
    scb = sc.reshape(rows, K // 256, 2, 4, 2).permute(0, 1, 2, 4, 3)      # -> sc[half][is][quarter]
    scb = sc.reshape(rows, K // 256, 2, 4, 2)                              # stored as sc[half*8 + quarter*2 + is]
    out = torch.cat([ql.reshape(rows, K // 256, 128).to(torch.uint8), qh.reshape(rows, K // 256, 64).to(torch.uint8),
                     scb.reshape(rows, K // 256, 16).to(torch.int8).view(torch.uint8), _f16_bytes(d)], dim=-1)
    return out.reshape(rows, -1)


# ------------------------------------------------------------------------------------------------ dispatch
def quantize(x: torch.Tensor, ggml_type: int) -> torch.Tensor:
    if ggml_type == GGML_Q8_0:
        return quantize_q8_0(x)
    if ggml_type == GGML_Q4_0:
        return quantize_q4_0(x)
    if ggml_type == GGML_Q4_K:
        return quantize_q4_k(x)
    if ggml_type == GGML_Q6_K:
        return quantize_q6_k(x)
    if ggml_type == GGML_F16:
        return x.to(torch.float16).contiguous().view(torch.uint8).reshape(x.shape[0], -1)
    if ggml_type == GGML_BF16:
        return x.to(torch.bfloat16).contiguous().view(torch.uint8).reshape(x.shape[0], -1)
    if ggml_type == GGML_F32:
        return x.float().contiguous().view(torch.uint8).reshape(x.shape[0], -1)
    raise ValueError(f"unsupported ggml type {ggml_type}")


def dequantize(raw: torch.Tensor, ggml_type: int, K: int) -> torch.Tensor:
    if ggml_type == GGML_Q8_0:
        return dequantize_q8_0(raw, K)
    if ggml_type == GGML_Q4_0:
        return dequantize_q4_0(raw, K)
    if ggml_type == GGML_Q4_K:
        return dequantize_q4_k(raw, K)
    if ggml_type == GGML_Q6_K:
        return dequantize_q6_k(raw, K)
    rows = raw.shape[0]
    if ggml_type == GGML_F16:
        return raw.contiguous().view(torch.float16).reshape(rows, K).float()
    if ggml_type == GGML_BF16:
        return raw.contiguous().view(torch.bfloat16).reshape(rows, K).float()
    if ggml_type == GGML_F32:
        return raw.contiguous().view(torch.float32).reshape(rows, K)
    raise ValueError(f"unsupported ggml type {ggml_type}")


def linear_q8_0_cpu_semantics(x: torch.Tensor, w_raw: torch.Tensor, K: int) -> torch.Tensor:
    """y = x W^T with the CPU backend's arithmetic: activation rows quantised to Q8_0, integer block dots."""
    xq = quantize_q8_0(x.float())
    dx, qx = split_q8_0(xq, K)
    dw, qw = split_q8_0(w_raw, K)
    dots = torch.einsum("mbk,nbk->mnb", qx.float(), qw.float())        # exact: |sum| < 2^24
    return torch.einsum("mnb,mb,nb->mn", dots, dx, dw)
