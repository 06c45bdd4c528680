"""GGUF block formats in vectorised PyTorch (CPU or GPU): the oracle of the fused dequant mat-vec kernels,
the quantise-at-write path of the synthetic checkpoint writers, and the CPU linear semantics.

Block layouts are the ggml ones the reference consumes (inc/engine/modules/gguf.h:18-27; vendored codecs under
src/kernels/cpu/gguf/ggml): little-endian, fp16 scales.
  Q8_0  32 values : f16 d, int8 q[32]                                   x = d * q
  Q4_0  32 values : f16 d, 16 bytes (low nibble = first half)            x = d * (q - 8)
  Q4_K 256 values : f16 d, f16 dmin, 12 bytes of 6-bit (scale, min) x 8, 128 bytes   x = d*sc*q - dmin*m
  Q6_K 256 values : 128 bytes low 4 bits, 64 bytes high 2 bits, int8 sc[16], f16 d    x = d * sc * (q - 32)
  Q4_1 / Q5_0 / Q5_1 (32 values; f16 d [, f16 m] [, 32 high bits], 16 bytes of nibbles)
  Q2_K (16 x {4-bit scale, 4-bit min}, 64 bytes of 2-bit values, d, dmin), Q3_K (32 bytes of high bits, 64 bytes of
  2-bit values, 16 packed 6-bit scales, d), Q5_K (Q4_K plus 32 bytes of high bits)
  IQ4_NL (Q4_0 container over 16 non-uniform levels), IQ4_XS (256 values, 8 six-bit sub-block scales over the levels)
  IQ1_S, IQ1_M, IQ2_XXS, IQ2_XS, IQ2_S, IQ3_XXS, IQ3_S: codebook formats, see quant/gguf_iq.py
Read-only formats (no quantiser): a synthetic block is random bytes with finite fp16 fields (`random_blocks`).
CPU linear semantics (src/backend/cpu/linear_gguf.cpp:65-113): the activation row is quantised to Q8_0,
each block contributes an integer dot product scaled by both block scales, accumulated in fp32.
"""
from __future__ import annotations

import torch

GGML_F32, GGML_F16, GGML_Q4_0, GGML_Q8_0, GGML_Q4_K, GGML_Q6_K, GGML_BF16 = 0, 1, 2, 8, 12, 14, 30
GGML_Q4_1, GGML_Q5_0, GGML_Q5_1, GGML_Q2_K, GGML_Q3_K, GGML_Q5_K, GGML_IQ4_NL, GGML_IQ4_XS = 3, 6, 7, 10, 11, 13, 20, 23
BLOCK = {GGML_Q4_0: (32, 18), GGML_Q8_0: (32, 34), GGML_Q4_K: (256, 144), GGML_Q6_K: (256, 210),
         GGML_Q4_1: (32, 20), GGML_Q5_0: (32, 22), GGML_Q5_1: (32, 24), GGML_Q2_K: (256, 84), GGML_Q3_K: (256, 110),
         GGML_Q5_K: (256, 176), GGML_IQ4_NL: (32, 18), GGML_IQ4_XS: (256, 136),
         GGML_F32: (1, 4), GGML_F16: (1, 2), GGML_BF16: (1, 2)}
NAMES = {GGML_F32: "F32", GGML_F16: "F16", GGML_Q4_0: "Q4_0", GGML_Q8_0: "Q8_0", GGML_Q4_K: "Q4_K",
         GGML_Q6_K: "Q6_K", GGML_BF16: "BF16", GGML_Q4_1: "Q4_1", GGML_Q5_0: "Q5_0", GGML_Q5_1: "Q5_1",
         GGML_Q2_K: "Q2_K", GGML_Q3_K: "Q3_K", GGML_Q5_K: "Q5_K", GGML_IQ4_NL: "IQ4_NL", GGML_IQ4_XS: "IQ4_XS"}
# byte offsets of the fp16 fields of one block (what a synthetic block must keep finite)
F16_FIELDS = {GGML_Q4_0: (0,), GGML_Q8_0: (0,), GGML_Q4_1: (0, 2), GGML_Q5_0: (0,), GGML_Q5_1: (0, 2),
              GGML_Q2_K: (80, 82), GGML_Q3_K: (108,), GGML_Q4_K: (0, 2), GGML_Q5_K: (0, 2), GGML_Q6_K: (208,),
              GGML_IQ4_NL: (0,), GGML_IQ4_XS: (0,)}
# the 16 non-uniform levels of the IQ4 formats
IQ4_LEVELS = (-127, -104, -83, -65, -49, -35, -22, -10, 1, 13, 25, 38, 53, 69, 89, 113)


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



# ------------------------------------------------------------------------------------------------ 32-value formats
def _nib(qs):
    return torch.cat([qs & 15, qs >> 4], dim=-1).long()


def _high_bits32(qh: torch.Tensor) -> torch.Tensor:
    """[..., 4] uint8 (little-endian 32-bit word) -> [..., 32] the bits, element j = bit j."""
    bits = (qh.long()[..., :, None] >> torch.arange(8, device=qh.device)) & 1
    return bits.reshape(*qh.shape[:-1], 32)


def dequantize_q4_1(raw, K):
    rows = raw.shape[0]
    b = raw.reshape(rows, K // 32, 20)
    d, m = _f16(b[..., 0:2]), _f16(b[..., 2:4])
    return (_nib(b[..., 4:]).float() * d[..., None] + m[..., None]).reshape(rows, K)


def quantize_q4_1(x):
    rows, K = x.shape
    xb = x.float().reshape(rows, K // 32, 32)
    mn, mx = xb.amin(-1), xb.amax(-1)
    d = ((mx - mn) / 15.0).to(torch.float16)
    m = mn.to(torch.float16)
    inv = torch.where(d.float() > 0, 1.0 / d.float().clamp(min=1e-30), torch.zeros_like(mn))
    q = torch.round((xb - m.float()[..., None]) * inv[..., None]).clamp(0, 15).to(torch.uint8)
    return torch.cat([_f16_bytes(d), _f16_bytes(m), q[..., :16] | (q[..., 16:] << 4)], -1).reshape(rows, -1)


def dequantize_q5_0(raw, K):
    rows = raw.shape[0]
    b = raw.reshape(rows, K // 32, 22)
    q = (_nib(b[..., 6:]) | (_high_bits32(b[..., 2:6]) << 4)) - 16
    return (q.float() * _f16(b[..., 0:2])[..., None]).reshape(rows, K)


def _pack_high32(h):
    """[..., 32] of 0/1 -> [..., 4] uint8."""
    w = (h.long().reshape(*h.shape[:-1], 4, 8) << torch.arange(8, device=h.device)).sum(-1)
    return w.to(torch.uint8)


def quantize_q5_0(x):
    rows, K = x.shape
    xb = x.float().reshape(rows, K // 32, 32)
    mxv = xb.gather(-1, xb.abs().argmax(-1, keepdim=True)).squeeze(-1)
    d = (mxv / -16.0).to(torch.float16)
    inv = torch.where(d.float() != 0, 1.0 / d.float(), torch.zeros_like(mxv))
    q = (torch.round(xb * inv[..., None]) + 16).clamp(0, 31).long()
    lo = (q & 15).to(torch.uint8)
    return torch.cat([_f16_bytes(d), _pack_high32(q >> 4), lo[..., :16] | (lo[..., 16:] << 4)], -1).reshape(rows, -1)


def dequantize_q5_1(raw, K):
    rows = raw.shape[0]
    b = raw.reshape(rows, K // 32, 24)
    q = _nib(b[..., 8:]) | (_high_bits32(b[..., 4:8]) << 4)
    return (q.float() * _f16(b[..., 0:2])[..., None] + _f16(b[..., 2:4])[..., None]).reshape(rows, K)


def quantize_q5_1(x):
    rows, K = x.shape
    xb = x.float().reshape(rows, K // 32, 32)
    mn, mx = xb.amin(-1), xb.amax(-1)
    d = ((mx - mn) / 31.0).to(torch.float16)
    m = mn.to(torch.float16)
    inv = torch.where(d.float() > 0, 1.0 / d.float().clamp(min=1e-30), torch.zeros_like(mn))
    q = torch.round((xb - m.float()[..., None]) * inv[..., None]).clamp(0, 31).long()
    lo = (q & 15).to(torch.uint8)
    return torch.cat([_f16_bytes(d), _f16_bytes(m), _pack_high32(q >> 4), lo[..., :16] | (lo[..., 16:] << 4)],
                     -1).reshape(rows, -1)


def dequantize_iq4_nl(raw, K):
    rows = raw.shape[0]
    b = raw.reshape(rows, K // 32, 18)
    lv = torch.tensor(IQ4_LEVELS, dtype=torch.float32, device=raw.device)
    return (lv[_nib(b[..., 2:])] * _f16(b[..., 0:2])[..., None]).reshape(rows, K)


def quantize_iq4_nl(x):
    rows, K = x.shape
    xb = x.float().reshape(rows, K // 32, 32)
    lv = torch.tensor(IQ4_LEVELS, dtype=torch.float32, device=x.device)
    mxv = xb.gather(-1, xb.abs().argmax(-1, keepdim=True)).squeeze(-1)
    d = (mxv / -127.0).to(torch.float16)
    inv = torch.where(d.float() != 0, 1.0 / d.float(), torch.zeros_like(mxv))
    q = ((xb * inv[..., None])[..., None] - lv).abs().argmin(-1).to(torch.uint8)
    return torch.cat([_f16_bytes(d), q[..., :16] | (q[..., 16:] << 4)], -1).reshape(rows, -1)


# ------------------------------------------------------------------------------------------------ more K-quants
def dequantize_q2_k(raw, K):
    rows, nb = raw.shape[0], K // 256
    b = raw.reshape(rows, nb, 84)
    sc = b[..., 0:16].long().reshape(rows, nb, 2, 4, 2)                 # [half][shift][16-value part]
    qs = b[..., 16:80].long().reshape(rows, nb, 2, 1, 32)
    d, dmin = _f16(b[..., 80:82]), _f16(b[..., 82:84])
    sh = (torch.arange(4, device=raw.device) * 2).reshape(1, 1, 1, 4, 1)
    q = ((qs >> sh) & 3).reshape(rows, nb, 2, 4, 2, 16).float()
    dl = (d[..., None, None, None] * (sc & 15).float())[..., None]
    ml = (dmin[..., None, None, None] * (sc >> 4).float())[..., None]
    return (dl * q - ml).reshape(rows, K)


def _scales_q3k(s12: torch.Tensor) -> torch.Tensor:
    """[..., 12] uint8 -> [..., 16] signed 6-bit scales (already minus 32)."""
    s = s12.long()
    lo = torch.cat([s[..., 0:8] & 15, s[..., 0:8] >> 4], -1)
    hi = torch.cat([(s[..., 8:12] >> (2 * i)) & 3 for i in range(4)], -1)
    return (lo | (hi << 4)) - 32


def dequantize_q3_k(raw, K):
    rows, nb = raw.shape[0], K // 256
    b = raw.reshape(rows, nb, 110)
    hm = b[..., 0:32].long().reshape(rows, nb, 1, 1, 32)
    qs = b[..., 32:96].long().reshape(rows, nb, 2, 1, 32)
    sc = _scales_q3k(b[..., 96:108]).reshape(rows, nb, 2, 4, 2).float()
    d = _f16(b[..., 108:110])
    sh = (torch.arange(4, device=raw.device) * 2).reshape(1, 1, 1, 4, 1)
    bit = torch.arange(8, device=raw.device).reshape(1, 1, 2, 4, 1)     # mask bit = half * 4 + shift index
    q = ((qs >> sh) & 3) - torch.where(((hm >> bit) & 1) == 1, 0, 4)
    q = q.reshape(rows, nb, 2, 4, 2, 16).float()
    return (q * (d[..., None, None, None] * sc)[..., None]).reshape(rows, K)


def dequantize_q5_k(raw, K):
    rows, nb = raw.shape[0], K // 256
    b = raw.reshape(rows, nb, 176)
    d, dmin = _f16(b[..., 0:2]), _f16(b[..., 2:4])
    sc, mn = _unpack_scales_k4(b[..., 4:16])
    qh = b[..., 16:48].long().reshape(rows, nb, 1, 32)
    qs = b[..., 48:].reshape(rows, nb, 4, 32)
    q = torch.stack([qs & 15, qs >> 4], dim=3).reshape(rows, nb, 8, 32).long()
    hb = (qh >> torch.arange(8, device=raw.device).reshape(1, 1, 8, 1)) & 1
    q = (q | (hb << 4)).float()
    x = q * (d[..., None] * sc.float())[..., None] - (dmin[..., None] * mn.float())[..., None]
    return x.reshape(rows, K)


def dequantize_iq4_xs(raw, K):
    rows, nb = raw.shape[0], K // 256
    b = raw.reshape(rows, nb, 136)
    d = _f16(b[..., 0:2])
    sh = b[..., 2].long() | (b[..., 3].long() << 8)
    sl = b[..., 4:8].long()
    ib = torch.arange(8, device=raw.device)
    ls = ((sl[..., ib // 2] >> (4 * (ib % 2))) & 15) | (((sh[..., None] >> (2 * ib)) & 3) << 4)
    lv = torch.tensor(IQ4_LEVELS, dtype=torch.float32, device=raw.device)
    q = lv[_nib(b[..., 8:].reshape(rows, nb, 8, 16))]
    return (q * (d[..., None] * (ls - 32).float())[..., None]).reshape(rows, K)


def random_blocks(ggml_type: int, rows: int, K: int, seed: int = 0, amp: float = 0.02, device="cpu") -> torch.Tensor:
    """Synthetic packed rows: uniformly random payload bytes, fp16 fields set to small finite values. ``device``: where
    the bytes are drawn (a CUDA device draws a large bank in place; the values then differ from the CPU stream)."""
    if ggml_type in IQ_TYPES:
        return _iq.random_iq_blocks(ggml_type, rows, K, seed, amp, device)
    n, bs = BLOCK[ggml_type]
    g = torch.Generator(device=device).manual_seed(seed)
    raw = torch.randint(0, 256, (rows, K // n, bs), dtype=torch.uint8, generator=g, device=device)
    for off in F16_FIELDS[ggml_type]:
        v = (torch.rand(rows, K // n, generator=g, device=device) * 0.9 + 0.1) * amp
        v = v * (torch.randint(0, 2, (rows, K // n), generator=g, device=device) * 2 - 1)
        raw[..., off:off + 2] = _f16_bytes(v)
    return raw.reshape(rows, -1)

# ------------------------------------------------------------------------------------------------ dispatch
_QUANT = {}
_DEQUANT = {}

def quantize(x: torch.Tensor, ggml_type: int) -> torch.Tensor:
    if ggml_type == GGML_Q8_0:
        return quantize_q8_0(x)
    if ggml_type == GGML_Q4_0:
        return quantize_q4_0(x)
    if ggml_type == GGML_Q4_K:
        return quantize_q4_k(x)
    if ggml_type == GGML_Q6_K:
        return quantize_q6_k(x)
    if ggml_type in _QUANT:
        return _QUANT[ggml_type](x)
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
    if ggml_type in _DEQUANT:
        return _DEQUANT[ggml_type](raw, K)
    rows = raw.shape[0]
    if ggml_type == GGML_F16:
        return raw.contiguous().view(torch.float16).reshape(rows, K).float()
    if ggml_type == GGML_BF16:
        return raw.contiguous().view(torch.bfloat16).reshape(rows, K).float()
    if ggml_type == GGML_F32:
        return raw.contiguous().view(torch.float32).reshape(rows, K)
    raise ValueError(f"unsupported ggml type {ggml_type}")


from . import gguf_iq as _iq          # noqa: E402  (the codebook formats live in their own module)

GGML_IQ2_XXS, GGML_IQ2_XS, GGML_IQ3_XXS, GGML_IQ1_S, GGML_IQ3_S, GGML_IQ2_S, GGML_IQ1_M = (
    _iq.GGML_IQ2_XXS, _iq.GGML_IQ2_XS, _iq.GGML_IQ3_XXS, _iq.GGML_IQ1_S, _iq.GGML_IQ3_S, _iq.GGML_IQ2_S, _iq.GGML_IQ1_M)
IQ_TYPES = frozenset(_iq.IQ_BLOCK)
BLOCK.update(_iq.IQ_BLOCK)
NAMES.update(_iq.IQ_NAMES)
_DEQUANT.update(_iq.IQ_DEQUANT)

_QUANT.update({GGML_Q4_1: quantize_q4_1, GGML_Q5_0: quantize_q5_0, GGML_Q5_1: quantize_q5_1,
               GGML_IQ4_NL: quantize_iq4_nl})
_DEQUANT.update({GGML_Q4_1: dequantize_q4_1, GGML_Q5_0: dequantize_q5_0, GGML_Q5_1: dequantize_q5_1,
                 GGML_IQ4_NL: dequantize_iq4_nl, GGML_Q2_K: dequantize_q2_k, GGML_Q3_K: dequantize_q3_k,
                 GGML_Q5_K: dequantize_q5_k, GGML_IQ4_XS: dequantize_iq4_xs})


def linear_q8_0_cpu_semantics(x: torch.Tensor, w_raw: torch.Tensor, K: int) -> torch.Tensor:
    """y = x W^T with the CPU backend's arithmetic: activation rows quantised to Q8_0, integer block dots."""
    xq = quantize_q8_0(x.float())
    dx, qx = split_q8_0(xq, K)
    dw, qw = split_q8_0(w_raw, K)
    dots = torch.einsum("mbk,nbk->mnb", qx.float(), qw.float())        # exact: |sum| < 2^24
    return torch.einsum("mnb,mb,nb->mn", dots, dx, dw)
