"""The codebook ("IQ") block formats of GGUF in vectorised PyTorch: IQ1_S, IQ1_M, IQ2_XXS, IQ2_XS, IQ2_S, IQ3_XXS, IQ3_S.

Every format stores, per group of 8 (IQ1 / IQ2) or 4 (IQ3) weights, an index into a fixed grid of small integer
vectors, plus sign bits (IQ2 / IQ3) or a shared +-1/8 shift (IQ1), and 3- or 4-bit scales per 16 or 32 weights under one
fp16 scale per 256-weight super-block. The grids are format constants of ggml (its ``iq2xxs_grid`` .. ``iq1s_grid`` and
``ksigns_iq2xs`` tables); they are kept as one binary file beside this module, ``data/iq_grids.bin``:

    offset      0  ksigns   [128]      u8   sign byte of a 7-bit sign index (bit 7 = parity of the other seven)
              128  iq2xxs   [256][8]   u8
             2176  iq2xs    [512][8]   u8
             6272  iq2s     [1024][8]  u8
            14464  iq3xxs   [256][4]   u8
            15488  iq3s     [512][4]   u8
            17536  iq1s     [2048][8]  i8   (values -1, 0, 1)

The same bytes are uploaded once per device for the CUDA decoders (csrc/cuda/gguf_gemv.cu). Block layouts (bytes):
    IQ2_XXS  66: f16 d | 8 x { 4 grid bytes, u32: 4 x 7-bit sign index + 4-bit scale }
    IQ2_XS   74: f16 d | 32 x u16 { 9-bit grid index, 7-bit sign index } | 8 x { 2 x 4-bit scale }
    IQ2_S    82: f16 d | 32 grid low bytes | 32 sign bytes | 8 x qh (2 high index bits per group) | 8 scale bytes
    IQ3_XXS  98: f16 d | 64 grid bytes (two per group of 8) | 8 x u32 { 4 x 7-bit sign index, 4-bit scale }
    IQ3_S   110: f16 d | 64 grid low bytes | 8 qh bytes (ninth index bit) | 32 sign bytes | 4 scale bytes
    IQ1_S    50: f16 d | 32 grid low bytes | 8 x u16 { 4 x 3 high index bits, 3-bit scale, shift sign }
    IQ1_M    56: 32 grid low bytes | 16 qh bytes { 3 high bits + shift sign, per group } | 4 x u16 { 4 x 3-bit scale, 4 bits
                 of the fp16 super-block scale }
Reference: src/kernels/cpu/gguf/ggml/ggml-common.h (block structs and tables), ggml-quants.c (row dequantisers),
src/kernels/cuda/gguf/gguf_moe.cu:497-523 (IQ1 decode on the device).
"""
from __future__ import annotations

import os

import numpy as np
import torch

GGML_IQ2_XXS, GGML_IQ2_XS, GGML_IQ3_XXS, GGML_IQ1_S, GGML_IQ3_S, GGML_IQ2_S, GGML_IQ1_M = 16, 17, 18, 19, 21, 22, 29
IQ_BLOCK = {GGML_IQ2_XXS: (256, 66), GGML_IQ2_XS: (256, 74), GGML_IQ2_S: (256, 82), GGML_IQ3_XXS: (256, 98),
            GGML_IQ3_S: (256, 110), GGML_IQ1_S: (256, 50), GGML_IQ1_M: (256, 56)}
IQ_NAMES = {GGML_IQ2_XXS: "IQ2_XXS", GGML_IQ2_XS: "IQ2_XS", GGML_IQ2_S: "IQ2_S", GGML_IQ3_XXS: "IQ3_XXS",
            GGML_IQ3_S: "IQ3_S", GGML_IQ1_S: "IQ1_S", GGML_IQ1_M: "IQ1_M"}
IQ1_DELTA = 0.125
GRID_FILE = os.path.join(os.path.dirname(os.path.abspath(__file__)), "data", "iq_grids.bin")
OFF_SIGNS, OFF_2XXS, OFF_2XS, OFF_2S, OFF_3XXS, OFF_3S, OFF_1S, GRID_BYTES = 0, 128, 2176, 6272, 14464, 15488, 17536, 33920

_tables: dict = {}


def grid_blob() -> bytes:
    with open(GRID_FILE, "rb") as f:
        blob = f.read()
    assert len(blob) == GRID_BYTES
    return blob


def tables(device="cpu") -> dict:
    """The grids as tensors on ``device``: ksigns [128] int64, grids [n, 8 or 4] float32."""
    key = str(device)
    t = _tables.get(key)
    if t is None:
        raw = np.frombuffer(grid_blob(), dtype=np.uint8)

        def u8(lo, n, w):
            return torch.from_numpy(raw[lo:lo + n * w].astype(np.float32).reshape(n, w)).to(device)
        t = {"signs": torch.from_numpy(raw[:128].astype(np.int64)).to(device),
             "2xxs": u8(OFF_2XXS, 256, 8), "2xs": u8(OFF_2XS, 512, 8), "2s": u8(OFF_2S, 1024, 8),
             "3xxs": u8(OFF_3XXS, 256, 4), "3s": u8(OFF_3S, 512, 4),
             "1s": torch.from_numpy(raw[OFF_1S:].view(np.int8).astype(np.float32).reshape(2048, 8)).to(device)}
        _tables[key] = t
    return t


def _blocks(raw: torch.Tensor, K: int, bs: int) -> torch.Tensor:
    rows = raw.shape[0]
    return raw.reshape(rows, K // 256, bs).to(torch.int64)


def _f16(lo: torch.Tensor, hi: torch.Tensor) -> torch.Tensor:
    """Two bytes (low, high) -> the fp16 value they encode, as fp32."""
    v = lo | (hi << 8)
    v = torch.where(v >= 32768, v - 65536, v)
    return v.to(torch.int16).view(torch.float16).float()


def _u16(b: torch.Tensor) -> torch.Tensor:
    """[..., 2n] bytes -> [..., n] little-endian 16-bit values."""
    return b[..., 0::2] | (b[..., 1::2] << 8)


def _u32(b: torch.Tensor) -> torch.Tensor:
    return b[..., 0::4] | (b[..., 1::4] << 8) | (b[..., 2::4] << 16) | (b[..., 3::4] << 24)


def _apply_signs(vals: torch.Tensor, sign_byte: torch.Tensor) -> torch.Tensor:
    """vals [..., 8], sign_byte [...]: bit j set -> element j negated."""
    bits = (sign_byte.unsqueeze(-1) >> torch.arange(8, device=vals.device)) & 1
    return vals * (1.0 - 2.0 * bits.float())


def dequantize_iq2_xxs(raw, K):
    T = tables(raw.device)
    b = _blocks(raw, K, 66)
    d = _f16(b[..., 0], b[..., 1])
    q = b[..., 2:].reshape(*b.shape[:2], 8, 8)                      # per 32 weights: 4 grid bytes + u32
    aux = _u32(q[..., 4:8]).squeeze(-1)                              # [rows, nb, 8]
    db = d[..., None] * (0.5 + (aux >> 28).float()) * 0.25
    sidx = (aux.unsqueeze(-1) >> (7 * torch.arange(4, device=raw.device))) & 127
    vals = _apply_signs(T["2xxs"][q[..., :4]], T["signs"][sidx])     # [rows, nb, 8, 4, 8]
    return (vals * db[..., None, None]).reshape(raw.shape[0], K)


def dequantize_iq2_xs(raw, K):
    T = tables(raw.device)
    b = _blocks(raw, K, 74)
    d = _f16(b[..., 0], b[..., 1])
    q = _u16(b[..., 2:66]).reshape(*b.shape[:2], 8, 4)
    sc = b[..., 66:74]
    db = d[..., None, None] * (0.5 + torch.stack([sc & 15, sc >> 4], -1).float()) * 0.25      # [rows, nb, 8, 2]
    vals = _apply_signs(T["2xs"][q & 511], T["signs"][q >> 9])
    return (vals * db.repeat_interleave(2, -1)[..., None]).reshape(raw.shape[0], K)


def dequantize_iq2_s(raw, K):
    T = tables(raw.device)
    b = _blocks(raw, K, 82)
    d = _f16(b[..., 0], b[..., 1])
    lo = b[..., 2:34].reshape(*b.shape[:2], 8, 4)
    sg = b[..., 34:66].reshape(*b.shape[:2], 8, 4)
    qh = b[..., 66:74]
    sc = b[..., 74:82]
    l = torch.arange(4, device=raw.device)
    idx = lo | ((qh.unsqueeze(-1) << (8 - 2 * l)) & 0x300)
    db = d[..., None, None] * (0.5 + torch.stack([sc & 15, sc >> 4], -1).float()) * 0.25
    vals = _apply_signs(T["2s"][idx], sg)
    return (vals * db.repeat_interleave(2, -1)[..., None]).reshape(raw.shape[0], K)


def dequantize_iq3_xxs(raw, K):
    T = tables(raw.device)
    b = _blocks(raw, K, 98)
    d = _f16(b[..., 0], b[..., 1])
    q = b[..., 2:66].reshape(*b.shape[:2], 8, 4, 2)                  # two 4-value grid entries per group of 8
    aux = _u32(b[..., 66:98])                                        # [rows, nb, 8]
    db = d[..., None] * (0.5 + (aux >> 28).float()) * 0.5
    sidx = (aux.unsqueeze(-1) >> (7 * torch.arange(4, device=raw.device))) & 127
    vals = T["3xxs"][q].reshape(*b.shape[:2], 8, 4, 8)
    vals = _apply_signs(vals, T["signs"][sidx])
    return (vals * db[..., None, None]).reshape(raw.shape[0], K)


def dequantize_iq3_s(raw, K):
    T = tables(raw.device)
    b = _blocks(raw, K, 110)
    d = _f16(b[..., 0], b[..., 1])
    lo = b[..., 2:66].reshape(*b.shape[:2], 8, 4, 2)
    qh = b[..., 66:74]
    sg = b[..., 74:106].reshape(*b.shape[:2], 8, 4)
    sc = b[..., 106:110]
    l = torch.arange(4, device=raw.device)
    hi0 = (qh.unsqueeze(-1) << (8 - 2 * l)) & 256
    hi1 = (qh.unsqueeze(-1) << (7 - 2 * l)) & 256
    idx = lo | torch.stack([hi0, hi1], -1)
    nib = torch.stack([sc & 15, sc >> 4], -1).reshape(*b.shape[:2], 8)
    db = d[..., None] * (1.0 + 2.0 * nib.float())
    vals = _apply_signs(T["3s"][idx].reshape(*b.shape[:2], 8, 4, 8), sg)
    return (vals * db[..., None, None]).reshape(raw.shape[0], K)


def dequantize_iq1_s(raw, K):
    T = tables(raw.device)
    b = _blocks(raw, K, 50)
    d = _f16(b[..., 0], b[..., 1])
    lo = b[..., 2:34].reshape(*b.shape[:2], 8, 4)
    qh = _u16(b[..., 34:50])                                         # [rows, nb, 8]
    dl = d[..., None] * (2.0 * ((qh >> 12) & 7).float() + 1.0)
    delta = torch.where((qh & 0x8000) != 0, -IQ1_DELTA, IQ1_DELTA)
    idx = lo | (((qh.unsqueeze(-1) >> (3 * torch.arange(4, device=raw.device))) & 7) << 8)
    vals = T["1s"][idx] + delta[..., None, None]
    return (vals * dl[..., None, None]).reshape(raw.shape[0], K)


def dequantize_iq1_m(raw, K):
    T = tables(raw.device)
    b = _blocks(raw, K, 56)
    lo = b[..., 0:32].reshape(*b.shape[:2], 8, 4)
    qh = b[..., 32:48].reshape(*b.shape[:2], 8, 2)
    sc = _u16(b[..., 48:56])                                         # [rows, nb, 4]
    bits = (sc[..., 0] >> 12) | ((sc[..., 1] >> 8) & 0x00F0) | ((sc[..., 2] >> 4) & 0x0F00) | (sc[..., 3] & 0xF000)
    d = _f16(bits & 0xFF, bits >> 8)
    ib = torch.arange(8, device=raw.device)
    s16 = sc[..., ib // 2]                                           # [rows, nb, 8]
    dl1 = d[..., None] * (2.0 * ((s16 >> (6 * (ib % 2))) & 7).float() + 1.0)
    dl2 = d[..., None] * (2.0 * ((s16 >> (6 * (ib % 2) + 3)) & 7).float() + 1.0)
    q0, q1 = qh[..., 0], qh[..., 1]
    hi = torch.stack([(q0 << 8) & 0x700, (q0 << 4) & 0x700, (q1 << 8) & 0x700, (q1 << 4) & 0x700], -1)
    neg = torch.stack([q0 & 0x08, q0 & 0x80, q1 & 0x08, q1 & 0x80], -1) != 0
    delta = torch.where(neg, -IQ1_DELTA, IQ1_DELTA)
    dl = torch.stack([dl1, dl1, dl2, dl2], -1)
    vals = T["1s"][lo | hi] + delta[..., None]
    return (vals * dl[..., None]).reshape(raw.shape[0], K)


IQ_DEQUANT = {GGML_IQ2_XXS: dequantize_iq2_xxs, GGML_IQ2_XS: dequantize_iq2_xs, GGML_IQ2_S: dequantize_iq2_s,
              GGML_IQ3_XXS: dequantize_iq3_xxs, GGML_IQ3_S: dequantize_iq3_s, GGML_IQ1_S: dequantize_iq1_s,
              GGML_IQ1_M: dequantize_iq1_m}


def random_iq_blocks(ggml_type: int, rows: int, K: int, seed: int = 0, amp: float = 0.02, device="cpu") -> torch.Tensor:
    """Synthetic packed rows: uniformly random payload bytes (every bit pattern of the payload is a valid block) with a
    small finite super-block scale."""
    n, bs = IQ_BLOCK[ggml_type]
    g = torch.Generator(device=device).manual_seed(seed)
    nb = K // n
    raw = torch.randint(0, 256, (rows, nb, bs), dtype=torch.uint8, generator=g, device=device)
    v = ((torch.rand(rows, nb, generator=g, device=device) * 0.9 + 0.1) * amp).to(torch.float16).view(torch.int16).to(torch.int32) & 0xFFFF
    if ggml_type == GGML_IQ1_M:
        # the fp16 scale is spread over the top nibbles of the four 16-bit scale words
        for i in range(4):
            nib = (v >> (4 * i)) & 15
            hi = raw[..., 48 + 2 * i + 1].to(torch.int32)
            raw[..., 48 + 2 * i + 1] = ((hi & 0x0F) | (nib << 4)).to(torch.uint8)
    else:
        raw[..., 0] = (v & 0xFF).to(torch.uint8)
        raw[..., 1] = (v >> 8).to(torch.uint8)
    return raw.reshape(rows, -1)
