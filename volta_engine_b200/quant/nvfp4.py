"""NVFP4 codec in plain PyTorch (runs on CPU or GPU): the oracle for the CUDA kernels and the
quantise-at-load path.

Format (reference: inc/engine/quant/fp4_fp8.h:14-40, src/loader/nvfp4.cpp:36-57,261-300):
``value = e2m1(code) * e4m3(block_scale) * global_scale`` with one E4M3 scale per 16 consecutive k and
two codes per byte (even k in the low nibble).  The at-load quantiser picks, per block, the E4M3 scale
nearest ``amax/6`` and then the best of the +-2 neighbouring scale codes by squared error; the global
scale maps the largest block scale onto the E4M3 maximum (448).
"""
from __future__ import annotations

import torch

E2M1_VALUES = (0.0, 0.5, 1.0, 1.5, 2.0, 3.0, 4.0, 6.0)
_BOUNDS_GT = (0.25, 1.25, 2.5, 5.0)    # tie -> lower (even) code
_BOUNDS_GE = (0.75, 1.75, 3.5)         # tie -> upper (even) code


def e2m1_encode(x: torch.Tensor) -> torch.Tensor:
    """Round to the nearest E2M1 value (ties to the even code, saturating). Returns uint8 codes 0..15."""
    a = x.abs().float()
    code = torch.zeros_like(a, dtype=torch.uint8)
    for b in _BOUNDS_GT:
        code += (a > b).to(torch.uint8)
    for b in _BOUNDS_GE:
        code += (a >= b).to(torch.uint8)
    sign = (x < 0) | ((x == 0) & torch.signbit(x))
    return code | (sign.to(torch.uint8) << 3)


def e2m1_decode(code: torch.Tensor) -> torch.Tensor:
    lut = torch.tensor(E2M1_VALUES + tuple(-v for v in E2M1_VALUES), dtype=torch.float32, device=code.device)
    return lut[code.long() & 15]


def e4m3_encode(x: torch.Tensor) -> torch.Tensor:
    """float -> E4M3 (fn variant, saturating at 448) byte."""
    return x.float().clamp(-448.0, 448.0).to(torch.float8_e4m3fn).view(torch.uint8)


def e4m3_decode(b: torch.Tensor) -> torch.Tensor:
    return b.view(torch.float8_e4m3fn).float()


def pack_codes(codes: torch.Tensor) -> torch.Tensor:
    """[..., K] codes -> [..., K/2] bytes, even k in the low nibble."""
    return (codes[..., 0::2] | (codes[..., 1::2] << 4)).contiguous()


def unpack_codes(packed: torch.Tensor) -> torch.Tensor:
    lo = packed & 15
    hi = packed >> 4
    return torch.stack((lo, hi), dim=-1).flatten(-2)


def quantize_nvfp4(w: torch.Tensor, search: bool = True, global_scale: float | None = None):
    """Quantise ``w`` [N, K] (K % 16 == 0). Returns (packed u8 [N,K/2], scales u8 [N,K/16], gscale float)."""
    N, K = w.shape
    assert K % 16 == 0
    wf = w.float().reshape(N, K // 16, 16)
    amax = wf.abs().amax(dim=-1)
    if global_scale is None:
        gmax = float(amax.max().item()) if amax.numel() else 0.0
        global_scale = gmax / (6.0 * 448.0) if gmax > 0 else 1.0
    sc_code = e4m3_encode(amax / 6.0 / global_scale)
    if search:
        best_err = None
        best_code = sc_code.clone()
        base = sc_code.to(torch.int16)
        for delta in (0, -1, 1, -2, 2):
            cand = (base + delta).clamp(0, 126).to(torch.uint8)
            s = e4m3_decode(cand) * global_scale
            inv = torch.where(s > 0, 1.0 / s, torch.zeros_like(s))
            q = e2m1_decode(e2m1_encode(wf * inv[..., None]))
            err = ((q * s[..., None] - wf) ** 2).sum(-1)
            if best_err is None:
                best_err = err
            else:
                take = err < best_err
                best_err = torch.where(take, err, best_err)
                best_code = torch.where(take, cand, best_code)
        sc_code = best_code
    s = e4m3_decode(sc_code) * global_scale
    inv = torch.where(s > 0, 1.0 / s, torch.zeros_like(s))
    codes = e2m1_encode(wf * inv[..., None]).reshape(N, K)
    return pack_codes(codes), sc_code.contiguous(), float(global_scale)


def dequantize_nvfp4(packed: torch.Tensor, scales: torch.Tensor, gscale: float) -> torch.Tensor:
    """-> fp32 [N, K]"""
    N = packed.shape[0]
    vals = e2m1_decode(unpack_codes(packed)).reshape(N, -1, 16)
    return (vals * (e4m3_decode(scales) * gscale)[..., None]).reshape(N, -1)


def quantize_rows_nvfp4(x: torch.Tensor):
    """Activation rows [T, K] -> (packed, scales) with global scale 1 and scale = e4m3(amax/6) (no search)."""
    T, K = x.shape
    xf = x.float().reshape(T, K // 16, 16)
    sc = e4m3_encode(xf.abs().amax(-1) / 6.0)
    s = e4m3_decode(sc)
    inv = torch.where(s > 0, 1.0 / s, torch.zeros_like(s))
    codes = e2m1_encode(xf * inv[..., None]).reshape(T, K)
    return pack_codes(codes), sc.contiguous()


def scales_blocked_k128(scales: torch.Tensor) -> torch.Tensor:
    """[N, K/16] -> [N/128, K/128, 128, 8] contiguous: the per-stage scale tile of the W4A16 GEMM loader."""
    N, KB = scales.shape
    assert N % 128 == 0 and KB % 8 == 0
    return scales.reshape(N // 128, 128, KB // 8, 8).permute(0, 2, 1, 3).contiguous()


def scales_atoms_512(scales: torch.Tensor) -> torch.Tensor:
    """[R, K/16] -> [ceil(R/128), K/64, 512]: tensor-core scale atoms.

    Byte ``(r % 32) * 16 + (r // 32) * 4 + j`` of atom (rb, kg) holds the scale of row ``rb*128 + r`` and
    block ``kg*4 + j``; rows beyond R are zero.
    """
    R, KB = scales.shape
    assert KB % 4 == 0
    RB = (R + 127) // 128
    pad = torch.zeros(RB * 128, KB, dtype=scales.dtype, device=scales.device)
    pad[:R] = scales
    t = pad.reshape(RB, 4, 32, KB // 4, 4)          # rb, r//32, r%32, kg, j
    return t.permute(0, 3, 2, 1, 4).reshape(RB, KB // 4, 512).contiguous()


# ---------------------------------------------------------------------------------------------------
# Decode ("GV") layout: weights re-ordered at load time into the register order of the tensor-core
# mat-vec kernel. One 32-bit word per lane per 16x16 (rows x k) block holds that lane's 8 codes as four
# (first, second) pairs p = 0..3:
#     bits [3p+2 : 3p]      magnitude of the pair's first code     bit 12+p   its sign
#     bits [16+3p+2 : 16+3p] magnitude of the second code           bit 28+p   its sign
# so that ((W << 6) >> 3p) & 0x01C001C0 | (W << (3-p)) & 0x80008000 is the bf16x2 register holding
# code * 2^-126 (an E2M1 magnitude m placed at bf16 bits [8:6] is exactly m * 2^-126, subnormal included).
# Lane (g, t) of block kb owns rows g, g+8 and k = 16*kb + 4t .. 4t+3:
#     p0 = row g   (k+0, k+1)   p1 = row g+8 (k+0, k+1)   p2 = row g (k+2, k+3)   p3 = row g+8 (k+2, k+3)
# Words of 4 consecutive k blocks are adjacent, so a warp reads 512 contiguous bytes per 16 rows x 64 k.
# ---------------------------------------------------------------------------------------------------
def prepack_gv(packed: torch.Tensor, scales: torch.Tensor):
    """(packed [N,K/2], scales [N,K/16]) -> (Wg int32 [N/16, K/64, 32, 4], Sg uint8 [N/16, K/64, 16, 4])."""
    N, K = packed.shape[0], packed.shape[1] * 2
    assert N % 16 == 0 and K % 64 == 0
    codes = unpack_codes(packed).to(torch.int64)              # [N, K]
    c = codes.reshape(N // 16, 2, 8, K // 64, 4, 4, 4)         # rb, half(h), g, kg, kb, t, j (k = 16kb + 4t + j)
    mag, sgn = c & 7, (c >> 3) & 1
    word = torch.zeros(N // 16, 8, K // 64, 4, 4, dtype=torch.int64, device=packed.device)  # rb, g, kg, kb, t
    for p in range(4):
        h, j0 = p & 1, (p >> 1) * 2
        m0, s0 = mag[:, h, :, :, :, :, j0], sgn[:, h, :, :, :, :, j0]
        m1, s1 = mag[:, h, :, :, :, :, j0 + 1], sgn[:, h, :, :, :, :, j0 + 1]
        word |= (m0 << (3 * p)) | (s0 << (12 + p)) | (m1 << (16 + 3 * p)) | (s1 << (28 + p))
    # -> [rb, kg, lane = g*4 + t, kb]
    wg = word.permute(0, 2, 1, 4, 3).reshape(N // 16, K // 64, 32, 4)
    wg = torch.where(wg >= 2 ** 31, wg - 2 ** 32, wg).to(torch.int32).contiguous()
    sg = scales.reshape(N // 16, 16, K // 64, 4).permute(0, 2, 1, 3).contiguous()
    return wg, sg


def unpack_gv(wg: torch.Tensor, sg: torch.Tensor):
    """Inverse of :func:`prepack_gv` (test helper): -> (packed [N,K/2], scales [N,K/16])."""
    RB, KG = wg.shape[0], wg.shape[1]
    N, K = RB * 16, KG * 64
    w = wg.to(torch.int64) & 0xFFFFFFFF
    w = w.reshape(RB, KG, 8, 4, 4)                              # rb, kg, g, t, kb
    codes = torch.zeros(RB, 2, 8, KG, 4, 4, 4, dtype=torch.int64, device=wg.device)
    for p in range(4):
        h, j0 = p & 1, (p >> 1) * 2
        m0, s0 = (w >> (3 * p)) & 7, (w >> (12 + p)) & 1
        m1, s1 = (w >> (16 + 3 * p)) & 7, (w >> (28 + p)) & 1
        codes[:, h, :, :, :, :, j0] = (m0 | (s0 << 3)).permute(0, 2, 1, 4, 3)
        codes[:, h, :, :, :, :, j0 + 1] = (m1 | (s1 << 3)).permute(0, 2, 1, 4, 3)
    packed = pack_codes(codes.reshape(N, K).to(torch.uint8))
    scales = sg.permute(0, 2, 1, 3).reshape(N, K // 16).contiguous()
    return packed, scales
