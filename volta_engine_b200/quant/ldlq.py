"""Hessian-aware quantisation: block LDL error feedback around a block rounding function.

For a linear y = x W with W [K, N] and the calibration Hessian H = sum x^T x [K, K], the layer-wise loss of a
quantised W' is tr(E^T H E), E = W - W'. With the block factorisation H = L D L^T (L unit block-lower-triangular,
D block-diagonal, blocks of ``block`` input channels) the loss is sum_k || D_k^(1/2) (E_k + sum_{j>k} L[j,k]^T E_j) ||^2,
so the blocks are rounded from the last to the first, each one's target moved by the errors of the blocks after it:

    target_k = W_k + sum_{j>k} L[j,k]^T (W_j - W'_j),     W'_k = round_block(target_k, D_k)

Two rounding functions are provided: NVFP4 (E2M1 codes, one E4M3 scale per 16 input channels and output column, a
second pass of element-wise feedback inside the block under D_k) and the EXL3 trellis (tail-biting Viterbi per 16x16
tile in the rotated space). The reported proxy error is tr(E^T H E) / tr(W^T H W) with the damping taken out of H.

Reference: docs/QUANTIZATION.md:92 ("Per tensor": damping, block LDL factor, blocks quantised last to first, proxy
error), tests/tools/nvfp4_ldlq.py (the NVFP4 form), src/kernels/cuda/trellis/quant/ (the encoder).
"""
from __future__ import annotations

import torch

from . import nvfp4 as qn

BLOCK = 16


def damp(H: torch.Tensor, sigma_reg: float = 0.025) -> torch.Tensor:
    """Mean Hessian plus ``sigma_reg`` of its mean diagonal on the diagonal; dead channels get a unit diagonal."""
    H = H.double().clone()
    d = H.diagonal()
    mean = float(d.mean())
    dead = d <= 0
    if mean <= 0:
        return torch.eye(H.shape[0], dtype=torch.float64, device=H.device)
    d[dead] = mean
    d += sigma_reg * mean
    return H


def block_ldl(H: torch.Tensor, block: int = BLOCK):
    """H (symmetric positive definite, [K, K], K a multiple of ``block``) -> (L, D): L unit block-lower-triangular
    [K, K] (identity diagonal blocks), D [K / block, block, block], H = L blockdiag(D) L^T."""
    K = H.shape[0]
    assert K % block == 0
    C = torch.linalg.cholesky(H.double())
    nb = K // block
    Ckk = torch.stack([C[i * block:(i + 1) * block, i * block:(i + 1) * block] for i in range(nb)])
    inv = torch.linalg.inv(Ckk)
    L = C.clone()
    for i in range(nb):
        L[:, i * block:(i + 1) * block] = C[:, i * block:(i + 1) * block] @ inv[i]
    D = Ckk @ Ckk.transpose(1, 2)
    return L, D


def proxy_error(W: torch.Tensor, Wq: torch.Tensor, H: torch.Tensor) -> float:
    """tr(E^T H E) / tr(W^T H W) for W, Wq [K, N] and H [K, K] (any positive scale of H gives the same value)."""
    H = H.double()
    E = (W.double() - Wq.double())
    den = float((W.double() * (H @ W.double())).sum())
    return float((E * (H @ E)).sum()) / max(den, 1e-300)


# ------------------------------------------------------------------------------------------------ block rounders
def _nvfp4_scale_codes(t: torch.Tensor, g: float) -> torch.Tensor:
    """One E4M3 scale code per column of a [16, N] block (value in units of the tensor scale ``g``)."""
    return qn.e4m3_encode((t.abs().amax(dim=0) / 6.0 / g).clamp(max=448.0))


def nvfp4_round_block(t: torch.Tensor, Dk: torch.Tensor, g: float, search=(0, -1, 1)):
    """Rounds a [16, N] target block. For every candidate scale (the code of the column maximum and its neighbours)
    the rows are rounded from the last to the first with element-wise LDL feedback under D_k; each column keeps the
    candidate with the smallest e^T D_k e. -> (dequantised block fp64, codes uint8 [16, N], scales fp32 [N])."""
    R, N = t.shape
    base = _nvfp4_scale_codes(t.float(), g).to(torch.int16)
    cand = torch.stack([(base + d).clamp(0, 126) for d in search]).to(torch.uint8)          # [C, N]
    C = cand.shape[0]
    s = (qn.e4m3_decode(cand).float() * g).reshape(-1)                                        # [C*N]
    s_safe = torch.where(s > 0, s, torch.ones_like(s))
    Lk, _ = block_ldl(Dk, 1)
    tt = t.double().repeat(1, C)                                                              # [R, C*N]
    q = torch.zeros_like(tt)
    codes = torch.zeros(tt.shape, dtype=torch.uint8, device=t.device)
    for i in range(R - 1, -1, -1):
        tgt = tt[i]
        if i + 1 < R:
            tgt = tgt + Lk[i + 1:, i] @ (tt[i + 1:] - q[i + 1:])
        c = qn.e2m1_encode((tgt / s_safe).float())
        codes[i] = c
        q[i] = (qn.e2m1_decode(c).float() * s).double()
    E = tt - q
    err = (E * (Dk.double() @ E)).sum(0).reshape(C, N)
    pick = err.argmin(0)                                                                      # [N]
    col = pick * N + torch.arange(N, device=t.device)
    return q[:, col], codes[:, col], s[col]


def ldlq(W: torch.Tensor, H: torch.Tensor, round_block, block: int = BLOCK, sigma_reg: float = 0.025):
    """Generic driver. W [K, N], H [K, K] (sum or mean); ``round_block(target [block, N] fp64, D_k, k)`` returns the
    dequantised block first and anything else after it. -> (Wq fp32 [K, N], list of the extra returns per block)."""
    K = W.shape[0]
    Hd = damp(H.to(W.device), sigma_reg)
    L, D = block_ldl(Hd, block)
    Wd = W.double()
    Wq = torch.zeros_like(Wd)
    extras = [None] * (K // block)
    for k in range(K // block - 1, -1, -1):
        lo, hi = k * block, (k + 1) * block
        tgt = Wd[lo:hi]
        if hi < K:
            tgt = tgt + L[hi:, lo:hi].t() @ (Wd[hi:] - Wq[hi:])
        out = round_block(tgt, D[k], k)
        Wq[lo:hi] = out[0]
        extras[k] = out[1:]
    return Wq.float(), extras


def quantize_nvfp4_hessian(w: torch.Tensor, H: torch.Tensor, sigma_reg: float = 0.025, global_scale: float | None = None):
    """Hessian-aware NVFP4 of a checkpoint-orientation weight ``w`` [N, K] (y = x w^T) under H [K, K].
    -> (packed uint8 [N, K/2], scales E4M3 bytes [N, K/16], gscale) exactly as ``quantize_nvfp4`` returns them."""
    N, K = w.shape
    W = w.float().t().contiguous()
    g = float(global_scale) if global_scale else max(float(W.abs().max()) / (6.0 * 448.0), 1e-30)
    Wq, ex = ldlq(W, H, lambda t, Dk, k: nvfp4_round_block(t, Dk, g), BLOCK, sigma_reg)
    codes = torch.cat([e[0] for e in ex], 0).t().contiguous()                       # [N, K]
    scales = torch.stack([e[1] for e in ex], 1)                                    # [N, K/16] fp32 (decoded, in g units)
    sb = qn.e4m3_encode((scales / g).float())
    return qn.pack_codes(codes), sb, g


def exl3_round_block_factory(bits: int, cb: int, scale: float, layout: str = "stock"):
    """Rounding function of one 16-row block in the rotated space of the trellis format: every 16x16 tile of the
    block is Viterbi-encoded against the target (joint over its 256 values), no feedback inside the block."""
    from . import exl3 as ex
    row, col = ex._tile_positions(layout)

    def rnd(t, Dk, k):
        N = t.shape[1]
        codes = torch.zeros(N // 16, 16 * bits, dtype=torch.int16)
        tn = (t / scale).float()
        for nt in range(N // 16):
            tile = tn[:, nt * 16:(nt + 1) * 16]
            codes[nt] = ex.viterbi_encode_tile(tile[row, col].contiguous(), bits, cb).cpu()
        deq = ex.reconstruct(codes[None].to(t.device), bits, cb, layout).double() * scale
        return deq, codes

    return rnd


def quantize_exl3_hessian(W: torch.Tensor, H: torch.Tensor, bits: int, cb: int | None = None, seed: int = 0,
                          sigma_reg: float = 0.025):
    """Hessian-aware trellis quantisation of W [K, N] (y = x W): the Hessian is carried into the rotated space
    (H_r = Had Su H Su Had), the blocks of 16 rotated input channels are encoded last to first with the LDL feedback.
    -> (codes, suh, svh) as ``exl3.quantize`` returns them. Cost as the plain quantiser: small matrices only."""
    from . import exl3 as ex
    cb = ex.CB_MUL1 if cb is None else cb
    K, N = W.shape
    assert K % 128 == 0 and N % 128 == 0
    g = torch.Generator().manual_seed(seed)
    su = (torch.randint(0, 2, (K,), generator=g).float() * 2 - 1).to(W.device)
    sv = (torch.randint(0, 2, (N,), generator=g).float() * 2 - 1).to(W.device)
    Wr = ex.had128((ex.had128((W.float() * su[:, None] * sv[None, :]).t().contiguous())).t().contiguous())
    Hs = H.float().to(W.device) * su[:, None] * su[None, :]
    Hr = ex.had128(ex.had128(Hs).t().contiguous())             # Had Hs Had (Had symmetric, applied to rows then columns)
    Hr = 0.5 * (Hr + Hr.t())
    scale = float(Wr.std().clamp(min=1e-12))
    Wq, extra = ldlq(Wr, Hr, exl3_round_block_factory(bits, cb, scale), BLOCK, sigma_reg)
    codes = torch.stack([e[0] for e in extra], 0)
    return codes.to(W.device), su.to(torch.float16), (sv * scale).to(torch.float16)
