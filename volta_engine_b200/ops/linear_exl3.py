"""Linear layer over EXL3 trellis-coded weights: ``y = had128(had128(x * suh) @ W) * svh``.

GPU: rows <= 16 run rotate -> fused decode mat-vec (mma.sync with the tile's native fragment order) -> rotate
(csrc/cuda/exl3.cu); larger row counts reconstruct W to bf16 once per call and run the tcgen05 GEMM between the
two rotations. CPU: the fp32 oracle of quant/exl3.py.
Reference: src/backend/cpu/linear_trellis.cpp:129-239, src/kernels/cuda/trellis/ (GEMV / GEMM split by row count).
"""
from __future__ import annotations

import torch

from .._lib import call, ptr
from ..quant import exl3 as ex
from . import kernels as K

_DT = {torch.bfloat16: 0, torch.float32: 1, torch.float16: 2}


def had128(x, scale=None, *, post=False, out_dtype=None, out=None, x2=None, scale2=None, act=0, expert=None,
           scale_stride=0, in_div=1, rows_per_group=1, rows=None):
    """GPU Hadamard rotation over blocks of 128 with the EXL3 channel scales folded in (see ve_had128)."""
    C = x.shape[-1]
    rows = rows if rows is not None else x.numel() // C
    out_dtype = out_dtype or x.dtype
    if out is None:
        out = torch.empty(rows, C, dtype=out_dtype, device=x.device)
    call("had128", "pppppp" + "liiiiiiii", ptr(x), ptr(x2), ptr(out), ptr(scale), ptr(scale2), ptr(expert),
         int(scale_stride), rows, C, 1 if post else 0, in_div, rows_per_group, act, _DT[x.dtype], _DT[out.dtype])
    return out


def exl3_gemv(codes, x_rot, M, K_, N, bits, cb, out=None, expert=None, expert_stride=0, groups=1):
    if out is None:
        out = torch.empty(groups * M, N, dtype=torch.float32, device=x_rot.device)
    call("exl3_gemv", "pppiiiiipli", ptr(codes), ptr(x_rot), ptr(out), M, K_, N, bits, cb, ptr(expert),
         int(expert_stride), groups)
    return out


def exl3_reconstruct(codes, K_, N, bits, cb, out=None):
    if out is None:
        out = torch.empty(N, K_, dtype=torch.bfloat16, device=codes.device)
    call("exl3_reconstruct", "ppiiii", ptr(codes), ptr(out), K_, N, bits, cb)
    return out


def exl3_viterbi(targets: torch.Tensor, bits: int, cb: int = ex.CB_MUL1, ctas: int | None = None) -> torch.Tensor:
    """Trellis-encode tiles on the GPU: ``targets`` fp32 [tiles, 256] (stream-position order, codebook units) -> codes
    int16 [tiles, 16 * bits]; the exact Viterbi search of ``quant.exl3.viterbi_encode_tile`` (bits 2..8)."""
    assert targets.is_cuda and targets.dtype == torch.float32 and targets.shape[-1] == 256 and 2 <= bits <= 8
    targets = targets.contiguous()
    tiles = targets.shape[0]
    ctas = ctas or min(tiles, 148)
    per = 255 * (1 << (16 - bits))
    back = torch.empty(ctas * per, dtype=torch.uint8, device=targets.device)
    codes = torch.empty(tiles, 16 * bits, dtype=torch.int16, device=targets.device)
    call("exl3_viterbi", "pppiiii", ptr(targets), ptr(codes), ptr(back), tiles, bits, cb, ctas)
    return codes


class LinearEXL3:
    """codes int16 [K/16, N/16, 16*bits] (16*bits + 8 for the half-integer rate bits + 0.5); suh fp16 [K]; svh fp16 [N];
    optional bias."""

    def __init__(self, codes, suh, svh, bits: int | None = None, cb: int = ex.CB_MUL1, bias=None,
                 layout: str = "stock", tstart=None, tgain=None):
        self.codes = codes.contiguous()
        self.layout = layout          # "volta": tiles in the reference engine's lane order
        self._dense = None            # bf16 expansion used on the GPU for the non-stock order
        self.bits = int(bits) if bits is not None else codes.shape[-1] // 16
        self.tstart, self.tgain = tstart, tgain  # extended trellis: per-tile start states / gain codes [K/16, N/16] or None
        self.half = ex.is_half_rate(codes)       # rate bits + 0.5 (16 * bits + 8 code words per tile): no device decoder,
                                                 # expanded to bf16 when it moves to a GPU (so is an extended trellis)
        self.cb = cb
        self.in_features, self.out_features = codes.shape[0] * 16, codes.shape[1] * 16
        self.suh, self.svh = suh.to(torch.float16).contiguous(), svh.to(torch.float16).contiguous()
        self.bias = bias

    @classmethod
    def synth(cls, in_features, out_features, bits=4, std=0.02, gen=None, device="cpu"):
        return cls(*ex.synth_linear(in_features, out_features, bits, std, gen, device), bits=bits)

    @classmethod
    def from_dense(cls, w: torch.Tensor, bits: int):
        """w: [out, in] like nn.Linear."""
        return cls(*ex.quantize(w.t().contiguous().float(), bits), bits=bits)

    def to(self, device):
        ext = self.tstart is not None or self.tgain is not None
        if (self.layout != "stock" or self.half or ext) and torch.device(device).type == "cuda" and self._dense is None:
            w = ex.reconstruct(self.codes.cpu(), self.bits, self.cb, self.layout,
                               None if self.tstart is None else self.tstart.cpu(), None if self.tgain is None else self.tgain.cpu())
            self._dense = w.t().contiguous().to(torch.bfloat16).to(device)
        self.codes, self.suh, self.svh = self.codes.to(device), self.suh.to(device), self.svh.to(device)
        if self.bias is not None:
            self.bias = self.bias.to(device)
        return self

    def dequant(self) -> torch.Tensor:
        """Effective dense weight [out, in] (fp32), rotations and scales included."""
        return ex.effective_weight(self.codes.cpu(), self.bits, self.suh.cpu(), self.svh.cpu(), self.cb, self.layout,
                                   None if self.tstart is None else self.tstart.cpu(),
                                   None if self.tgain is None else self.tgain.cpu()).t().contiguous()

    def forward(self, x, residual=None, out=None, out_f32=False):
        Kf, N = self.in_features, self.out_features
        if not x.is_cuda:
            y = ex.linear_reference(x.float(), self.codes, self.bits, self.suh, self.svh, self.cb, self.layout, self.tstart, self.tgain)
            if self.bias is not None:
                y = y + self.bias.float()
            if residual is not None:
                y = y + residual.float()
            return y if out_f32 else y.to(x.dtype)
        rows = x.shape[0]
        odt = torch.float32 if out_f32 else torch.bfloat16
        if rows <= 16 and self._dense is None:
            xr = had128(x, self.suh, out_dtype=torch.float16)
            acc = exl3_gemv(self.codes, xr, rows, Kf, N, self.bits, self.cb)
            y = had128(acc, self.svh, post=True, out_dtype=odt, out=out if residual is None and self.bias is None else None)
        else:
            xr = had128(x, self.suh, out_dtype=torch.bfloat16)
            w = self._dense if self._dense is not None else exl3_reconstruct(self.codes, Kf, N, self.bits, self.cb)
            acc = K.gemm_bf16(w, xr, out_f32=True)
            y = had128(acc, self.svh, post=True, out_dtype=odt, out=out if residual is None and self.bias is None else None)
        if self.bias is not None:
            y = y + self.bias.to(y.dtype)
        if residual is not None:
            y = y + residual.to(y.dtype)
        if out is not None and y is not out:
            out.copy_(y)
            return out
        return y

    __call__ = forward

    def nbytes(self):
        return self.codes.numel() * 2 + (self.suh.numel() + self.svh.numel()) * 2
