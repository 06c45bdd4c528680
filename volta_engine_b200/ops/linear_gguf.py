"""Linear layer over GGUF block-quantised weights (Q8_0, Q4_0/1, Q5_0/1, Q2_K..Q6_K, IQ4_NL/XS, IQ1_S/M, IQ2_XXS/XS/S,
IQ3_XXS/S; F16/BF16 pass through).

GPU: rows <= 16 use the fused dequant mat-vec (csrc/cuda/gguf_gemv.cu); larger row counts dequantise to bf16
and run the tcgen05 GEMM. CPU: fp32 oracle, optionally with the CPU backend's Q8_0 activation semantics
(reference: src/backend/cpu/linear_gguf.cpp:65-113, dispatch src/kernels/cuda/gguf/gguf_linear.cu:1-5).
"""
from __future__ import annotations

import ctypes

import torch

from .. import _lib
from .._lib import call, ptr
from ..quant import gguf as gq
from . import kernels as K


FUSED_TYPES = frozenset((gq.GGML_Q8_0, gq.GGML_Q4_0, gq.GGML_Q4_K, gq.GGML_Q6_K, gq.GGML_Q4_1, gq.GGML_Q5_0, gq.GGML_Q5_1,
                         gq.GGML_Q2_K, gq.GGML_Q3_K, gq.GGML_Q5_K, gq.GGML_IQ4_NL, gq.GGML_IQ4_XS)) | gq.IQ_TYPES

_iq_tables: dict = {}


def ensure_iq_grids(device) -> None:
    """The codebook formats read their grids from one table in device memory: upload it once per device."""
    device = torch.device(device)
    key = device.index if device.index is not None else torch.cuda.current_device()
    if key in _iq_tables:
        return
    from ..quant import gguf_iq
    t = torch.frombuffer(bytearray(gguf_iq.grid_blob()), dtype=torch.uint8).to(device)
    with torch.cuda.device(device):
        rc = _lib.kernels().ve_gguf_set_iq_grids(ctypes.c_void_p(t.data_ptr()))
    if rc != 0:
        raise RuntimeError(f"ve_gguf_set_iq_grids failed with CUDA error {rc}")
    _iq_tables[key] = t


class LinearGGUF:
    def __init__(self, raw: torch.Tensor, ggml_type: int, out_features: int, in_features: int, act_q8: bool = False):
        self.raw = raw.contiguous().reshape(out_features, -1)
        self.ggml_type, self.out_features, self.in_features = ggml_type, out_features, in_features
        self.row_bytes = self.raw.shape[1]
        assert self.row_bytes == gq.row_bytes(ggml_type, in_features)
        self.act_q8 = act_q8
        if self.raw.is_cuda and ggml_type in gq.IQ_TYPES:
            ensure_iq_grids(self.raw.device)

    @classmethod
    def from_dense(cls, w: torch.Tensor, ggml_type: int, act_q8: bool = False):
        return cls(gq.quantize(w, ggml_type), ggml_type, w.shape[0], w.shape[1], act_q8)

    def dequant(self) -> torch.Tensor:
        if self.raw.is_cuda and self.ggml_type in gq.IQ_TYPES:
            ensure_iq_grids(self.raw.device)
        if self.raw.is_cuda and self.ggml_type in FUSED_TYPES:
            out = torch.empty(self.out_features, self.in_features, dtype=torch.bfloat16, device=self.raw.device)
            call("gguf_dequant", "pilpli", ptr(self.raw), self.ggml_type, self.row_bytes, ptr(out), self.out_features,
                 self.in_features)
            return out
        return gq.dequantize(self.raw, self.ggml_type, self.in_features).to(torch.bfloat16)

    def forward(self, x, residual=None, out=None, out_f32=False):
        if not x.is_cuda:
            if self.act_q8 and self.ggml_type == gq.GGML_Q8_0:
                y = gq.linear_q8_0_cpu_semantics(x.float(), self.raw, self.in_features)
            else:
                y = x.float() @ gq.dequantize(self.raw, self.ggml_type, self.in_features).t()
            if residual is not None:
                y = y + residual.float()
            return y if out_f32 else y.to(x.dtype)
        rows = x.shape[0]
        if self.ggml_type in gq.IQ_TYPES:
            ensure_iq_grids(x.device)
        quant = self.ggml_type in FUSED_TYPES
        if rows <= 16 and quant and residual is None:
            if out is None:
                out = torch.empty(rows, self.out_features, dtype=torch.float32 if out_f32 else torch.bfloat16,
                                  device=x.device)
            call("gguf_gemv", "pilplpliiii", ptr(self.raw), self.ggml_type, self.row_bytes, ptr(x), x.stride(0),
                 ptr(out), out.stride(0), 1 if out.dtype == torch.float32 else 0, rows, self.out_features,
                 self.in_features)
            return out
        w = self.dequant()
        if rows <= 16 and out_f32 and residual is None:
            return K.bf16_gemv_f32(w, x, out)
        return K.gemm_bf16(w, x, out=out, residual=residual, out_f32=out_f32)

    def nbytes(self):
        return self.raw.numel()
