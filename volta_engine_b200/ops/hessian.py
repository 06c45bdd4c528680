"""Hessian accumulation for calibration: H += X^T X over batches of layer inputs (fp32 accumulator).

The product runs on the tcgen05 GEMM (bf16 operands, fp32 accumulation): with W = X^T as the weight operand and X^T as
the activation operand, out[a, b] = sum_t X[t, a] X[t, b]. Rows are zero-padded to a multiple of 64 (the GEMM's k tile).
Reference: src/backend/cuda/modules/hessian.cu (``transpose_pad_kernel`` + GEMM).
"""
from __future__ import annotations

import torch

from . import kernels as K


class HessianAccumulator:
    def __init__(self, features: int, device):
        self.features = features
        self.H = torch.zeros(features, features, dtype=torch.float32, device=device)
        self.rows = 0

    def add(self, x: torch.Tensor):
        """x [rows, features] (any float dtype)."""
        rows = x.shape[0]
        if not x.is_cuda:
            xf = x.float()
            self.H += xf.t() @ xf
        else:
            pad = (rows + 63) // 64 * 64
            xt = torch.zeros(self.features, pad, dtype=torch.bfloat16, device=x.device)
            xt[:, :rows] = x.to(torch.bfloat16).t()
            self.H += K.gemm_bf16(xt, xt, out_f32=True)
        self.rows += rows
        return self

    def mean(self) -> torch.Tensor:
        return self.H / max(1, self.rows)
