"""Linear layers over the supported weight formats (reference: inc/engine/modules/linear.h:143-190
dispatches on QuantType {FP16, TRELLIS, NVFP4, FP8, GGUF}).

Kernel choice by row count on a GPU:
  * rows <= GEMV_MAX_ROWS : HBM-streaming mat-vec (one pass over the weights for up to 4 rows)
  * otherwise            : tcgen05 GEMM, weights as the UMMA A operand
``gemm_mode`` selects the prefill arithmetic for NVFP4 weights:
  ``w4a16``  bf16 activations, weights dequantised to f16 inside the tile loader (exact products)
  ``w4a4``   activations quantised to NVFP4 per 16 elements, native block-scaled FP4 MMA
  ``dequant`` weights expanded to bf16 in global memory + bf16 tcgen05 GEMM (debug / oracle)
"""
from __future__ import annotations

import torch

from ..quant import nvfp4 as qn
from . import kernels as K

GEMV_MAX_ROWS = 16
# A/B switch: "cublas" routes every multi-row product through torch.matmul on dequantised weights (library
# baseline / bring-up aid); unset = hand-written kernels only.
import os
GEMM_BACKEND = os.environ.get("VOLTA_GEMM_BACKEND", "native")
# auto | tc (tcgen05 block-scaled FP4 with residual-expanded activations) | mma (prepacked mma.sync mat-vec) | simt
GEMV_KERNEL = os.environ.get("VOLTA_GEMV", "auto")


class LinearBF16:
    def __init__(self, weight: torch.Tensor):
        self.weight = weight.contiguous()  # [N, K]
        self.out_features, self.in_features = weight.shape

    def forward(self, x, residual=None, out=None, out_f32=False):
        if not x.is_cuda:
            y = x.float() @ self.weight.float().t()
            if residual is not None:
                y = y + residual.float()
            return y if out_f32 else y.to(x.dtype)
        if x.shape[0] <= GEMV_MAX_ROWS and out_f32 and residual is None:
            return K.bf16_gemv_f32(self.weight, x, out)
        if GEMM_BACKEND == "cublas":
            y = torch.matmul(x, self.weight.t())
            if residual is not None:
                y = y + residual
            return y.float() if out_f32 else y
        return K.gemm_bf16(self.weight, x, out=out, residual=residual, out_f32=out_f32)

    def nbytes(self):
        return self.weight.numel() * self.weight.element_size()


class LinearNVFP4:
    """NVFP4 weight: packed codes [N, K/2], E4M3 block scales [N, K/16], fp32 tensor scale."""

    def __init__(self, packed, scales, gscale: float, gemm_mode: str = "w4a16"):
        self.packed, self.scales, self.gscale = packed.contiguous(), scales.contiguous(), float(gscale)
        self.out_features, self.in_features = packed.shape[0], packed.shape[1] * 2
        self.gemm_mode = gemm_mode
        self._sf_k128 = None
        self._sf_atoms = None
        self._gv = None

    @classmethod
    def from_dense(cls, w: torch.Tensor, gemm_mode="w4a16", search=True, global_scale: float | None = None):
        """``global_scale``: the tensor scale to quantise against (default: from this matrix's largest magnitude). A
        shard quantised against the scale of the whole matrix equals the slice of the quantised whole matrix."""
        p, s, g = qn.quantize_nvfp4(w, search=search, global_scale=global_scale)
        return cls(p, s, g, gemm_mode)

    def prepare(self):
        """Build the loader-side scale layouts once (load time, not on the hot path)."""
        if self.gemm_mode == "w4a16" and self._sf_k128 is None and self.out_features % 128 == 0:
            self._sf_k128 = qn.scales_blocked_k128(self.scales)
        tc = self._tc_ok() and GEMV_KERNEL in ("auto", "tc")
        if (self.gemm_mode == "w4a4" or tc) and self._sf_atoms is None and self.out_features % 128 == 0 \
                and self.in_features % 64 == 0:
            a = qn.scales_atoms_512(self.scales)
            nkg = self.in_features // 64
            if nkg % 4:         # K a multiple of 128 only: pad the k-groups with zero scales to whole 256-wide tiles
                a = a.reshape(self.out_features // 128, nkg, 512)
                a = torch.cat([a, torch.zeros(a.shape[0], (-nkg) % 4, 512, dtype=a.dtype, device=a.device)], 1).contiguous()
            self._sf_atoms = a
        if self._gv is None and self.packed.is_cuda and self.out_features % 16 == 0 and self.in_features % 64 == 0 \
                and (GEMV_KERNEL == "mma" or (GEMV_KERNEL == "auto" and not tc)):
            self._gv = qn.prepack_gv(self.packed, self.scales)
        return self

    def _tc_ok(self) -> bool:
        return (self.packed.is_cuda and self.out_features % 128 == 0 and self.in_features % 128 == 0
                and self.in_features <= K.DW_MAX_K)

    def dequant(self):
        return K.nvfp4_dequant(self.packed, self.scales, self.gscale)

    def addnorm_ready(self, rows: int) -> bool:
        """True when ``forward_addnorm`` runs as one launch for this row count."""
        return (rows <= GEMV_MAX_ROWS and GEMV_KERNEL in ("auto", "tc") and self._sf_atoms is not None and self._tc_ok()
                and self.out_features % 8 == 0)

    def rope_ready(self, rows: int, hd: int) -> bool:
        return hd == 128 and self.addnorm_ready(rows)

    def forward_rope(self, x, pos, slot, page_table, kpool, vpool, nq, nkv, rot_dim, theta):
        """The stacked q | k | v projection (head_dim 128) with the rotary embedding of q and k and the write of k and v
        into the paged cache done by the tile that finishes each head: returns the rotated qkv rows."""
        return K.decode_w4a4(self.packed, self._sf_atoms, self.gscale, x,
                             rope=(pos, slot, page_table, kpool, vpool, nq, nkv, rot_dim, theta))

    def forward_addnorm(self, x, resid, norm_w, eps, wbias=0.0):
        """resid += x W^T (in place); returns RMSNorm(resid) * (norm_w + wbias): the product, the residual add and the next
        block's input norm in one launch of the decode kernel (the tile that finishes last normalises the rows)."""
        rows = x.shape[0]
        normed = torch.empty(rows, self.out_features, dtype=torch.bfloat16, device=x.device)
        K.decode_w4a4(self.packed, self._sf_atoms, self.gscale, x, addnorm=(resid, norm_w, normed, eps, wbias))
        return normed

    def forward(self, x, residual=None, out=None, push=None, out_f32=False):
        """``push``: a communicator with ``push_target(rows, N)``; when the decode kernel runs, its epilogue also sends
        the rows into the peers' all-reduce staging area and ``push.pushed`` is set for the collective behind.
        ``out_f32``: fp32 result (logits of a quantised LM head)."""
        if push is not None:
            push.pushed = False
        if not x.is_cuda:
            y = x.float() @ qn.dequantize_nvfp4(self.packed, self.scales, self.gscale).t()
            if residual is not None:
                y = y + residual.float()
            return y if out_f32 else y.to(x.dtype)
        rows = x.shape[0]
        if out_f32:
            if rows <= GEMV_MAX_ROWS and self._sf_atoms is not None and self._tc_ok() and GEMV_KERNEL in ("auto", "tc"):
                return K.decode_w4a4(self.packed, self._sf_atoms, self.gscale, x, out=out, out_f32=True)
            y = self.forward(x, residual=residual).float()       # many rows: bf16 product widened (perplexity tools)
            if out is not None:
                out.copy_(y)
                return out
            return y
        if rows <= GEMV_MAX_ROWS:
            # tcgen05 path: the tensor core decodes the FP4 weights itself; activations ride as 4 residual NVFP4
            # terms per row (error below bf16 rounding), cost independent of the row count
            if GEMV_KERNEL in ("auto", "tc") and self._sf_atoms is not None and self._tc_ok():
                target = push.push_target(rows, self.out_features) if (push is not None and residual is None) else 0
                y = K.decode_w4a4(self.packed, self._sf_atoms, self.gscale, x, out=out, residual=residual, push_args=target)
                if target:
                    push.pushed = True
                return y
            # one row: the SIMT streaming kernel is faster; 2..16 rows: the tensor-core kernel costs the same
            # as one row. Both sum exact products in fp32, so they agree to fp32 rounding.
            if self._gv is not None and (GEMV_KERNEL == "mma" or (GEMV_KERNEL == "auto" and rows > 1)):
                return K.nvfp4_gemv_mma(self._gv[0], self._gv[1], self.gscale, x, self.out_features,
                                        self.in_features, out=out, residual=residual)
            return K.nvfp4_gemv(self.packed, self.scales, self.gscale, x, out=out, residual=residual)
        mode = self.gemm_mode
        if GEMM_BACKEND == "cublas":
            y = torch.matmul(x, self.dequant().t())
            return y + residual if residual is not None else y
        if mode == "w4a16" and self.out_features % 128 == 0 and self.in_features % 128 == 0:
            if self._sf_k128 is None:
                self.prepare()
            return K.gemm_w4a16(self.packed, self._sf_k128, self.gscale, x, out=out, residual=residual)
        if mode == "w4a4" and self.out_features % 128 == 0 and self.in_features % 256 == 0:
            if self._sf_atoms is None:
                self.prepare()
            xp, xs = K.nvfp4_quant_rows(x, blocked=True)
            return K.gemm_w4a4(self.packed, self._sf_atoms, self.gscale, xp, xs, rows, out=out, residual=residual)
        return K.gemm_bf16(self.dequant(), x, out=out, residual=residual)

    def interleave_gated(self):
        """For a stacked [gate | up] projection: reorder the rows to [64 gate | 64 up] per 128-row tile, so that the decode
        kernel can apply act(gate) * up in its epilogue (the prefill path reads the same layout through ``gated_act``)."""
        N = self.out_features
        I = N // 2
        if getattr(self, "gated", False) or N % 128 or I % 64:
            return self
        idx = torch.arange(I, device=self.packed.device).reshape(-1, 64)
        order = torch.stack([idx, idx + I], 1).reshape(-1)
        self.packed, self.scales = self.packed[order].contiguous(), self.scales[order].contiguous()
        self._sf_k128 = self._sf_atoms = self._gv = None
        self.gated = True
        return self.prepare() if self.packed.is_cuda else self

    def tc_ready(self) -> bool:
        """True when decode rows of this layer run on the tcgen05 decode linear."""
        return GEMV_KERNEL in ("auto", "tc") and self._sf_atoms is not None and self._tc_ok()

    def forward_prenorm(self, resid, delta, norm_w, eps, wbias, resid_out, act=None, limit: float = 0.0, rope=None):
        """Decode rows (<= 4) with the RMSNorm in front fused into the kernel: input RMSNorm(resid + delta) * (w + wbias),
        resid + delta written to ``resid_out``; ``act`` (0 SiLU / 1 GELU) additionally applies the gated activation;
        ``rope`` (the tuple of :meth:`forward_rope`) additionally rotates q / k and stores k / v from the epilogue."""
        return K.decode_w4a4(self.packed, self._sf_atoms, self.gscale, None, act=0 if act is None else 1 + act,
                             act_limit=limit, prenorm=(norm_w, resid, delta, resid_out, eps, wbias), rope=rope)

    def forward_gated(self, x, act: int = 0, limit: float = 0.0):
        """act(gate) * up of a ``interleave_gated`` projection: [rows, N/2]."""
        assert getattr(self, "gated", False)
        if x.is_cuda and x.shape[0] <= GEMV_MAX_ROWS and GEMV_KERNEL in ("auto", "tc") and self._sf_atoms is not None \
                and self._tc_ok():
            return K.decode_w4a4(self.packed, self._sf_atoms, self.gscale, x, act=1 + act, act_limit=limit)
        return K.gated_act(self.forward(x), self.out_features // 2, act, limit, interleave=64)

    def nbytes(self):
        return self.packed.numel() + self.scales.numel()


class LinearGroup:
    """Several linears over the same input whose outputs are concatenated along the feature axis (q/k/v or gate/up
    stored as separate quantised tensors with scales that cannot be merged)."""

    def __init__(self, parts):
        self.parts = list(parts)
        self.in_features = self.parts[0].in_features
        self.out_features = sum(p.out_features for p in self.parts)

    def forward(self, x, residual=None, out=None, **kw):
        ys = [p.forward(x, **kw) for p in self.parts]
        y = torch.cat(ys, dim=-1)
        if residual is not None:
            y = y + residual.to(y.dtype)
        if out is not None:
            out.copy_(y)
            return out
        return y

    def nbytes(self):
        return sum(p.nbytes() for p in self.parts)


def fuse_linears(parts):
    """One linear computing the concatenated outputs of ``parts``: a true merge where the formats allow it
    (dense rows; NVFP4 tensors sharing one tensor scale; EXL3 tensors sharing the input scales and codebook),
    otherwise a LinearGroup."""
    parts = list(parts)
    if len(parts) == 1:
        return parts[0]
    if all(isinstance(p, LinearBF16) for p in parts):
        return LinearBF16(torch.cat([p.weight for p in parts], 0))
    if all(isinstance(p, LinearNVFP4) for p in parts) and len({p.gscale for p in parts}) == 1 \
            and len({p.gemm_mode for p in parts}) == 1:
        m = LinearNVFP4(torch.cat([p.packed for p in parts], 0), torch.cat([p.scales for p in parts], 0),
                        parts[0].gscale, parts[0].gemm_mode)
        return m.prepare() if m.packed.is_cuda else m
    from .linear_exl3 import LinearEXL3
    if all(isinstance(p, LinearEXL3) for p in parts) and len({(p.bits, p.cb, p.layout) for p in parts}) == 1 \
            and all(p.bias is None for p in parts) and all(torch.equal(p.suh, parts[0].suh) for p in parts[1:]):
        return LinearEXL3(torch.cat([p.codes for p in parts], 1), parts[0].suh, torch.cat([p.svh for p in parts]),
                          bits=parts[0].bits, cb=parts[0].cb, layout=parts[0].layout)
    return LinearGroup(parts)
