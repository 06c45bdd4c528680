"""Routed experts stored as GGUF blocks (any block type of quant/gguf.py, the codebook formats included).

``GGUFExpertBank`` holds this rank's experts back to back: gate|up rows ``[E, 2I, row_bytes(H)]`` and down rows
``[E, H, row_bytes(I)]`` as raw blocks, one ggml type per projection (a checkpoint's experts usually mix a low-bit type
for gate / up with a wider one for down). Three ways through it:

  * decode / verify rows (<= 16): the fused dequant mat-vec per route (csrc/cuda/gguf_gemv.cu ``gguf_moe_gemv``), gated
    activation inside the gate|up launch, rows of experts owned by other ranks come out as zeros;
  * prefill chunks: routes sorted by expert, then per slab of experts: blocks -> bf16 (``gguf_dequant``) into a bounded
    scratch, grouped tcgen05 GEMMs over the slab's tiles, activation, down projection; the slab's rows are scattered back
    into route order. No host synchronisation: the tile table of every slab is built on the device;
  * CPU: the fp32 statement (dequantise, matmul, bf16 rounding between the stages).
Reference: src/kernels/cuda/gguf/gguf_moe.cu:38-1042 (MoEGguf: per-route mat-vec and grouped tiles),
inc/engine/modules/moe_gguf.h.
"""
from __future__ import annotations

import torch

from .._lib import call, ptr
from ..quant import gguf as gq
from . import kernels as K
from .linear_gguf import FUSED_TYPES, ensure_iq_grids

SLAB_BYTES = 2 << 30          # bf16 scratch for the dequantised experts of one slab (gate|up and down share it)


_TYPE_BY_NAME = {v.lower(): k for k, v in gq.NAMES.items()}


def parse_expert_quant(spec: str) -> tuple[int, int]:
    """"gguf_iq2_xxs" -> (IQ2_XXS, IQ2_XXS); "gguf_iq2_xxs+q4_k" -> (IQ2_XXS for gate / up, Q4_K for down)."""
    assert spec.startswith("gguf_"), spec
    parts = spec[5:].lower().split("+")
    try:
        gt = _TYPE_BY_NAME[parts[0]]
        dt = _TYPE_BY_NAME[parts[1]] if len(parts) > 1 else gt
    except KeyError as e:
        raise ValueError(f"unknown GGUF block type in '{spec}'; known: {sorted(_TYPE_BY_NAME)}") from e
    return gt, dt


class GGUFExpertBank:
    def __init__(self, gu_raw: torch.Tensor, gu_type: int, dn_raw: torch.Tensor, dn_type: int, e0: int, inter: int,
                 hidden: int):
        E = gu_raw.shape[0]
        self.gu_raw = gu_raw.contiguous().reshape(E, 2 * inter, -1)
        self.dn_raw = dn_raw.contiguous().reshape(E, hidden, -1)
        self.gu_type, self.dn_type = gu_type, dn_type
        self.e0, self.e_local, self.inter, self.hidden = e0, E, inter, hidden
        assert self.gu_raw.shape[2] == gq.row_bytes(gu_type, hidden) and self.dn_raw.shape[2] == gq.row_bytes(dn_type, inter)
        assert gu_type in FUSED_TYPES and dn_type in FUSED_TYPES, "expert banks hold block-quantised types"
        if self.gu_raw.is_cuda and (gu_type in gq.IQ_TYPES or dn_type in gq.IQ_TYPES):
            ensure_iq_grids(self.gu_raw.device)
        self.gu_sf = self.dn_sf = None          # (attribute of the NVFP4 bank that callers test)

    @classmethod
    def from_dense(cls, gate_up: torch.Tensor, down: torch.Tensor, gu_type: int, dn_type: int, e0: int = 0):
        """gate_up [E, 2I, H], down [E, H, I] fp32 -> quantised bank (types with a quantiser only)."""
        E, I2, H = gate_up.shape
        gu = torch.stack([gq.quantize(gate_up[e].float(), gu_type) for e in range(E)])
        dn = torch.stack([gq.quantize(down[e].float(), dn_type) for e in range(E)])
        return cls(gu, gu_type, dn, dn_type, e0, I2 // 2, H)

    @classmethod
    def random(cls, E: int, inter: int, hidden: int, gu_type: int, dn_type: int, e0: int = 0, seed: int = 0, device="cpu",
               amp: float = 0.02):
        """Synthetic bank (random payload bytes, small finite scales): any block type, no quantiser needed."""
        draw = device if torch.device(device).type == "cuda" else "cpu"
        gu = gq.random_blocks(gu_type, E * 2 * inter, hidden, seed, amp, draw).reshape(E, 2 * inter, -1)
        dn = gq.random_blocks(dn_type, E * hidden, inter, seed + 1, amp, draw).reshape(E, hidden, -1)
        return cls(gu.to(device), gu_type, dn.to(device), dn_type, e0, inter, hidden)

    def to(self, device):
        return GGUFExpertBank(self.gu_raw.to(device), self.gu_type, self.dn_raw.to(device), self.dn_type, self.e0, self.inter,
                              self.hidden)

    def nbytes(self) -> int:
        return self.gu_raw.numel() + self.dn_raw.numel()

    def dequant(self, which: str, e: int) -> torch.Tensor:
        raw, t, k = (self.gu_raw, self.gu_type, self.hidden) if which == "gu" else (self.dn_raw, self.dn_type, self.inter)
        return gq.dequantize(raw[e], t, k)

    # ------------------------------------------------------------------------------------------ decode rows
    def routes_decode(self, x: torch.Tensor, ids: torch.Tensor, act: int, limit: float) -> torch.Tensor:
        """x [rows, H] bf16, ids [rows, k] int32 -> d [rows * k, H]: the down projection of every route (zeros for
        experts of other ranks)."""
        rows, H = x.shape
        k = ids.shape[1]
        routes, I = rows * k, self.inter
        a = torch.empty(routes, I, dtype=x.dtype, device=x.device)
        call("gguf_moe_gemv", "pilpiiplipliiiiif", ptr(self.gu_raw), self.gu_type, self.gu_raw.shape[2], ptr(ids), self.e0,
             self.e_local, ptr(x), x.stride(0), k, ptr(a), a.stride(0), routes, 2 * I, H, 1, act, float(limit))
        d = torch.empty(routes, H, dtype=x.dtype, device=x.device)
        call("gguf_moe_gemv", "pilpiiplipliiiiif", ptr(self.dn_raw), self.dn_type, self.dn_raw.shape[2], ptr(ids), self.e0,
             self.e_local, ptr(a), a.stride(0), 1, ptr(d), d.stride(0), routes, H, I, 0, act, 0.0)
        return d

    # ------------------------------------------------------------------------------------------ prefill chunks
    def slab_experts(self) -> int:
        per = 2 * self.inter * self.hidden * 2 + self.hidden * self.inter * 2
        return max(1, min(self.e_local, SLAB_BYTES // per))

    def routes_prefill(self, x: torch.Tensor, ids: torch.Tensor, act: int, limit: float) -> torch.Tensor:
        """Same result layout as :meth:`routes_decode` for a chunk of rows, through the grouped tensor-core GEMM."""
        rows, H = x.shape
        k = ids.shape[1]
        routes, I, dev = rows * k, self.inter, x.device
        G = self.slab_experts()
        bn = 64 if routes // max(1, self.e_local) < 96 else 128
        d_all = torch.zeros(routes, H, dtype=x.dtype, device=dev)
        w_gu = torch.empty(G * 2 * I, H, dtype=torch.bfloat16, device=dev)
        w_dn = torch.empty(G * H, I, dtype=torch.bfloat16, device=dev)
        st = K.status_word(dev)
        for g0 in range(0, self.e_local, G):
            g = min(G, self.e_local - g0)
            max_tiles = routes // bn + g + 1
            inv = torch.empty(routes, dtype=torch.int32, device=dev)
            srt = torch.empty(routes, dtype=torch.int32, device=dev)
            tab = torch.empty(max_tiles, 4, dtype=torch.int32, device=dev)
            totals = torch.zeros(2, dtype=torch.int32, device=dev)
            call("moe_sort", "piiiipppip", ptr(ids), routes, self.e0 + g0, g, bn, ptr(inv), ptr(srt), ptr(tab), max_tiles,
                 ptr(totals))
            xs = torch.zeros(routes, H, dtype=x.dtype, device=dev)
            call("moe_gather", "plppiplii", ptr(x), x.stride(0), ptr(srt), ptr(totals), k, ptr(xs), xs.stride(0), H, routes)
            call("gguf_dequant", "pilpli", ptr(self.gu_raw[g0:g0 + g]), self.gu_type, self.gu_raw.shape[2], ptr(w_gu),
                 g * 2 * I, H)
            call("gguf_dequant", "pilpli", ptr(self.dn_raw[g0:g0 + g]), self.dn_type, self.dn_raw.shape[2], ptr(w_dn),
                 g * H, I)
            gu = torch.zeros(routes, 2 * I, dtype=x.dtype, device=dev)
            call("gemm_grouped_bf16", "plplpliiiiipip", ptr(w_gu), H, ptr(xs), xs.stride(0), ptr(gu), gu.stride(0), routes, g,
                 2 * I, H, bn, ptr(tab), max_tiles, ptr(st))
            a = K.gated_act(gu, I, act, limit)
            ds = torch.zeros(routes, H, dtype=x.dtype, device=dev)
            call("gemm_grouped_bf16", "plplpliiiiipip", ptr(w_dn), I, ptr(a), a.stride(0), ptr(ds), ds.stride(0), routes, g, H,
                 I, bn, ptr(tab), max_tiles, ptr(st))
            mine = inv >= 0
            d_all = torch.where(mine[:, None], ds[inv.clamp(min=0).long()], d_all)
        return d_all

    # ------------------------------------------------------------------------------------------ statement
    def routes_reference(self, x: torch.Tensor, ids: torch.Tensor, act: int, limit: float) -> torch.Tensor:
        rows, H = x.shape
        k = ids.shape[1]
        d = torch.zeros(rows * k, H, dtype=x.dtype)
        for t in range(rows):
            for j in range(k):
                e = int(ids[t, j]) - self.e0
                if e < 0 or e >= self.e_local:
                    continue
                gu = (x[t:t + 1].float() @ self.dequant("gu", e).t()).to(x.dtype)
                a = K.gated_act(gu, self.inter, act, limit)
                d[t * k + j] = (a.float() @ self.dequant("dn", e).t()).to(x.dtype)[0]
        return d

    def routes(self, x: torch.Tensor, ids: torch.Tensor, act: int = 0, limit: float = 0.0) -> torch.Tensor:
        if not x.is_cuda:
            return self.routes_reference(x, ids, act, limit)
        if self.gu_type in gq.IQ_TYPES or self.dn_type in gq.IQ_TYPES:
            ensure_iq_grids(x.device)             # (a bank moved to the device after it was built has not done this yet)
        if x.shape[0] <= 16:
            return self.routes_decode(x, ids, act, limit)
        return self.routes_prefill(x, ids, act, limit)
