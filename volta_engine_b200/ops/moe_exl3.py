"""Routed experts stored as EXL3 (trellis-coded) weights.

``EXL3ExpertBank`` holds this rank's experts back to back: gate, up ``[E, H/16, I/16, 16 bits]`` and down
``[E, I/16, H/16, 16 bits]`` code tensors with their input / output channel scales (``suh`` / ``svh``, fp16) per expert.
An EXL3 linear is ``y = had(had(x * suh) @ W) * svh`` with 128-point Hadamard rotations on both sides, so a routed
expert costs rotations around each of its three matrices:

  * decode / verify rows (<= 16): per route, the activation row rotated with the route's expert scales
    (``had128(expert=)``), the fused trellis decode + mat-vec with one group per route (``exl3_gemv(expert=)``), then one
    launch that rotates both projections back, applies their output scales and the gated activation
    (``had128(x2=, act=)``); the same again around the down projection. Routes of experts owned by other ranks come out
    as zeros;
  * prefill chunks: routes sorted by expert, then per slab of experts: codes -> bf16 cores (``exl3_reconstruct_batch``)
    into a bounded scratch, rows rotated with their expert's scales, grouped tcgen05 GEMMs over the slab's tiles, rotated
    back; the slab's rows are scattered back into route order (no host synchronisation);
  * CPU: the fp32 statement (``quant.exl3.linear_reference`` per route).
Reference: src/kernels/cuda/trellis/exl3_moe_coop.cu:1034-1205 (rotation kernel, gate / up mat-vec per expert run, down
mat-vec), exl3_moe_kernel.cuh (prefill work items), inc/engine/modules/moe.h:79-195.
"""
from __future__ import annotations

import torch

from .._lib import call, ptr
from ..quant import exl3 as ex
from . import kernels as K
from .linear_exl3 import exl3_gemv, had128

SLAB_BYTES = 2 << 30


class EXL3ExpertBank:
    def __init__(self, gate, up, down, scales: dict, bits: int, e0: int, inter: int, hidden: int, cb: int = ex.CB_MUL1):
        """gate / up [E, H/16, I/16, 16 bits], down [E, I/16, H/16, 16 bits] int16; ``scales``: fp16 tensors
        g_suh / u_suh [E, H], g_svh / u_svh [E, I], d_suh [E, I], d_svh [E, H]."""
        self.gate, self.up, self.down = gate.contiguous(), up.contiguous(), down.contiguous()
        self.s = {k: v.to(torch.float16).contiguous() for k, v in scales.items()}
        self.bits, self.cb = bits, cb
        self.e0, self.e_local, self.inter, self.hidden = e0, gate.shape[0], inter, hidden
        assert gate.shape[1:] == (hidden // 16, inter // 16, 16 * bits) and down.shape[1:] == (inter // 16, hidden // 16, 16 * bits)
        assert hidden % 128 == 0 and inter % 128 == 0, "the Hadamard rotations work on blocks of 128"
        self.gu_sf = self.dn_sf = None          # (attribute of the NVFP4 bank that callers test)

    @classmethod
    def random(cls, E: int, inter: int, hidden: int, bits: int, e0: int = 0, seed: int = 0, device="cpu", std: float = 0.02):
        """Synthetic bank: uniformly random code streams (random windows decode to near-Gaussian unit values, which is
        what a trellis encoding of random weights looks like), random sign input scales, output scales of ``std``."""
        draw = device if torch.device(device).type == "cuda" else "cpu"
        g = torch.Generator(device=draw).manual_seed(seed)

        def codes(K_, N):
            return torch.randint(0, 65536, (E, K_ // 16, N // 16, 16 * bits), generator=g, device=draw, dtype=torch.int32).to(torch.int16)

        def signs(n, amp=1.0):
            return ((torch.randint(0, 2, (E, n), generator=g, device=draw).float() * 2 - 1) * amp).to(torch.float16)
        sc = {"g_suh": signs(hidden), "u_suh": signs(hidden), "g_svh": signs(inter, std), "u_svh": signs(inter, std),
              "d_suh": signs(inter), "d_svh": signs(hidden, std)}
        bank = cls(codes(hidden, inter), codes(hidden, inter), codes(inter, hidden), sc, bits, e0, inter, hidden)
        return bank.to(device)

    def to(self, device):
        return EXL3ExpertBank(self.gate.to(device), self.up.to(device), self.down.to(device),
                              {k: v.to(device) for k, v in self.s.items()}, self.bits, self.e0, self.inter, self.hidden, self.cb)

    def nbytes(self) -> int:
        return (self.gate.numel() + self.up.numel() + self.down.numel()) * 2 + sum(v.numel() * 2 for v in self.s.values())

    def dequant(self, which: str, e: int) -> torch.Tensor:
        """Effective dense weights of expert ``e`` (rotations and scales included): "gu" -> [2I, H], "dn" -> [H, I]."""
        def eff(codes, su, sv):
            return ex.effective_weight(codes.cpu(), self.bits, su.cpu(), sv.cpu(), self.cb).t().contiguous()
        if which == "gu":
            return torch.cat([eff(self.gate[e], self.s["g_suh"][e], self.s["g_svh"][e]),
                              eff(self.up[e], self.s["u_suh"][e], self.s["u_svh"][e])], 0)
        return eff(self.down[e], self.s["d_suh"][e], self.s["d_svh"][e])

    # ------------------------------------------------------------------------------------------ decode rows
    def routes_decode(self, x: torch.Tensor, ids: torch.Tensor, act: int, limit: float) -> torch.Tensor:
        rows, H = x.shape
        k = ids.shape[1]
        R, I, dev = rows * k, self.inter, x.device
        e = ids.reshape(-1) - self.e0
        e = torch.where((e >= 0) & (e < self.e_local), e, torch.full_like(e, -1)).to(torch.int32).contiguous()
        per_gu, per_dn = self.gate[0].numel(), self.down[0].numel()
        s = self.s
        f16 = torch.float16
        xg = had128(x, s["g_suh"], out_dtype=f16, expert=e, scale_stride=H, in_div=k, rows=R, out=torch.zeros(R, H, dtype=f16, device=dev))
        xu = had128(x, s["u_suh"], out_dtype=f16, expert=e, scale_stride=H, in_div=k, rows=R, out=torch.zeros(R, H, dtype=f16, device=dev))
        ga = exl3_gemv(self.gate, xg, 1, H, I, self.bits, self.cb, out=torch.zeros(R, I, dtype=torch.float32, device=dev),
                       expert=e, expert_stride=per_gu, groups=R)
        ua = exl3_gemv(self.up, xu, 1, H, I, self.bits, self.cb, out=torch.zeros(R, I, dtype=torch.float32, device=dev),
                       expert=e, expert_stride=per_gu, groups=R)
        a = had128(ga, s["g_svh"], post=True, out_dtype=f16, x2=ua, scale2=s["u_svh"], act=act, expert=e, scale_stride=I,
                   rows=R, out=torch.zeros(R, I, dtype=f16, device=dev))
        if limit > 0:
            raise NotImplementedError("clamped gated activation on the EXL3 expert path")
        xd = had128(a, s["d_suh"], out_dtype=f16, expert=e, scale_stride=I, rows=R, out=torch.zeros(R, I, dtype=f16, device=dev))
        da = exl3_gemv(self.down, xd, 1, I, H, self.bits, self.cb, out=torch.zeros(R, H, dtype=torch.float32, device=dev),
                       expert=e, expert_stride=per_dn, groups=R)
        return had128(da, s["d_svh"], post=True, out_dtype=x.dtype, expert=e, scale_stride=H, rows=R,
                      out=torch.zeros(R, H, dtype=x.dtype, device=dev))

    # ------------------------------------------------------------------------------------------ prefill chunks
    def slab_experts(self) -> int:
        per = 3 * self.inter * self.hidden * 2
        return max(1, min(self.e_local, SLAB_BYTES // per))

    def routes_prefill(self, x: torch.Tensor, ids: torch.Tensor, act: int, limit: float) -> torch.Tensor:
        if limit > 0:
            raise NotImplementedError("clamped gated activation on the EXL3 expert path")
        rows, H = x.shape
        k = ids.shape[1]
        R, I, dev = rows * k, self.inter, x.device
        G = self.slab_experts()
        bn = 64 if R // max(1, self.e_local) < 96 else 128
        flat = ids.reshape(-1)
        d_all = torch.zeros(R, H, dtype=x.dtype, device=dev)
        bf = torch.bfloat16
        w_g = torch.empty(G * I, H, dtype=bf, device=dev)
        w_u = torch.empty(G * I, H, dtype=bf, device=dev)
        w_d = torch.empty(G * H, I, dtype=bf, device=dev)
        st = K.status_word(dev)
        s = self.s
        ar = torch.arange(R, device=dev)
        for g0 in range(0, self.e_local, G):
            g = min(G, self.e_local - g0)
            max_tiles = R // bn + g + 1
            inv = torch.empty(R, dtype=torch.int32, device=dev)
            srt = torch.zeros(R, dtype=torch.int32, device=dev)
            tab = torch.empty(max_tiles, 4, dtype=torch.int32, device=dev)
            totals = torch.zeros(2, dtype=torch.int32, device=dev)
            call("moe_sort", "piiiipppip", ptr(flat), R, self.e0 + g0, g, bn, ptr(inv), ptr(srt), ptr(tab), max_tiles, ptr(totals))
            xs = torch.zeros(R, H, dtype=x.dtype, device=dev)
            call("moe_gather", "plppiplii", ptr(x), x.stride(0), ptr(srt), ptr(totals), k, ptr(xs), xs.stride(0), H, R)
            # expert (index into this bank) of every sorted row; rows past the slab's routes carry -1 and are skipped
            e_rows = torch.where(ar < totals[0], flat[srt.long()] - self.e0, torch.full_like(flat, -1)).to(torch.int32).contiguous()
            for codes, out, K_, N in ((self.gate, w_g, H, I), (self.up, w_u, H, I), (self.down, w_d, I, H)):
                call("exl3_reconstruct_batch", "ppiiiii", ptr(codes[g0:g0 + g]), ptr(out), K_, N, self.bits, self.cb, g)
            xg = had128(xs, s["g_suh"], out_dtype=bf, expert=e_rows, scale_stride=H, rows=R, out=torch.zeros(R, H, dtype=bf, device=dev))
            xu = had128(xs, s["u_suh"], out_dtype=bf, expert=e_rows, scale_stride=H, rows=R, out=torch.zeros(R, H, dtype=bf, device=dev))
            ga = torch.zeros(R, I, dtype=bf, device=dev)
            ua = torch.zeros(R, I, dtype=bf, device=dev)
            call("gemm_grouped_bf16", "plplpliiiiipip", ptr(w_g), H, ptr(xg), xg.stride(0), ptr(ga), ga.stride(0), R, g, I, H, bn,
                 ptr(tab), max_tiles, ptr(st))
            call("gemm_grouped_bf16", "plplpliiiiipip", ptr(w_u), H, ptr(xu), xu.stride(0), ptr(ua), ua.stride(0), R, g, I, H, bn,
                 ptr(tab), max_tiles, ptr(st))
            a = had128(ga, s["g_svh"], post=True, out_dtype=bf, x2=ua, scale2=s["u_svh"], act=act, expert=e_rows, scale_stride=I,
                       rows=R, out=torch.zeros(R, I, dtype=bf, device=dev))
            xd = had128(a, s["d_suh"], out_dtype=bf, expert=e_rows, scale_stride=I, rows=R, out=torch.zeros(R, I, dtype=bf, device=dev))
            da = torch.zeros(R, H, dtype=bf, device=dev)
            call("gemm_grouped_bf16", "plplpliiiiipip", ptr(w_d), I, ptr(xd), xd.stride(0), ptr(da), da.stride(0), R, g, H, I, bn,
                 ptr(tab), max_tiles, ptr(st))
            ds = had128(da, s["d_svh"], post=True, out_dtype=x.dtype, expert=e_rows, scale_stride=H, rows=R,
                        out=torch.zeros(R, H, dtype=x.dtype, device=dev))
            mine = inv >= 0
            d_all = torch.where(mine[:, None], ds[inv.clamp(min=0).long()], d_all)
        return d_all

    # ------------------------------------------------------------------------------------------ statement
    def routes_reference(self, x: torch.Tensor, ids: torch.Tensor, act: int, limit: float) -> torch.Tensor:
        rows, H = x.shape
        k = ids.shape[1]
        d = torch.zeros(rows * k, H, dtype=x.dtype)
        s = self.s
        for t in range(rows):
            for j in range(k):
                e = int(ids[t, j]) - self.e0
                if e < 0 or e >= self.e_local:
                    continue
                xt = x[t:t + 1].float()
                g = ex.linear_reference(xt, self.gate[e], self.bits, s["g_suh"][e], s["g_svh"][e], self.cb)
                u = ex.linear_reference(xt, self.up[e], self.bits, s["u_suh"][e], s["u_svh"][e], self.cb)
                a = (torch.nn.functional.silu(g) if act == 0 else torch.nn.functional.gelu(g, approximate="tanh")) * u
                a = a.to(torch.float16).float()                       # the kernels hand the activation on in fp16
                d[t * k + j] = ex.linear_reference(a, self.down[e], self.bits, s["d_suh"][e], s["d_svh"][e], self.cb).to(x.dtype)[0]
        return d

    def routes(self, x: torch.Tensor, ids: torch.Tensor, act: int = 0, limit: float = 0.0) -> torch.Tensor:
        if not x.is_cuda:
            return self.routes_reference(x, ids, act, limit)
        if x.shape[0] <= 16:
            return self.routes_decode(x, ids, act, limit)
        return self.routes_prefill(x, ids, act, limit)
