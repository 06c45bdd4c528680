"""Host side of the persistent decode-step kernel (csrc/cuda/decode_step.cu): builds the op list of one decode step of a
dense GQA decoder (per layer: qkv linear, finalise = split sum + rotary + KV store, split-KV attention, split merge,
o_proj, gate/up, down; then the LM head), the tensor maps of every weight and of the paged KV pools, and the buffers the
stages hand results through, and launches the whole step as one kernel.

The reference runs the same step as a CUDA graph of ~8 kernels per layer plus two all-reduce kernels
(src/models/gemma4.cpp:438-521); here one launch walks the list with one CTA per SM, weights streaming ahead of the
dependency chain.
"""
from __future__ import annotations

import ctypes
import os

import numpy as np
import torch

from .. import _lib
from . import kernels as K

OP_LINEAR, OP_QKV_FIN, OP_ATTN, OP_MERGE, OP_NORMOUT = 0, 1, 2, 3, 4
IN_X, IN_NORM, IN_GATED, IN_EMBED = 0, 1, 2, 3
OUT_PART, OUT_LOGITS, OUT_TICKET = 0, 1, 2
MAXM = 4
CACHE_SLOTS = 20          # k-tiles of one op a CTA keeps expanded (DS_SLOTS of the kernel)

# Off by default: measured on the 27B flagship the persistent step is 5.9 ms on one GPU against 5.0 ms for the
# kernel-per-op graph (each of its six stages per layer costs 5-12 us of dependent L2 round trips: arrival counter, input
# read, operand fill, issue, epilogue, ticket), so the engine opts in with VOLTA_PSTEP=1 / enable().
ENABLED = os.environ.get("VOLTA_PSTEP", "0") == "1"


class enabled:
    """Context manager / switch: ``with decode_step.enabled(True): ...``"""

    def __init__(self, on: bool):
        self.on = on

    def __enter__(self):
        global ENABLED
        self.prev, ENABLED = ENABLED, self.on
        return self

    def __exit__(self, *exc):
        global ENABLED
        ENABLED = self.prev
        return False
COOPERATIVE = os.environ.get("VOLTA_PSTEP_COOP", "1") != "0"


class StepOp(ctypes.Structure):
    """Mirror of ``ve::StepOp``."""
    _fields_ = [("type", ctypes.c_int), ("in_mode", ctypes.c_int), ("out_mode", ctypes.c_int), ("map", ctypes.c_int),
                ("N", ctypes.c_int), ("K", ctypes.c_int), ("upc", ctypes.c_int), ("src", ctypes.c_int),
                ("alpha", ctypes.c_float), ("ws_off", ctypes.c_int), ("ms", ctypes.c_int), ("tk_off", ctypes.c_int),
                ("ncontrib", ctypes.c_int), ("layer", ctypes.c_int), ("hpar", ctypes.c_int), ("ypar", ctypes.c_int),
                ("ar", ctypes.c_int), ("flags", ctypes.c_int), ("wt", ctypes.c_void_p), ("norm_w", ctypes.c_void_p)]


class StepParams(ctypes.Structure):
    """Mirror of ``ve::StepParams``."""
    _fields_ = [(n, ctypes.c_void_p) for n in (
        "ops", "maps", "cnt", "ctrl", "tickets", "ws", "ybuf", "hbuf", "qbuf", "attn_out", "o_part", "lse_part", "xfinal",
        "logits", "ids", "pos", "slot", "page_table", "embed", "kpool", "vpool", "status", "prof", "dbg")] + [
        ("peer", ctypes.c_void_p * 8), ("seq", ctypes.c_void_p),
        ("off_ll", ctypes.c_ulonglong), ("ll_row_bytes", ctypes.c_ulonglong), ("budget_ns", ctypes.c_ulonglong),
        ("ldl", ctypes.c_long), ("pool_layer_rows", ctypes.c_long)] + [(n, ctypes.c_int) for n in (
        "nops", "kmap", "vmap", "M", "H", "nq", "nkv", "S", "max_pages", "vocab", "rot", "act", "rank", "size", "n_ar",
        "prof_cta", "ns", "scr")] + [(n, ctypes.c_float) for n in ("eps", "wbias", "scale_log2", "rope_theta", "act_limit", "embed_scale")]


_sizes = None


def native_sizes():
    global _sizes
    if _sizes is None:
        out = (ctypes.c_int * 4)()
        _lib.kernels().ve_decode_step_sizes(out)
        _sizes = tuple(out)
        assert _sizes[0] == ctypes.sizeof(StepOp) and _sizes[1] == ctypes.sizeof(StepParams), \
            (_sizes, ctypes.sizeof(StepOp), ctypes.sizeof(StepParams))
    return _sizes


def _tmap(base: int, dtype: int, elem: int, rows: int, cols: int, pitch: int, box_rows: int, box_cols: int) -> bytes:
    buf = (ctypes.c_uint8 * 128)()
    fn = _lib.kernels().ve_make_tmap_2d
    fn.argtypes = [ctypes.c_void_p, ctypes.c_void_p, ctypes.c_int, ctypes.c_int, ctypes.c_long, ctypes.c_long,
                   ctypes.c_long, ctypes.c_int, ctypes.c_int, ctypes.c_int]
    rc = fn(buf, base, dtype, elem, rows, cols, pitch, box_rows, box_cols, 1)
    if rc:
        raise _lib.NativeError(f"tensor map encode failed ({rc})")
    return bytes(buf)


def padded_atoms(lin) -> torch.Tensor:
    """Scale atoms [N/128][ceil(K/256)*4][512] of an NVFP4 linear: k-groups padded with zero scales so that a 256-wide
    k-tile always owns four atoms (K that is a multiple of 128 but not of 256 ends in a half tile)."""
    from ..quant import nvfp4 as qn
    a = qn.scales_atoms_512(lin.scales)
    N, Kk = lin.out_features, lin.in_features
    nkg = Kk // 64
    a = a.reshape(N // 128, nkg, 512)
    pad = (-nkg) % 4
    if pad:
        a = torch.cat([a, torch.zeros(N // 128, pad, 512, dtype=a.dtype, device=a.device)], 1).contiguous()
    return a


def weight_units(lin) -> torch.Tensor:
    """The weight of an NVFP4 linear as the step kernel streams it: [N/128][ceil(K/256)][18432] bytes, each unit the
    128 x 128 B tile of packed codes laid out as the 128-byte swizzle puts it in shared memory (16-byte chunk c of row r
    at chunk c ^ (r & 7)), followed by the tile's four 512 B scale atoms. Units of one tile row follow each other, so a
    CTA's run of units is one contiguous read."""
    N, Kk = lin.out_features, lin.in_features
    NT, KT = N // 128, (Kk + 255) // 256
    pk = lin.packed
    if pk.shape[1] != KT * 128:
        pk = torch.cat([pk, torch.zeros(N, KT * 128 - pk.shape[1], dtype=pk.dtype, device=pk.device)], 1)
    src = pk.view(NT, 16, 8, KT, 8, 16)                     # tile, row group, row in group, k-tile, chunk, byte
    out = torch.empty(NT, KT, 18432, dtype=torch.uint8, device=pk.device)
    dst = out[:, :, :16384].view(NT, KT, 16, 8, 8, 16)      # tile, k-tile, row group, row in group, chunk, byte
    ch = torch.arange(8, device=pk.device)
    for j in range(8):
        dst[:, :, :, j] = src[:, :, j].index_select(3, ch ^ j).permute(0, 2, 1, 3, 4)
    out[:, :, 16384:] = padded_atoms(lin).reshape(NT, KT, 2048)
    return out


def _splits(NT: int, KT: int, upc: int) -> int:
    """Most CTAs that share one tile when units are dealt in runs of ``upc``."""
    return max(((t + 1) * KT - 1) // upc - (t * KT) // upc + 1 for t in range(NT))


class StepProgram:
    """Op list, tensor maps and buffers of one decode step of ``model`` with ``rows`` rows on cache ``kv``."""

    def __init__(self, model, kv, rows: int):
        from .linear import LinearNVFP4
        native_sizes()
        cfg, dev = model.cfg, model.device
        self.model, self.kv, self.M = model, kv, rows
        self.G = torch.cuda.get_device_properties(dev).multi_processor_count
        G, M = self.G, rows
        H, nq, nkv = cfg.hidden, model.nq, model.nkv
        self.S = max(1, G // (M * nkv))
        comm = model.comm
        tp = comm.size
        self.head = isinstance(model.lm_head, LinearNVFP4)
        ops: list[StepOp] = []
        maps: list[bytes] = []
        self._keep = []                       # tensors referenced by address
        ws_off, tk_off = {}, {}
        ws_total = tk_total = 0
        n_ar = 0
        y_count = 0
        norm_count = 0

        def linear(lin, kind, li, in_mode, out_mode, src, norm_w=None, flags=0):
            nonlocal ws_total, tk_total, n_ar, y_count, norm_count
            N, Kk = lin.out_features, lin.in_features
            assert N % 128 == 0 and Kk % 128 == 0
            NT, KT = N // 128, (Kk + 255) // 256
            U = NT * KT
            upc = KT * ((NT + G - 1) // G) if out_mode == OUT_LOGITS else (U + G - 1) // G
            o = StepOp()
            o.type, o.in_mode, o.out_mode, o.N, o.K, o.upc, o.src, o.layer = OP_LINEAR, in_mode, out_mode, N, Kk, upc, src, li
            o.alpha = float(lin.gscale)
            o.ms = _splits(NT, KT, upc)
            if kind not in ws_off:
                ws_off[kind] = ws_total
                ws_total += NT * o.ms * MAXM * 128
                tk_off[kind] = tk_total
                tk_total += NT
            o.ws_off, o.tk_off = ws_off[kind], tk_off[kind]
            o.ncontrib = NT if out_mode == OUT_TICKET else (U + upc - 1) // upc
            if min(KT, upc) > CACHE_SLOTS:
                raise ValueError(f"{kind}: {min(KT, upc)} k-tiles per CTA exceed the kernel's operand cache")
            units = getattr(lin, "_step_units", None)        # built once per weight, shared by the programs of all row counts
            if units is None:
                units = lin._step_units = weight_units(lin)
            o.wt = units.data_ptr()
            if norm_w is not None:
                o.norm_w = norm_w.data_ptr()
            if in_mode == IN_EMBED:
                o.hpar = 1
            elif in_mode == IN_NORM:
                o.hpar = norm_count & 1
                norm_count += 1
            if out_mode == OUT_TICKET:
                o.ypar = y_count & 1
                y_count += 1
                o.ar = n_ar
                n_ar += 1
            o.flags = flags
            ops.append(o)
            return len(ops) - 1

        def small(tp_, src, li, ncontrib):
            o = StepOp()
            o.type, o.src, o.layer, o.ncontrib = tp_, src, li, ncontrib
            ops.append(o)
            return len(ops) - 1

        prev = -1
        heads = nq + 2 * nkv
        for li, L in enumerate(model.layers):
            qkv = linear(L.qkv, "qkv", li, IN_EMBED if li == 0 else IN_NORM, OUT_PART, prev, L.attn_norm)
            att = small(OP_ATTN, qkv, li, min(G, M * nkv * self.S))     # finalises q / k / v of the projection itself
            mrg = small(OP_MERGE, att, li, min(G, M * nq))
            op_o = linear(L.o_proj, "o", li, IN_X, OUT_TICKET, mrg)
            gu = linear(L.gate_up, "gu", li, IN_NORM, OUT_PART, op_o, L.ffn_norm)
            prev = linear(L.down, "down", li, IN_GATED, OUT_TICKET, gu)
        if self.head:
            linear(model.lm_head, "head", len(model.layers), IN_NORM, OUT_LOGITS, prev, model.final_norm, flags=1)
        else:
            o = StepOp()
            o.type, o.in_mode, o.src, o.flags = OP_NORMOUT, IN_NORM, prev, 1
            o.norm_w = model.final_norm.data_ptr()
            o.hpar = norm_count & 1
            norm_count += 1
            ops.append(o)
        self.final_hpar = ops[-1].hpar ^ 1
        self.nops = len(ops)
        self.n_ar = n_ar
        # K / V pool maps
        Lk, pages = kv.k.shape[0], kv.k.shape[1]
        rows_total = Lk * pages * nkv * 64
        kmap = len(maps)
        maps.append(_tmap(kv.k.data_ptr(), 1, 2, rows_total, 128, 256, 64, 64))
        maps.append(_tmap(kv.v.data_ptr(), 1, 2, rows_total, 128, 256, 64, 64))
        u8 = torch.uint8
        self.d_ops = torch.frombuffer(bytearray(b"".join(bytes(o) for o in ops)), dtype=u8).to(dev)
        self.d_maps = torch.frombuffer(bytearray(b"".join(maps)), dtype=u8).to(dev)
        assert self.d_maps.data_ptr() % 64 == 0
        self.cnt = torch.zeros(self.nops + 8, dtype=torch.int32, device=dev)
        self.ctrl = torch.zeros(8, dtype=torch.int32, device=dev)
        self.tickets = torch.zeros(max(1, tk_total), dtype=torch.int32, device=dev)
        self.ws = torch.empty(max(1, ws_total), dtype=torch.float32, device=dev)
        bf = torch.bfloat16
        self.ybuf = torch.zeros(2, MAXM, H, dtype=bf, device=dev)
        self.hbuf = torch.zeros(2, MAXM, H, dtype=bf, device=dev)
        self.qbuf = torch.zeros(MAXM, nq * 128, dtype=bf, device=dev)
        self.attn_out = torch.zeros(MAXM, nq * 128, dtype=bf, device=dev)
        self.o_part = torch.zeros(MAXM * nq * self.S * 128, dtype=torch.float32, device=dev)
        self.lse_part = torch.zeros(MAXM * nq * self.S, dtype=torch.float32, device=dev)
        self.xfinal = torch.zeros(MAXM, H, dtype=bf, device=dev)
        self.logits = torch.zeros(MAXM, model.vocab_local, dtype=torch.float32, device=dev) if self.head else None
        p = StepParams()
        p.ops, p.maps, p.cnt, p.ctrl = self.d_ops.data_ptr(), self.d_maps.data_ptr(), self.cnt.data_ptr(), self.ctrl.data_ptr()
        p.tickets, p.ws, p.ybuf, p.hbuf = self.tickets.data_ptr(), self.ws.data_ptr(), self.ybuf.data_ptr(), self.hbuf.data_ptr()
        p.qbuf, p.attn_out, p.o_part, p.lse_part = (self.qbuf.data_ptr(), self.attn_out.data_ptr(), self.o_part.data_ptr(),
                                                    self.lse_part.data_ptr())
        p.xfinal = self.xfinal.data_ptr()
        p.logits = self.logits.data_ptr() if self.head else 0
        p.page_table, p.embed = kv.page_table.data_ptr(), model.embed.data_ptr()
        p.kpool, p.vpool = kv.k.data_ptr(), kv.v.data_ptr()
        p.status = K.status_word(dev).data_ptr()
        self.dbg = torch.zeros(8 + 6 * 1000, dtype=torch.int32, device=dev)
        p.dbg = self.dbg.data_ptr()
        p.ldl = model.vocab_local
        p.pool_layer_rows = pages * nkv * 64
        p.nops, p.kmap, p.vmap, p.M, p.H, p.nq, p.nkv, p.S = self.nops, kmap, kmap + 1, M, H, nq, nkv, self.S
        p.max_pages, p.vocab, p.rot = kv.page_table.shape[1], model.embed.shape[0], model.rot
        p.act = 1 if cfg.act == "silu" else 2
        p.rank, p.size, p.n_ar = comm.rank, tp, n_ar
        p.eps, p.wbias, p.scale_log2 = cfg.rms_eps, cfg.norm_bias, model.scale * 1.4426950408889634
        p.rope_theta, p.act_limit, p.embed_scale = cfg.rope_theta, cfg.act_limit, cfg.embed_scale
        if tp > 1:
            a = comm.args
            for i in range(8):
                p.peer[i] = a.peer[i]
            p.seq, p.off_ll, p.ll_row_bytes, p.budget_ns = a.seq, a.off_ll, a.ll_row_bytes, a.budget_ns
        self.params = p

    def enable_profile(self, cta: int = 0):
        """Per-op device timestamps of one CTA (ns): op entered, input ready, units done, op left."""
        self.prof = torch.zeros(self.nops, 4, dtype=torch.int64, device=self.dbg.device)
        self.params.prof, self.params.prof_cta = self.prof.data_ptr(), cta
        return self.prof

    def reset(self):
        """Host-side recovery after a step that gave up on a wait: arrival counters and tickets back to zero."""
        self.cnt.zero_()
        self.ctrl.zero_()
        self.tickets.zero_()

    def run(self, ids, pos, slot):
        """Launch one step for the rows described by the device tensors ``ids`` / ``pos`` / ``slot`` (int32, >= M entries).
        Returns (logits [M, vocab_local] fp32 or None, normalised final hidden [M, H], residual [M, H])."""
        p = self.params
        p.ids, p.pos, p.slot = ids.data_ptr(), pos.data_ptr(), slot.data_ptr()
        _lib.call("decode_step", "pii", ctypes.addressof(p), self.G, 1 if COOPERATIVE else 0)
        M = self.M
        return (self.logits[:M] if self.head else None), self.xfinal[:M], self.hbuf[self.final_hpar, :M]


def supported(model, b, kv) -> bool:
    """True when the rows of ``b`` can run as one persistent step on ``model``."""
    from .linear import LinearNVFP4
    from ..runtime.batch import LOGITS_ALL
    if not ENABLED or type(model).__name__ != "DenseModel" or not model.embed.is_cuda:
        return False
    cfg = model.cfg
    if b.n > MAXM or b.n * cfg.hidden * 2 > 40960 or b.logits != LOGITS_ALL or b.tiles is not None or b.key_end is not None:
        return False
    if b.pos3 is not None or b.embeds is not None or b.slot is None or getattr(b, "tree", None) is not None:
        return False
    ok = getattr(model, "_pstep_static", None)
    if ok is None:
        comm = model.comm
        ok = (cfg.residual == "plain" and not cfg.sandwich_norm and not cfg.qk_norm and not cfg.rope_interleaved
              and cfg.head_dim == 128 and cfg.sliding_window == 0 and cfg.logit_softcap == 0 and not cfg.mrope_sections
              and cfg.hidden % 128 == 0 and cfg.act in ("silu", "gelu_tanh") and model.rot % 2 == 0
              and model.nq // model.nkv <= 16 and (comm.size == 1 or hasattr(comm, "args")))
        for L in model.layers:
            for lin in (L.qkv, L.o_proj, L.gate_up, L.down):
                ok = ok and isinstance(lin, LinearNVFP4) and lin.packed.is_cuda and lin.out_features % 128 == 0 \
                    and lin.in_features % 128 == 0
            ok = ok and getattr(L.gate_up, "gated", False)
        if ok:
            G = torch.cuda.get_device_properties(model.device).multi_processor_count
            lins = [lin for L in model.layers for lin in (L.qkv, L.o_proj, L.gate_up, L.down)]
            if isinstance(model.lm_head, LinearNVFP4):
                lins.append(model.lm_head)
            for lin in lins:
                NT, KT = lin.out_features // 128, (lin.in_features + 255) // 256
                upc = KT * ((NT + G - 1) // G) if lin is model.lm_head else (NT * KT + G - 1) // G
                ok = ok and min(KT, upc) <= CACHE_SLOTS
        model._pstep_static = bool(ok)
    if not ok or kv.fmt != 0 or kv.head_dim != 128 or kv.v_head_dim != 128:
        return False
    return (getattr(model, "steer", None) is None and getattr(model, "tap_ring", None) is None
            and getattr(model, "hess", None) is None)


def program_for(model, kv, rows: int) -> StepProgram:
    cache = model.__dict__.setdefault("_pstep_programs", {})
    key = (id(kv), rows)
    prog = cache.get(key)
    if prog is None:
        prog = cache[key] = StepProgram(model, kv, rows)
    return prog
