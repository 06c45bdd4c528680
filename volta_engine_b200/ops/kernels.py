"""Op entry points. CUDA tensors go to the hand-written sm_100a kernels (libvolta_kernels.so, mandatory on
a GPU machine: a missing library raises); CPU tensors run the fp32 PyTorch oracle in
:mod:`volta_engine_b200.ops.reference` so host-side logic can be tested without a GPU.
"""
from __future__ import annotations

import ctypes
import os

import torch

from .. import _lib
from .._lib import call, ptr
from . import reference as ref

PAGE = ref.PAGE

_status = {}


def _lib_kernels():
    return _lib.kernels()
_scratch_registry = {}


def use_scratch(registry, device) -> None:
    """Kernel workspaces of ``device`` created after this call are carved from ``registry``
    (``runtime.arena.ScratchRegistry``) instead of the caching allocator: one device allocation per process, stable
    addresses for graph replay. ``None`` restores the allocator."""
    if registry is None:
        _scratch_registry.pop(str(device), None)
    else:
        _scratch_registry[str(device)] = registry


def _ws(name, shape, dtype, device, zero=False):
    reg = _scratch_registry.get(str(device))
    if reg is None:
        return (torch.zeros if zero else torch.empty)(shape, dtype=dtype, device=device)
    t = reg.typed(name, shape if isinstance(shape, tuple) else (shape,), dtype)
    return t.zero_() if zero else t


def status_word(device) -> torch.Tensor:
    """Per-device int32 word that kernels set when a bounded wait expires (0 = healthy)."""
    key = str(device)
    t = _status.get(key)
    if t is None:
        t = torch.zeros(1, dtype=torch.int32, device=device)
        _status[key] = t
    return t


def check_status(device) -> int:
    t = _status.get(str(device))
    return int(t.item()) if t is not None else 0


# ---------------------------------------------------------------------------------------------- norms
def rmsnorm(x, w, eps, wbias=0.0, residual=None, out=None):
    """out = RMSNorm(residual + x) * (w + wbias); residual updated in place when given."""
    if not x.is_cuda:
        o, r = ref.rmsnorm(x, w, eps, wbias, residual)
        if residual is not None:
            residual.copy_(r)
        if out is not None:
            out.copy_(o)
            return out
        return o
    rows, H = x.shape
    if out is None:
        out = torch.empty_like(x)
    call("rmsnorm", "ppippiiffll", ptr(x), ptr(residual),
         1 if (residual is not None and residual.dtype == torch.float32) else 0, ptr(w), ptr(out), rows, H,
         float(eps), float(wbias), x.stride(0), out.stride(0))
    return out


def rmsnorm_heads_(x, w, rows, heads, hd, row_stride, eps, wbias=0.0, offset=0):
    """In-place per-head RMSNorm over ``heads`` heads starting ``offset`` elements into each row."""
    if not x.is_cuda:
        v = x[:, offset: offset + heads * hd]
        x[:, offset: offset + heads * hd] = ref.rmsnorm_heads(v, w, heads, hd, eps, wbias)
        return x
    call("rmsnorm_heads", "ppiiilff", x.data_ptr() + offset * x.element_size(), ptr(w), rows, heads, hd,
         row_stride, float(eps), float(wbias))
    return x


def embed(ids, table, out=None, scale=1.0):
    if not table.is_cuda:
        o = (table[ids.long()].float() * scale).to(table.dtype)
        if out is not None:
            out.copy_(o)
            return out
        return o
    rows = ids.numel()
    V, H = table.shape
    if out is None:
        out = torch.empty(rows, H, dtype=table.dtype, device=table.device)
    call("embed", "pppiiif", ptr(ids), ptr(table), ptr(out), rows, H, V, float(scale))
    return out


def rope_store(qkv, pos, slot, page_table, kpool, vpool, nq, nkv, hd, rot_dim, theta, interleaved=False,
               pos_scale=1.0, mrope=None):
    """Rotate q, k inside ``qkv`` in place and write k, v rows into the paged cache. ``mrope`` = (pos3 [3, rows] int32,
    (s0, s1)): multimodal rotary embedding with time / height / width sections of s0 / s1 / rest rotary pairs."""
    fmt = kv_format_of(kpool)
    if not qkv.is_cuda:
        if fmt >= 2:
            _rope_store_quant_cpu(qkv, pos, slot, page_table, kpool, vpool, nq, nkv, hd, rot_dim, theta, interleaved,
                                  pos_scale, mrope, fmt)
            return
        ref.rope_store(qkv, pos, slot, page_table, kpool, vpool, nq, nkv, hd, rot_dim, theta, interleaved,
                       pos_scale, mrope)
        return
    rows = qkv.shape[0]
    pos3, (s0, s1) = mrope if mrope is not None else (None, (0, 0))
    # scaled formats: the rotation kernel leaves the rotated keys in ``qkv`` (store code 2 = no cache write) and the
    # quantising store kernel writes bytes and scales
    call("rope_store", "ppppippiiiiififipii", ptr(qkv), ptr(pos), ptr(slot), ptr(page_table), page_table.shape[1],
         ptr(kpool), ptr(vpool), rows, nq, nkv, hd, rot_dim, float(theta), 1 if interleaved else 0,
         float(pos_scale), 2 if fmt >= 2 else fmt, ptr(pos3), s0, s1)
    if fmt >= 2:
        call("kv_quant_store", "plpppippppiiiii", ptr(qkv), qkv.stride(0), ptr(pos), ptr(slot), ptr(page_table),
             page_table.shape[1], ptr(kpool), ptr(vpool), ptr(kpool.kv_scale), ptr(vpool.kv_scale), rows, nq, nkv, hd, fmt)


def kv_format_of(pool) -> int:
    """0 bf16, 1 E5M2, 2 k8v4, 3 nvfp4 (the scaled formats are tagged on the pool tensors by the cache)."""
    f = getattr(pool, "kv_fmt", None)
    if f is not None:
        return f
    return 1 if pool.dtype == torch.float8_e5m2 else 0


def _rope_store_quant_cpu(qkv, pos, slot, page_table, kpool, vpool, nq, nkv, hd, rot_dim, theta, interleaved, pos_scale,
                          mrope, fmt):
    from ..quant import kv_codec as C
    rows = qkv.shape[0]
    q = qkv[:, : nq * hd].reshape(rows, nq, hd)
    k = qkv[:, nq * hd:(nq + nkv) * hd].reshape(rows, nkv, hd)
    v = qkv[:, (nq + nkv) * hd:(nq + 2 * nkv) * hd].reshape(rows, nkv, hd)
    qkv[:, : nq * hd] = ref.rope_rotate(q, pos, rot_dim, theta, interleaved, pos_scale, mrope).reshape(rows, -1)
    kr = ref.rope_rotate(k, pos, rot_dim, theta, interleaved, pos_scale, mrope)
    qkv[:, nq * hd:(nq + nkv) * hd] = kr.reshape(rows, -1)
    kq, vq = C.FORMATS[fmt]
    kd, ks = C.encode(kr, kq)
    vd, vs = C.encode(v, vq)
    for r in range(rows):
        s = int(slot[r]) if slot is not None else 0
        if s < 0:
            continue
        p = int(pos[r])
        page = int(page_table[s, p // 64])
        kpool[page, :, p % 64], kpool.kv_scale[page, :, p % 64] = kd[r], ks[r]
        vpool[page, :, p % 64], vpool.kv_scale[page, :, p % 64] = vd[r], vs[r]


def _dequant_pools(kpool, vpool, hd):
    """bf16 copies of scaled-format pools (CPU path)."""
    from ..quant import kv_codec as C
    kq, vq = C.FORMATS[kpool.kv_fmt]
    return (C.decode(kpool, kpool.kv_scale, kq, hd).to(torch.bfloat16), C.decode(vpool, vpool.kv_scale, vq, hd).to(torch.bfloat16))


def gated_act(gu, I, act=0, limit=0.0, out=None, interleave=0):
    """act(gate) * up. ``interleave=64``: the row holds [64 gate | 64 up] per 128 columns instead of [all gate | all up]."""
    if not gu.is_cuda:
        if interleave:
            v = gu.reshape(gu.shape[0], -1, 2, interleave)
            gu = torch.cat([v[:, :, 0].reshape(gu.shape[0], I), v[:, :, 1].reshape(gu.shape[0], I)], 1)
        o = ref.gated_act(gu, I, act, limit)
        if out is not None:
            out.copy_(o)
            return out
        return o
    rows = gu.shape[0]
    if out is None:
        out = torch.empty(rows, I, dtype=gu.dtype, device=gu.device)
    call("gated_act", "ppliifi", ptr(gu), ptr(out), rows, I, act, float(limit), interleave)
    return out


def add_(a, b):
    if not a.is_cuda:
        a.add_(b)
        return a
    call("add", "ppl", ptr(a), ptr(b), a.numel())
    return a


# ---------------------------------------------------------------------------------------------- attention
# decode / verify tiles: 104 = four warps that split the keys of every page (default), 1 = one warp per tile
ATTN_DECODE_WARPS = 1 if os.environ.get("VOLTA_ATTN_DECODE", "ksplit") == "1warp" else 104
# "fused": the split CTA that finishes last merges the partials itself. Measured slower than the parallel merge kernel
# (one CTA walks 32 splits x 5 heads serially: 166 vs 192 tok/s on the 27B decode), so the kernel form is the default.
ATTN_FUSED_MERGE = os.environ.get("VOLTA_ATTN_MERGE", "kernel") == "fused"
# prefill tiles on the tcgen05 kernel where it applies (bf16 cache, head_dim 128); "mma" keeps the mma.sync kernel
ATTN_PREFILL_TC = os.environ.get("VOLTA_ATTN_PREFILL", "tc") != "mma"


class AttnWorkspace:
    """Split-KV partial buffers, allocated once (stable pointers for CUDA-graph replay)."""

    def __init__(self, max_rows, nq, hd, max_splits, device):
        self.max_splits = max_splits
        self.o_part = torch.empty(max_rows * nq * max_splits * hd, dtype=torch.float32, device=device)
        self.lse_part = torch.empty(max_rows * nq * max_splits, dtype=torch.float32, device=device)
        self.tickets = torch.zeros(max_rows * nq, dtype=torch.int32, device=device)   # (tile, kv head) arrival counters


def attention(q, pos, slot, page_table, kpool, vpool, nq, nkv, hd, scale, *, out=None, window=0, key_end=None,
              gate=None, tiles=None, nsplit=1, ws: AttnWorkspace | None = None, tree=None):
    """Paged GQA attention. ``q`` is the (rotated) fused qkv buffer [rows, >= nq*hd].

    ``tiles`` = (tile_first, tile_count, ntiles[, wide]) int32 device tensors grouping consecutive rows of one
    sequence for prefill (<= 64 // G tokens per tile); None = one row per tile (decode / verify). ``wide`` is the same
    grouping at <= 128 // G tokens per tile: with a bf16 cache and head_dim 128 the prefill runs on the tcgen05 kernel
    (128 query rows per CTA, accumulators in TMEM), otherwise on the mma.sync kernel over the 64-row tiles.
    ``tree`` = (base int32 [rows], mask int64 [rows]): rows of a verification tree. Keys at cache positions >= base[r]
    are the tree's own nodes and row r sees node j only if bit j of mask[r] is set (its ancestors and itself).
    """
    rows = q.shape[0]
    fmt = kv_format_of(kpool)
    if not q.is_cuda:
        if fmt >= 2:
            kpool, vpool = _dequant_pools(kpool, vpool, hd)
        o = ref.attention(q, pos, slot, page_table, kpool, vpool, nq, nkv, hd, scale, window, key_end, gate, tree)
        if out is not None:
            out.copy_(o)
            return out
        return o
    if out is None:
        out = torch.empty(rows, nq * hd, dtype=q.dtype, device=q.device)
    if tiles is None:
        tf = tc = None
        ntiles, warps = rows, ATTN_DECODE_WARPS
    else:
        tf, tc, ntiles = tiles[:3]
        warps = 4
        if (ATTN_PREFILL_TC and len(tiles) > 3 and tiles[3] is not None and hd == 128 and fmt == 0 and nsplit == 1
                and q.data_ptr() % 16 == 0 and q.stride(0) % 8 == 0 and out.data_ptr() % 16 == 0 and out.stride(0) % 8 == 0
                and (gate is None or (gate.data_ptr() % 16 == 0 and gate.stride(0) % 8 == 0))):
            tf, tc, ntiles = tiles[3]
            warps = 8
    if fmt >= 2 and warps == 1:
        warps = 104                      # the scaled formats are built for the four-warp kernels
    if nsplit > 1 and ws is None:
        raise ValueError("split-KV attention needs a workspace")
    assert tree is None or tiles is None, "tree rows are decode / verify rows"
    call("attention", "plplplpppppppiipippliiiifiiipppppp",
         ptr(q), q.stride(0), ptr(out), out.stride(0), ptr(gate), gate.stride(0) if gate is not None else 0,
         ptr(ws.o_part) if ws else 0, ptr(ws.lse_part) if ws else 0, ptr(pos), ptr(slot), ptr(key_end),
         ptr(tf), ptr(tc), ntiles, rows, ptr(page_table), page_table.shape[1], ptr(kpool), ptr(vpool),
         kpool.shape[0], nq, nkv, hd, nsplit, float(scale), window, warps,
         fmt, ptr(kpool.kv_scale) if fmt >= 2 else 0, ptr(vpool.kv_scale) if fmt >= 2 else 0,
         ptr(ws.tickets) if (ws is not None and ATTN_FUSED_MERGE) else 0,
         ptr(tree[0]) if tree is not None else 0, ptr(tree[1]) if tree is not None else 0, ptr(status_word(q.device)))
    return out


def make_prefill_tiles(slots, G, device, max_rows_per_tile=64, wide=True):
    """Host helper: group consecutive rows with the same slot into tiles of <= 64 // G tokens; ``wide`` appends the
    grouping at <= 128 // G tokens (what the tcgen05 prefill kernel takes) as a fourth element."""
    if wide and max_rows_per_tile == 64 and G <= 128:
        return make_prefill_tiles(slots, G, device, 64, False) + (make_prefill_tiles(slots, G, device, 128, False),)
    per = max(1, max_rows_per_tile // G)
    first, count = [], []
    i, n = 0, len(slots)
    while i < n:
        j = i
        while j < n and slots[j] == slots[i] and j - i < per:
            j += 1
        first.append(i)
        count.append(j - i)
        i = j
    tf = torch.tensor(first, dtype=torch.int32, device=device)
    tc = torch.tensor(count, dtype=torch.int32, device=device)
    return tf, tc, len(first)


# ---------------------------------------------------------------------------------------------- sampling
_argmax_scratch = {}
ARGMAX_NB = 64
def argmax(logits, id_offset=0, idx_out=None, val_out=None):
    if not logits.is_cuda:
        i, v = ref.argmax(logits, id_offset)
        if idx_out is not None:
            idx_out.copy_(i)
            if val_out is not None:
                val_out.copy_(v)
            return idx_out, val_out
        return i, v
    rows, V = logits.shape
    if idx_out is None:
        idx_out = torch.empty(rows, dtype=torch.int32, device=logits.device)
    if val_out is None:
        val_out = torch.empty(rows, dtype=torch.float32, device=logits.device)
    if V >= 8192 and rows <= 64:
        key = str(logits.device)
        sc = _argmax_scratch.get(key)
        if sc is None:
            sc = (torch.empty(64 * ARGMAX_NB, dtype=torch.float32, device=logits.device),
                  torch.empty(64 * ARGMAX_NB, dtype=torch.int32, device=logits.device))
            _argmax_scratch[key] = sc
        call("argmax2", "pliiippppi", ptr(logits), logits.stride(0), rows, V, id_offset, ptr(idx_out), ptr(val_out),
             ptr(sc[0]), ptr(sc[1]), ARGMAX_NB)
    else:
        call("argmax", "pliiipp", ptr(logits), logits.stride(0), rows, V, id_offset, ptr(idx_out), ptr(val_out))
    return idx_out, val_out


def topk(logits, k=16, id_offset=0):
    """-> (ids [rows,k] int32, vals [rows,k] fp32 descending, lse [rows])."""
    if not logits.is_cuda:
        return ref.topk(logits, k, id_offset)
    rows, V = logits.shape
    ids = torch.empty(rows, k, dtype=torch.int32, device=logits.device)
    vals = torch.empty(rows, k, dtype=torch.float32, device=logits.device)
    lse = torch.empty(rows, dtype=torch.float32, device=logits.device)
    call("topk", "pliiiippp", ptr(logits), logits.stride(0), rows, V, id_offset, k, ptr(ids), ptr(vals), ptr(lse))
    return ids, vals, lse


# ---------------------------------------------------------------------------------------------- NVFP4
def nvfp4_dequant(packed, scales, gscale, out=None):
    N, K2 = packed.shape
    K = K2 * 2
    if not packed.is_cuda:
        from ..quant import nvfp4 as q
        return q.dequantize_nvfp4(packed, scales, gscale).to(torch.bfloat16)
    if out is None:
        out = torch.empty(N, K, dtype=torch.bfloat16, device=packed.device)
    call("nvfp4_dequant", "ppfpli", ptr(packed), ptr(scales), float(gscale), ptr(out), N, K)
    return out


def nvfp4_quant_rows(x, blocked=True):
    """Activation rows -> (packed [T,K/2], scales). blocked=True gives 512 B tensor-core atoms."""
    T, K = x.shape
    if not x.is_cuda:
        from ..quant import nvfp4 as q
        p, s = q.quantize_rows_nvfp4(x)
        return p, (q.scales_atoms_512(s) if blocked else s)
    xp = torch.empty(T, K // 2, dtype=torch.uint8, device=x.device)
    if blocked:
        xs = torch.zeros((T + 127) // 128, K // 64, 512, dtype=torch.uint8, device=x.device)
    else:
        xs = torch.empty(T, K // 16, dtype=torch.uint8, device=x.device)
    call("nvfp4_quant_rows", "plppiifi", ptr(x), x.stride(0), ptr(xp), ptr(xs), T, K, 1.0, 1 if blocked else 0)
    return xp, xs


def nvfp4_gemv(packed, scales, gscale, x, out=None, residual=None):
    """x [M<=16.., K] bf16 -> out [M, N] bf16 (CUDA-core streaming mat-vec)."""
    N, K2 = packed.shape
    K = K2 * 2
    M = x.shape[0]
    if out is None:
        out = torch.empty(M, N, dtype=torch.bfloat16, device=x.device)
    call("nvfp4_gemv", "ppfplplpliii", ptr(packed), ptr(scales), float(gscale), ptr(x), x.stride(0), ptr(out),
         out.stride(0), ptr(residual), residual.stride(0) if residual is not None else 0, M, N, K)
    return out


_gv_scratch = {}


def gv_scratch(device):
    """Per-device split-K scratch of the tensor-core mat-vec: (fp32 partials, zeroed arrival counters)."""
    key = str(device)
    t = _gv_scratch.get(key)
    if t is None:
        t = (_ws("gemv/partials", GV_WS_ROWS * 16, torch.float32, device),
             _ws("gemv/counters", 4096, torch.int32, device, zero=True))
        _gv_scratch[key] = t
    return t


GV_WS_ROWS = 1 << 16  # KS * N may not exceed this


def gv_splits(N: int, K: int) -> int:
    ctas = N // 16
    ks = max(1, min(8, -(-148 * 6 // ctas)))
    ks = min(ks, max(1, (K // 64) // 4))
    while ks > 1 and ks * N > GV_WS_ROWS:
        ks -= 1
    return ks


def nvfp4_gemv_mma(wg, sg, gscale, x, N, K, out=None, residual=None, ks=None):
    """Decode / verify mat-vec (M <= 16) on the prepacked GV layout: out [M, N] bf16."""
    M = x.shape[0]
    if out is None:
        out = torch.empty(M, N, dtype=torch.bfloat16, device=x.device)
    if ks is None:
        ks = gv_splits(N, K)
    ws, cnt = gv_scratch(x.device)
    assert N // 16 <= cnt.numel()
    call("nvfp4_gemv_mma", "ppfplplpliiiipp", ptr(wg), ptr(sg), float(gscale), ptr(x), x.stride(0), ptr(out),
         out.stride(0), ptr(residual), residual.stride(0) if residual is not None else 0, M, N, K, ks, ptr(ws),
         ptr(cnt))
    return out


_dw_scratch = {}
DW_MAX_K = 1 << 16
DW_TERMS = 4


def dw_scratch(device):
    """Per-device buffers of the tcgen05 decode linear: expanded activation codes [64, DW_MAX_K/2], their scale atoms
    (zero-initialised: unused virtual rows keep scale 0), fp32 split-K partials and per-tile tickets."""
    key = str(device)
    t = _dw_scratch.get(key)
    if t is None:
        t = (_ws("decode_linear/codes", (64, DW_MAX_K // 2), torch.uint8, device, zero=True),
             _ws("decode_linear/scale_atoms", DW_MAX_K // 64 * 512, torch.uint8, device, zero=True),
             _ws("decode_linear/partials", 1024 * 16 * 128, torch.float32, device),
             _ws("decode_linear/tickets", 1024 + 8, torch.int32, device, zero=True))      # [1024] = ticket of the fused add + norm
        _dw_scratch[key] = t
    return t


def dw_splits(N: int, K: int) -> int:
    """K splits of the decode linear: about two waves of CTAs, at least two 256-wide k-tiles each."""
    tiles, nkt = N // 128, (K + 255) // 256
    ks = (2 * 148) // tiles                    # all CTAs resident at once (two per SM)
    ks = max(1, min(ks, nkt // 2, 32))
    while ks > 1 and ks * tiles > 1024:
        ks -= 1
    return ks


def nvfp4_expand_rows(x, terms=DW_TERMS):
    """bf16 rows -> residual NVFP4 expansion in the shared scratch; returns (codes, scale atoms) views."""
    M, K = x.shape
    xp, xs, _, _ = dw_scratch(x.device)
    assert K <= DW_MAX_K and M * terms <= 64
    xpv = xp.view(-1)[: 64 * (K // 2)].view(64, K // 2)
    call("nvfp4_expand_rows", "plppiii", ptr(x), x.stride(0), ptr(xpv), ptr(xs), M, K, terms)
    return xpv, xs


DW_PDL = os.environ.get("VOLTA_PDL", "1") != "0"


# L2 prefetch chain of the decode linears: weights of the linear that runs next in a decode step are requested into L2 by
# the CTAs of the current one (which streams its own weights evict-first), so the next kernel starts on L2 hits instead
# of HBM latency. VOLTA_L2_PREFETCH_MB: most bytes requested per launch (0 = off).
L2_PREFETCH_BYTES = int(float(os.environ.get("VOLTA_L2_PREFETCH_MB", "0")) * (1 << 20))
_prefetch_next: dict = {}


def link_prefetch(lin, nxt) -> None:
    """After the decode linear over ``lin``'s weights the step runs ``nxt``: remember what to request."""
    if lin is None or nxt is None or getattr(lin, "packed", None) is None or getattr(nxt, "packed", None) is None:
        return
    if not lin.packed.is_cuda or getattr(nxt, "_sf_atoms", None) is None:
        return
    w, sf = nxt.packed, nxt._sf_atoms
    _prefetch_next[lin.packed.data_ptr()] = (w.data_ptr(), w.numel() * w.element_size(), sf.data_ptr(), sf.numel() * sf.element_size())


def decode_w4a4(packed, sf_atoms, gscale, x, out=None, residual=None, out_f32=False, terms=DW_TERMS, ks=None, pdl=None,
                act=0, act_limit=0.0, prenorm=None, push_args=0, addnorm=None, rope=None):
    """Decode / verify linear (M <= 16 rows) on the block-scaled FP4 tensor-core path; the kernel expands each bf16
    activation row into ``terms`` residual NVFP4 rows itself (bf16-grade accuracy): out [M, N]."""
    N, K = packed.shape[0], packed.shape[1] * 2
    # prenorm = (norm_w, resid, delta | None, resid_out | None, eps, wbias): the kernel's input is
    # RMSNorm(resid + delta) * (norm_w + wbias) and it writes resid + delta to resid_out; ``x`` is ignored (M <= 4)
    pn_w, pn_resid, pn_delta, pn_out, pn_eps, pn_bias = prenorm if prenorm is not None else (None, None, None, None, 0.0, 0.0)
    if prenorm is not None:
        x = pn_resid
    M = x.shape[0]
    if out is None:
        out = torch.empty(M, N // 2 if act else N, dtype=torch.float32 if out_f32 else torch.bfloat16, device=x.device)
    f32 = out.dtype == torch.float32
    _, _, ws, tickets = dw_scratch(x.device)
    if ks is None:
        ks = dw_splits(N, K)
    assert ks == 1 or ks * (N // 128) <= 1024      # split-K workspace and tickets hold 1024 tiles
    if pdl is None:
        pdl = DW_PDL
    # push_args: address of the communicator's argument block: the epilogue also sends the result rows to every peer's
    # all-reduce staging area (the all-reduce behind is then called with ``pushed=True``)
    # addnorm = (resid [M, N], norm_w [N], normed_out [M, N], eps, wbias): the tile that finishes last adds the product
    # to ``resid`` in place and writes RMSNorm(resid) * (norm_w + wbias) to ``normed_out`` (no separate norm launch)
    an_r, an_w, an_o, an_eps, an_bias = addnorm if addnorm is not None else (None, None, None, 0.0, 0.0)
    # rope = (pos, slot, page_table, kpool, vpool, nq, nkv, rot_dim, theta): a stacked q | k | v projection with head_dim
    # 128 rotates its q / k heads and writes k / v into the paged cache from its own epilogue
    rp = rope if rope is not None else (None, None, None, None, None, 0, 0, 0, 0.0)
    rp_table = rp[2]
    nxt = _prefetch_next.get(packed.data_ptr()) if L2_PREFETCH_BYTES > 0 else None
    if nxt is not None:
        wb = min(nxt[1], L2_PREFETCH_BYTES)
        sb = min(nxt[3], max(0, L2_PREFETCH_BYTES - wb))
        _lib_kernels().ve_decode_set_prefetch(ctypes.c_void_p(nxt[0]), ctypes.c_size_t(wb), ctypes.c_void_p(nxt[2]), ctypes.c_size_t(sb))
    call("decode_w4a4", "pppl" + "plppl" + "iiifiiiif" + "ppppff" + "ppppffp" + "pppippiiifi" + "ppp", ptr(packed), ptr(sf_atoms), ptr(x), x.stride(0),
         0 if f32 else ptr(out), out.stride(0), ptr(out) if f32 else 0, ptr(residual),
         residual.stride(0) if residual is not None else 0, M, N, K, float(gscale), terms, ks, 1 if pdl else 0,
         act, float(act_limit), ptr(pn_w), ptr(pn_resid), ptr(pn_delta), ptr(pn_out), float(pn_eps), float(pn_bias),
         int(push_args), ptr(an_r), ptr(an_w), ptr(an_o), float(an_eps), float(an_bias),
         tickets.data_ptr() + 4096 if addnorm is not None else 0,
         ptr(rp[0]), ptr(rp[1]), ptr(rp_table), rp_table.shape[1] if rp_table is not None else 0, ptr(rp[3]), ptr(rp[4]),
         rp[5], rp[6], rp[7], float(rp[8]), 1 if (rp[3] is not None and rp[3].dtype == torch.float8_e5m2) else 0,
         ptr(ws), ptr(tickets), ptr(status_word(x.device)))
    return out


def bf16_gemv_f32(W, x, out=None):
    N, K = W.shape
    M = x.shape[0]
    if out is None:
        out = torch.empty(M, N, dtype=torch.float32, device=x.device)
    call("bf16_gemv_f32", "pplpliii", ptr(W), ptr(x), x.stride(0), ptr(out), out.stride(0), M, N, K)
    return out


def gemm_bf16(W, x, out=None, residual=None, alpha=1.0, out_f32=False):
    """out[t, n] = alpha * sum_k W[n,k] x[t,k] on tcgen05 (bf16 x bf16, fp32 accumulate)."""
    N, K = W.shape
    T = x.shape[0]
    if out is None:
        out = torch.empty(T, N, dtype=torch.float32 if out_f32 else torch.bfloat16, device=x.device)
    f32 = out.dtype == torch.float32
    call("gemm_bf16", "plplplppliiifp", ptr(W), W.stride(0), ptr(x), x.stride(0), 0 if f32 else ptr(out),
         out.stride(0), ptr(out) if f32 else 0, ptr(residual), residual.stride(0) if residual is not None else 0,
         T, N, K, float(alpha), ptr(status_word(x.device)))
    return out


GEMM_WIDE = os.environ.get("VOLTA_GEMM_WIDE", "1") != "0"


def gemm_w4a16(packed, sf_blocked, gscale, x, out=None, residual=None):
    N, K2 = packed.shape
    K = K2 * 2
    T = x.shape[0]
    if out is None:
        out = torch.empty(T, N, dtype=torch.bfloat16, device=x.device)
    if T > 128 and N % 256 == 0 and K % 128 == 0 and GEMM_WIDE and out.dtype == torch.bfloat16:
        # prefill chunks: 256 x 256 tiles, two weight sub-tiles per activation tile (csrc/cuda/gemm_w4a16_wide.cu)
        call("gemm_w4a16_wide", "ppplplpliiifp", ptr(packed), ptr(sf_blocked), ptr(x), x.stride(0), ptr(out), out.stride(0),
             ptr(residual), residual.stride(0) if residual is not None else 0, T, N, K, float(gscale),
             ptr(status_word(x.device)))
        return out
    call("gemm_w4a16", "ppplplppliiifp", ptr(packed), ptr(sf_blocked), ptr(x), x.stride(0), ptr(out),
         out.stride(0), 0, ptr(residual), residual.stride(0) if residual is not None else 0, T, N, K,
         float(gscale), ptr(status_word(x.device)))
    return out


def gemm_w4a4(packed, sf_atoms, gscale, xp, xs_atoms, T, out=None, residual=None):
    N, K2 = packed.shape
    K = K2 * 2
    if out is None:
        out = torch.empty(T, N, dtype=torch.bfloat16, device=packed.device)
    call("gemm_w4a4", "pppppl" + "ppliiifp", ptr(packed), ptr(sf_atoms), ptr(xp), ptr(xs_atoms), ptr(out),
         out.stride(0), 0, ptr(residual), residual.stride(0) if residual is not None else 0, T, N, K,
         float(gscale), ptr(status_word(packed.device)))
    return out


def native_launches() -> int:
    return _lib.launch_count
