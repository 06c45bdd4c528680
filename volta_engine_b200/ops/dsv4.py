"""DeepSeek-V4-style attention pieces: sliding-window KV ring, compressed KV shared between layers, indexer, attention.

Every layer attends over a sliding window of its own raw KV (one 512-wide vector per token, shared by all heads as
key and value) and, on compressing layers, over at most 512 compressed entries that a source layer produced and an
indexer picked for the query. Rotary embedding acts on adjacent pairs of the last 64 dims; the attention output gets
the inverse rotation. Caches hold the model's quantisation grids (they are part of its numerics):

    window row        512 E4M3 codes + 16 power-of-two (E8M0) exponents, one per 32 values      (MXFP8)
    compressed entry  256 bytes of E2M1 pairs + 32 E4M3 scales, one per 16 values               (NVFP4)
    index key         128 values on the E2M1 x power-of-two-per-32 grid, kept as bf16 (exact)   (MXFP4 values)
    attention output  E4M3 x power-of-two-per-32 grid, kept as bf16 (exact)

All caches are indexed by position per slot, so a rewind needs no state copy. The device path dequantises a row's
window entries and selected compressed entries into latent scratch pages (bf16 holds every grid value exactly) and
runs the latent attention kernel of csrc/cuda/mla.cu over that short virtual sequence; the per-head sink is one more
key whose value is zero and whose score comes from an extra query element. The functions below are the fp32 PyTorch
statement (CPU path and test oracle) and the dispatch to csrc/cuda/dsv4.cu.

Reference: inc/engine/modules/dsv4.h:12-124 (cache layouts, grids, window_store / compress / index_key_store /
indexer / attend / route / engram_gate), src/models/deepseek_v41.cpp:2155-2259 (their order in a layer).
"""
from __future__ import annotations

import math

import torch

from .._lib import call, ptr

HD, ROPE, WINDOW, RING = 512, 64, 128, 1024
IDX_HEADS, IDX_DIM, TOPK, GROUP_HEADS = 32, 128, 512, 8
WIN_ROW, COMP_ROW = HD + HD // 32, HD // 2 + HD // 16
LAT_ROW = 576                      # row of the latent attention kernel: 512 values + 64 (element 512 carries the sink)
KEYS_MAX = WINDOW + TOPK + 1
PAGES_PER_ROW = (KEYS_MAX + 63) // 64
_E2M1 = (0.0, 0.5, 1.0, 1.5, 2.0, 3.0, 4.0, 6.0)


# ------------------------------------------------------------------------------------------------ rotary tables
def rope_table(max_pos: int, theta: float, original_len: int = 0, factor: float = 1.0, beta_fast: float = 32.0,
               beta_slow: float = 1.0, device="cpu") -> torch.Tensor:
    """[max_pos, 32, 2] fp32 (cos, sin); with ``original_len`` > 0 the frequencies get the YaRN ramp between the dims
    that turn ``beta_fast`` and ``beta_slow`` times over the original context (those beyond are divided by ``factor``)."""
    dim = ROPE
    freqs = 1.0 / (theta ** (torch.arange(0, dim, 2, dtype=torch.float32) / dim))
    if original_len > 0:
        def corrected(rot):
            return dim * math.log(original_len / (rot * 2 * math.pi)) / (2 * math.log(theta))
        low, high = max(math.floor(corrected(beta_fast)), 0), min(math.ceil(corrected(beta_slow)), dim - 1)
        ramp = ((torch.arange(dim // 2, dtype=torch.float32) - low) / max(high - low, 1e-3)).clamp(0, 1)
        freqs = freqs / factor * ramp + freqs * (1 - ramp)
    ang = torch.outer(torch.arange(max_pos, dtype=torch.float32), freqs)
    return torch.stack((ang.cos(), ang.sin()), -1).contiguous().to(device)


def rope_tail(x: torch.Tensor, cs: torch.Tensor, inverse: bool = False) -> torch.Tensor:
    """Rotates the last 64 dims of fp32 ``x`` [..., D] by ``cs`` [..., 32, 2] (adjacent pairs); returns a new tensor."""
    out = x.clone()
    t = x[..., -ROPE:].reshape(*x.shape[:-1], ROPE // 2, 2)
    c, s = cs[..., 0], (-cs[..., 1] if inverse else cs[..., 1])
    out[..., -ROPE:] = torch.stack((t[..., 0] * c - t[..., 1] * s, t[..., 1] * c + t[..., 0] * s), -1).reshape(*x.shape[:-1], ROPE)
    return out


# ------------------------------------------------------------------------------------------------ grids
def _bf(x):
    return x.to(torch.bfloat16).float()


def pow2_ceil(v: torch.Tensor) -> torch.Tensor:
    m, e = torch.frexp(v)
    return torch.ldexp(torch.ones_like(v), e - (m == 0.5).to(e.dtype))


def e2m1_round(x: torch.Tensor) -> torch.Tensor:
    """Nearest E2M1 value of |x| <= 6, ties to the even mantissa."""
    a = x.abs()
    r = torch.zeros_like(a)
    for bound, val, incl in ((0.25, 0.5, False), (0.75, 1.0, True), (1.25, 1.5, False), (1.75, 2.0, True), (2.5, 3.0, False),
                             (3.5, 4.0, True), (5.0, 6.0, False)):
        r = torch.where((a >= bound) if incl else (a > bound), torch.full_like(a, val), r)
    return torch.copysign(r, x)


def mxfp8_quant(x: torch.Tensor):
    """fp32 [..., D] -> (E4M3 codes uint8 [..., D], E8M0 exponents uint8 [..., D / 32]); scale = 2^ceil(log2(amax / 448))."""
    xb = x.float().reshape(*x.shape[:-1], -1, 32)
    s = pow2_ceil(xb.abs().amax(-1, keepdim=True).clamp_min(1e-4) / 448.0)
    q = (xb / s).clamp(-448.0, 448.0).to(torch.float8_e4m3fn)
    exps = (torch.frexp(s.squeeze(-1))[1] - 1 + 127).to(torch.uint8)
    return q.view(torch.uint8).reshape(x.shape), exps


def mxfp8_dequant(codes: torch.Tensor, exps: torch.Tensor) -> torch.Tensor:
    v = codes.view(torch.float8_e4m3fn).float().reshape(*codes.shape[:-1], -1, 32)
    return (v * torch.exp2((exps.int() - 127).float())[..., None]).reshape(codes.shape)


def mxfp8_round(x: torch.Tensor) -> torch.Tensor:
    return mxfp8_dequant(*mxfp8_quant(x))


def nvfp4_quant16(x: torch.Tensor):
    """fp32 [..., D] -> (packed uint8 [..., D / 2] even dim in the low nibble, E4M3 scale bytes [..., D / 16])."""
    from ..quant import nvfp4 as qn
    xb = x.float().reshape(*x.shape[:-1], -1, 16)
    s8 = (xb.abs().amax(-1).clamp_min(6 * 2.0 ** -9) / 6.0).to(torch.float8_e4m3fn)
    s = s8.float()[..., None]
    codes = qn.e2m1_encode(e2m1_round((xb / s).clamp(-6.0, 6.0))).reshape(x.shape)
    return qn.pack_codes(codes), s8.view(torch.uint8)


def nvfp4_dequant16(packed: torch.Tensor, scales: torch.Tensor) -> torch.Tensor:
    from ..quant import nvfp4 as qn
    v = qn.e2m1_decode(qn.unpack_codes(packed)).reshape(*packed.shape[:-1], -1, 16)
    return (v * scales.view(torch.float8_e4m3fn).float()[..., None]).reshape(*packed.shape[:-1], -1)


def mxfp4_round(x: torch.Tensor) -> torch.Tensor:
    """Value form of the E2M1 x power-of-two-per-32 grid."""
    xb = x.float().reshape(*x.shape[:-1], -1, 32)
    s = pow2_ceil(xb.abs().amax(-1, keepdim=True).clamp_min(6 * 2.0 ** -126) / 6.0)
    return (e2m1_round((xb / s).clamp(-6.0, 6.0)) * s).reshape(x.shape)


# ------------------------------------------------------------------------------------------------ state
class DSV4State:
    """Caches of one model instance. ``sources`` lists (layer, ratio) of the layers that compress KV."""

    def __init__(self, slots: int, layers: int, sources, max_seq: int, device):
        dev = device
        self.slots, self.max_seq = slots, max_seq
        self.win = torch.zeros(slots, layers, RING, WIN_ROW, dtype=torch.uint8, device=dev)
        self.ratios = [r for _, r in sources]
        self.caps = [(max_seq + r - 1) // r for r in self.ratios]
        self.cring_kv = [torch.zeros(slots, RING, HD, dtype=torch.float32, device=dev) if r > 1 else None for r in self.ratios]
        self.cring_sc = [torch.zeros(slots, RING, HD, dtype=torch.float32, device=dev) if r > 1 else None for r in self.ratios]
        self.comp = [torch.zeros(slots, c, COMP_ROW, dtype=torch.uint8, device=dev) for c in self.caps]
        self.idxk = [torch.zeros(slots, c, IDX_DIM, dtype=torch.bfloat16, device=dev) for c in self.caps]
        self.sel = None          # (sel [rows, TOPK] int32, nsel [rows] int32) of the latest index source
        self.cand = None         # bool / uint8 [rows, cap / block] of the candidate source
        self.scratch = None

    def nbytes(self) -> int:
        t = [self.win] + [x for x in self.cring_kv + self.cring_sc + self.comp + self.idxk if x is not None]
        return sum(x.numel() * x.element_size() for x in t)


# ------------------------------------------------------------------------------------------------ cache writes
def window_store(st: DSV4State, layer: int, kv_n: torch.Tensor, rope: torch.Tensor, slot: torch.Tensor, pos: torch.Tensor,
                 norm=None):
    """kv_n [rows, 512] bf16 (normed) -> rope at pos, bf16 rounding, MXFP8 -> win[slot, layer, pos % RING].
    ``norm`` = (weight, eps, weight bias): the rows are the raw projection and their RMSNorm is applied here first."""
    rows = kv_n.shape[0]
    if kv_n.is_cuda:
        w, eps, wb = norm if norm is not None else (None, 0.0, 0.0)
        call("dsv4_window_store", "plppppilipff", ptr(kv_n), kv_n.stride(0), ptr(st.win), ptr(rope), ptr(slot), ptr(pos), layer,
             st.win.stride(0), rows, ptr(w), float(eps), float(wb))
        return
    if norm is not None:
        from . import reference as ref
        kv_n = ref.rmsnorm(kv_n, norm[0], norm[1], norm[2])[0]
    ok = slot >= 0
    v = _bf(rope_tail(kv_n.float(), rope[pos.long()]))
    codes, exps = mxfp8_quant(v)
    row = torch.cat((codes, exps), -1)
    st.win[slot[ok].long(), layer, (pos[ok] % RING).long()] = row[ok]


def compress(st: DSV4State, src: int, ckv: torch.Tensor, csc, norm_w: torch.Tensor, rope: torch.Tensor, slot, pos, eps: float):
    """Compressor of source ``src``. ratio 1: latent = rmsnorm(ckv). ratio r > 1: rows go to the ring, and the row that
    completes a group (pos % r == r - 1) pools latent[d] = sum_t softmax_t(score[t][d]) ckv[t][d] over the group, then
    rmsnorm. A completing row writes the unrotated latent (bf16) to the returned [rows, 512] tensor (other rows: zero) and
    the compressed entry pos // r: the latent roped at the group's first position on the NVFP4 grid."""
    ratio = st.ratios[src]
    rows = ckv.shape[0]
    latent = torch.zeros(rows, HD, dtype=torch.bfloat16, device=ckv.device)
    if ckv.is_cuda:
        if ratio > 1:
            call("dsv4_cring_store", "plplpppplii", ptr(ckv), ckv.stride(0), ptr(csc), csc.stride(0), ptr(st.cring_kv[src]),
                 ptr(st.cring_sc[src]), ptr(slot), ptr(pos), st.cring_kv[src].stride(0), rows, 0)
        call("dsv4_compress", "plppppppppllifi", ptr(ckv), ckv.stride(0), ptr(st.cring_kv[src]) if ratio > 1 else 0,
             ptr(st.cring_sc[src]) if ratio > 1 else 0, ptr(norm_w), ptr(latent), ptr(st.comp[src]), ptr(rope), ptr(slot), ptr(pos),
             st.cring_kv[src].stride(0) if ratio > 1 else 0, st.comp[src].stride(0), ratio, float(eps), rows)
        return latent
    ok = slot >= 0
    if ratio > 1:
        st.cring_kv[src][slot[ok].long(), (pos[ok] % RING).long()] = ckv[ok].float()
        st.cring_sc[src][slot[ok].long(), (pos[ok] % RING).long()] = csc[ok].float()
    for r in range(rows):
        s, p = int(slot[r]), int(pos[r])
        if s < 0 or p % ratio != ratio - 1:
            continue
        if ratio == 1:
            pooled = ckv[r].float()
        else:
            at = [(p - ratio + 1 + j) % RING for j in range(ratio)]
            kvv, sc = st.cring_kv[src][s, at], st.cring_sc[src][s, at]
            pooled = _bf((kvv * torch.softmax(sc, dim=0)).sum(0))
        lat = _bf(pooled * torch.rsqrt(pooled.pow(2).mean() + eps) * norm_w.float())
        latent[r] = lat.to(torch.bfloat16)
        roped = _bf(rope_tail(lat, rope[p - ratio + 1]))
        pk, sc8 = nvfp4_quant16(roped)
        st.comp[src][s, p // ratio] = torch.cat((pk, sc8))
    return latent


def index_key_store(st: DSV4State, src: int, kraw: torch.Tensor, knorm_w: torch.Tensor, rope, slot, pos, eps: float):
    """Index keys of the completing rows: rmsnorm(kraw) * w, rope at the group's first position, MXFP4 grid -> idxk."""
    ratio = st.ratios[src]
    rows = kraw.shape[0]
    if kraw.is_cuda:
        call("dsv4_index_key_store", "plpppppplifi", ptr(kraw), kraw.stride(0), ptr(knorm_w), ptr(st.idxk[src]), ptr(rope), ptr(slot),
             ptr(pos), 0, st.idxk[src].stride(0), ratio, float(eps), rows)
        return
    for r in range(rows):
        s, p = int(slot[r]), int(pos[r])
        if s < 0 or p % ratio != ratio - 1:
            continue
        k = kraw[r].float()
        k = _bf(k * torch.rsqrt(k.pow(2).mean() + eps) * knorm_w.float())
        k = _bf(rope_tail(k, rope[p - ratio + 1]))
        st.idxk[src][s, p // ratio] = mxfp4_round(k).to(torch.bfloat16)


# ------------------------------------------------------------------------------------------------ indexer
def index_queries(q: torch.Tensor, rope, pos) -> torch.Tensor:
    """q [rows, 32 * 128] bf16 -> rope at pos on the last 64 dims of every head, MXFP4 grid (bf16 values)."""
    rows = q.shape[0]
    if q.is_cuda:
        out = torch.empty(rows, IDX_HEADS * IDX_DIM, dtype=torch.bfloat16, device=q.device)
        call("dsv4_index_q", "plpppi", ptr(q), q.stride(0), ptr(out), ptr(rope), ptr(pos), rows)
        return out
    v = q.float().reshape(rows, IDX_HEADS, IDX_DIM)
    v = _bf(rope_tail(v, rope[pos.long()][:, None]))
    return mxfp4_round(v).to(torch.bfloat16).reshape(rows, -1)


def index_scores_reference(st: DSV4State, src: int, qi, w, slot, pos) -> list:
    ratio = st.ratios[src]
    out = []
    for r in range(qi.shape[0]):
        n = (int(pos[r]) + 1) // ratio
        keys = st.idxk[src][int(slot[r]), :n].float()
        dots = torch.relu(torch.einsum("hd,td->ht", qi[r].float().reshape(IDX_HEADS, IDX_DIM), keys))
        out.append((w[r].float()[:, None] * dots).sum(0) / (IDX_DIM * IDX_HEADS) ** 0.5)
    return out


def candidate_blocks_reference(sc: torch.Tensor, blocks: int, block: int) -> torch.Tensor:
    """Level one of the two-level selection: bool [ceil(n / block)] of the ``blocks`` best blocks by their best entry;
    the block holding the newest entry is always kept."""
    n = sc.shape[0]
    nb = (n + block - 1) // block
    pad = torch.full((nb * block,), float("-inf"))
    pad[:n] = sc
    bs = pad.reshape(nb, block).amax(-1)
    bs[(n - 1) // block] = float("inf")
    keep = torch.zeros(nb, dtype=torch.bool)
    if nb <= blocks:
        keep[:] = True
        return keep
    order = torch.sort(bs, descending=True, stable=True).indices[:blocks]
    keep[order] = True
    return keep


def topk_reference(sc: torch.Tensor, k: int) -> list[int]:
    """The k best entries in position order; ties at the threshold go to the earlier positions."""
    n = sc.shape[0]
    if n <= k:
        return list(range(n))
    thr = torch.sort(sc, descending=True).values[k - 1]
    gt = [i for i in range(n) if float(sc[i]) > float(thr)]
    eq = [i for i in range(n) if float(sc[i]) == float(thr)][: k - len(gt)]
    return sorted(gt + eq)


def indexer(st: DSV4State, src: int, qi: torch.Tensor, w: torch.Tensor, slot, pos, cand_mode: int = 0, cand_blocks: int = 2048,
            cand_block: int = 8):
    """score[t] = (128 * 32)^-1/2 sum_h w[h] relu(q[h] . k[t]) over t < (pos + 1) // ratio; keeps the TOPK best (all when
    fewer). ``cand_mode`` 1: this layer first marks the best ``cand_blocks`` blocks of ``cand_block`` entries (stored in the
    state); 2: entries outside the stored blocks do not compete. -> (sel [rows, TOPK] int32 ascending, nsel [rows])."""
    rows = qi.shape[0]
    ratio = st.ratios[src]
    alloc = torch.empty if qi.is_cuda else torch.zeros          # the kernels write every entry that is read afterwards
    sel = alloc(rows, TOPK, dtype=torch.int32, device=qi.device)
    nsel = alloc(rows, dtype=torch.int32, device=qi.device)
    cap = st.caps[src]
    nblk = (cap + cand_block - 1) // cand_block
    if qi.is_cuda:
        scores = torch.empty(rows, cap, dtype=torch.float32, device=qi.device)
        call("dsa_score_div", "pppplppliiii", ptr(qi), ptr(w), ptr(st.idxk[src]), ptr(scores), scores.stride(0), ptr(slot), ptr(pos),
             st.idxk[src].stride(0), rows, cap, IDX_HEADS, ratio)
        if cand_mode == 1:
            st.cand = torch.empty(rows, nblk, dtype=torch.uint8, device=qi.device)
            call("dsv4_candidates", "plplppiiii", ptr(scores), scores.stride(0), ptr(st.cand), st.cand.stride(0), ptr(slot), ptr(pos),
                 ratio, cand_blocks, cand_block, rows)
        use_cand = cand_mode in (1, 2) and st.cand is not None and st.cand.shape[0] == rows
        call("dsv4_select", "plplippppii", ptr(scores), scores.stride(0), ptr(st.cand) if use_cand else 0,
             st.cand.stride(0) if use_cand else 0, cand_block, ptr(sel), ptr(nsel), ptr(slot), ptr(pos), ratio, rows)
        st.sel = (sel, nsel)
        return st.sel
    sc = index_scores_reference(st, src, qi, w.float(), slot, pos)
    if cand_mode == 1:
        st.cand = [candidate_blocks_reference(s, cand_blocks, cand_block) if s.numel() else None for s in sc]
    for r in range(rows):
        if int(slot[r]) < 0 or sc[r].numel() == 0:
            continue
        s = sc[r]
        if cand_mode in (1, 2) and st.cand is not None and st.cand[r] is not None:
            keep = st.cand[r].repeat_interleave(cand_block)[: s.numel()]
            s = torch.where(keep, s, torch.full_like(s, float("-inf")))
        pick = topk_reference(s, TOPK)
        pick = [i for i in pick if s[i] > float("-inf")]
        sel[r, :len(pick)] = torch.tensor(pick, dtype=torch.int32)
        nsel[r] = len(pick)
    st.sel = (sel, nsel)
    return st.sel


# ------------------------------------------------------------------------------------------------ attention
def _row_keys_reference(st: DSV4State, layer: int, src: int, s: int, p: int, sel, nsel, r: int, win_floor: int,
                        window: int = WINDOW):
    lo = max(0, p - window + 1, win_floor)
    at = [(t % RING) for t in range(lo, p + 1)]
    rows = st.win[s, layer, at]
    keys = mxfp8_dequant(rows[:, :HD].contiguous(), rows[:, HD:].contiguous()) if at else torch.zeros(0, HD)
    if src >= 0 and sel is not None and int(nsel[r]) > 0:
        ent = st.comp[src][s, sel[r, : int(nsel[r])].long()]
        keys = torch.cat((keys, nvfp4_dequant16(ent[:, : HD // 2].contiguous(), ent[:, HD // 2:].contiguous())))
    return keys


def attend(st: DSV4State, layer: int, src: int, q: torch.Tensor, sink: torch.Tensor, rope, slot, pos, nh: int, ws=None,
           win_floor: int = 0, nsplit: int = 1, key_end=None, window: int = WINDOW) -> torch.Tensor:
    """q [rows, nh * 512] bf16 unrotated. Softmax over the window and (``src`` >= 0) the state's selected compressed entries,
    logits scaled by 512^-1/2, exp(sink[h]) added to the denominator; the output is inverse-roped at pos, put on the MXFP8
    grid and returned group-major: [nh / 8, rows, 8 * 512] bf16. ``key_end`` [rows] (default: pos) is the newest ring position
    a row reads and ``window`` how many positions back from there: a drafter block, whose rows all see the whole block on top
    of the committed window, passes the block's last position and 128 + block size."""
    rows = q.shape[0]
    groups = nh // GROUP_HEADS
    scale = HD ** -0.5
    sel, nsel = st.sel if (src >= 0 and st.sel is not None) else (None, None)
    out = torch.zeros(groups, rows, GROUP_HEADS * HD, dtype=torch.bfloat16, device=q.device)
    if q.is_cuda:
        if st.scratch is None or st.scratch[0].shape[0] < rows * PAGES_PER_ROW:
            cap = max(16, rows)
            st.scratch = (torch.zeros(cap * PAGES_PER_ROW, 1, 64, LAT_ROW, dtype=torch.bfloat16, device=q.device),
                          torch.arange(cap * PAGES_PER_ROW, dtype=torch.int32, device=q.device).reshape(cap, PAGES_PER_ROW).contiguous(),
                          torch.zeros(cap, dtype=torch.int32, device=q.device),
                          torch.zeros(cap, dtype=torch.int32, device=q.device),
                          torch.zeros(cap, dtype=torch.int32, device=q.device))
        pages, table, a_slot, nkeys, a_pos = st.scratch
        comp = st.comp[src] if sel is not None else None
        q_abs = torch.empty(rows, nh, LAT_ROW, dtype=torch.bfloat16, device=q.device)
        call("dsv4_gather", "pilplppppppppiipi" + "plpppif", ptr(st.win), layer, st.win.stride(0), ptr(comp), comp.stride(0) if comp is not None else 0,
             ptr(sel), ptr(nsel), ptr(slot), ptr(pos), ptr(pages), ptr(nkeys), ptr(a_pos), ptr(a_slot), win_floor, rows,
             ptr(key_end), window, ptr(q), q.stride(0), ptr(q_abs), ptr(sink), ptr(rope), nh, float(scale))
        o_lat = torch.empty(rows, nh, HD, dtype=torch.bfloat16, device=q.device)
        if ws is None or ws[0].numel() < rows * nh * nsplit * HD:
            nsplit = 1
            ws = (torch.empty(rows * nh * HD, dtype=torch.float32, device=q.device),
                  torch.empty(rows * nh, dtype=torch.float32, device=q.device))
        from .kernels import status_word
        call("mla_decode", "pppppppipliiifp", ptr(q_abs), ptr(o_lat), ptr(ws[0]), ptr(ws[1]), ptr(a_pos), ptr(a_slot), ptr(table),
             table.shape[1], ptr(pages), pages.shape[0], rows, nh, nsplit, float(scale), ptr(status_word(q.device)))
        call("dsv4_attn_out", "pppppii", ptr(o_lat), ptr(out), ptr(rope), ptr(pos), ptr(slot), nh, rows)
        return out
    qv = _bf(rope_tail(q.float().reshape(rows, nh, HD), rope[pos.long()][:, None]))
    for r in range(rows):
        s, p = int(slot[r]), int(pos[r])
        if s < 0:
            continue
        keys = _row_keys_reference(st, layer, src, s, p if key_end is None else int(key_end[r]), sel, nsel, r, win_floor, window)
        if keys.shape[0] == 0:                                                  # only the sink: the output is zero
            continue
        sc = qv[r] @ keys.t() * scale                                           # [nh, keys]
        mx = torch.maximum(sc.amax(-1), sink.float())
        pr = torch.exp(sc - mx[:, None])
        o = _bf((pr @ keys) / (pr.sum(-1) + torch.exp(sink.float() - mx))[:, None])
        o = _bf(rope_tail(o, rope[p][None], inverse=True))
        o = mxfp8_round(o).to(torch.bfloat16)
        out[:, r] = o.reshape(groups, GROUP_HEADS * HD)
    return out


def grouped_out_proj(o: torch.Tensor, woa: torch.Tensor) -> torch.Tensor:
    """o [groups, rows, 8 * 512] bf16, woa [groups, O, 8 * 512] bf16 -> [rows, groups * O]: every group's heads through its own
    low-rank projection (block diagonal). Decode rows run one kernel; larger chunks one batched product."""
    groups, rows, _ = o.shape
    O = woa.shape[1]
    if o.is_cuda and rows <= 16:
        out = torch.empty(rows, groups * O, dtype=torch.bfloat16, device=o.device)
        call("dsv4_woa", "pppiii", ptr(o), ptr(woa), ptr(out), groups, O, rows)
        return out
    if o.is_cuda:
        return torch.bmm(o, woa.transpose(1, 2)).permute(1, 0, 2).reshape(rows, groups * O).contiguous()
    return torch.einsum("grd,god->rgo", o.float(), woa.float()).to(torch.bfloat16).reshape(rows, groups * O)


# ------------------------------------------------------------------------------------------------ routing
def route_sqrt_softplus(logits: torch.Tensor, bias, top_k: int, scale: float):
    """s = sqrt(softplus(logit)); experts = top_k of s + bias; weights = s / sum(s of the chosen) * scale (fp32 statement)."""
    s = torch.nn.functional.softplus(logits.float()).sqrt()
    sel = s + (bias.float() if bias is not None else 0.0)
    order = torch.sort(sel, dim=-1, descending=True, stable=True).indices[:, :top_k]
    w = s.gather(1, order)
    return order.int(), w / (w.sum(-1, keepdim=True) + 1e-20) * scale


# ------------------------------------------------------------------------------------------------ engram
def engram_ids(ids, slot, pos, hist: torch.Tensor, tables: int, table_rows: int, ngram: int) -> torch.Tensor:
    """Records the rows' tokens in ``hist`` int32 [slots + 1, max_seq] (the last row takes padding rows) and returns the hashed
    table row of every (row, engram layer) int32 [rows, tables]: h = fold over the last ``ngram`` tokens of the sequence
    (token 2 before its start) of (h * 1000003 + t * (2 j + 1) + 12345) mod (2^31 - 1); row_i = (h * (2 i + 3) + i) mod rows."""
    n = ids.shape[0]
    spare = hist.shape[0] - 1
    out = torch.empty(n, tables, dtype=torch.int32, device=ids.device)
    if ids.is_cuda:
        call("dsv4_engram_ids", "pppplipiiii", ptr(ids), ptr(slot), ptr(pos), ptr(hist), hist.stride(0), spare, ptr(out), tables,
             table_rows, ngram, n)
        return out
    sl = torch.where(slot < 0, torch.full_like(slot, spare), slot).long()
    p = pos.long()
    hist[sl, p] = ids.int()
    h = torch.zeros(n, dtype=torch.long)
    for j in range(ngram):
        t = hist[sl, (p - j).clamp_min(0)].long()
        t = torch.where(p - j >= 0, t, torch.full_like(t, 2))
        h = (h * 1000003 + t * (2 * j + 1) + 12345) % 2147483647
    for i in range(tables):
        out[:, i] = ((h * (2 * i + 3) + i) % table_rows).int()
    return out


def engram_gate(streams: torch.Tensor, kv: torch.Tensor, w: torch.Tensor, skip=None, eps: float = 1e-20) -> torch.Tensor:
    """streams fp32 [rows, 4, H] (in place), kv [rows, 5 * H] = [key 0..3 | value] of the looked-up rows, w [4, H] fp32:
    dot = sum_d s[h][d] w[h][d] key[h][d] * rstd(s[h]) * rstd(key[h]) / sqrt(H); gate = sigmoid(sign(dot) sqrt(max(|dot|, 1e-6)));
    s[h] += gate * value. Rows with skip != 0 stay untouched."""
    rows, hc, H = streams.shape
    if streams.is_cuda:
        call("dsv4_engram_gate", "ppppiifi", ptr(streams), ptr(kv), ptr(w), ptr(skip), H, hc, float(eps), rows)
        return streams
    key = kv.float()[:, : hc * H].reshape(rows, hc, H)
    val = kv.float()[:, hc * H:]
    rs = torch.rsqrt(streams.pow(2).mean(-1) + eps)
    rk = torch.rsqrt(key.pow(2).mean(-1) + eps)
    dot = (streams * w.float()[None] * key).sum(-1) * rs * rk / math.sqrt(H)
    gate = torch.sigmoid(torch.sign(dot) * torch.sqrt(dot.abs().clamp_min(1e-6)))
    if skip is not None:
        gate = gate * (skip == 0).float()[:, None]
    streams += gate[:, :, None] * val[:, None, :]
    return streams
