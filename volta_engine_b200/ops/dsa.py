"""Sparse-attention indexer with pooled keys: per-layer state, the CUDA path (csrc/cuda/dsa.cu) and the fp32 PyTorch
statement of the same arithmetic (CPU path and test oracle).

Reference: inc/engine/modules/dsa.h:11-54 (projection layout [k | w | gate], plane ring, pools of 4, top 2048 tokens),
src/backend/cpu/dsa_ref.cpp (score and the order of the selected list).
"""
from __future__ import annotations

from dataclasses import dataclass

import torch

from .._lib import call, ptr

HEADS, DIM, POOL, TOPK = 32, 128, 4, 2048
QSA_HEADS = 4
SEL_POOLS = TOPK // POOL
KPAD = 2112
PROJ = DIM + HEADS + DIM
PLANE_CAP = 1024
PAGES_PER_ROW = KPAD // 64


@dataclass
class DSAWeights:
    proj: object               # linear hidden -> 288 ([k | w | gate])
    q_proj: object             # linear q latent -> 32 * 128 indexer queries
    ln_w: torch.Tensor         # [128] bf16
    ln_b: torch.Tensor
    ape: torch.Tensor          # [4, 128] bf16: position-in-pool bias of the pooling softmax


class DSAState:
    """Indexer memory of one layer: the plane ring [slots, 1024, 256] and the pooled keys [slots, max_seq / 4, 128]."""

    def __init__(self, slots: int, max_seq: int, device):
        self.max_pools = (max_seq + POOL - 1) // POOL
        self.plane = torch.zeros(slots, PLANE_CAP, 2 * DIM, dtype=torch.bfloat16, device=device)
        self.pools = torch.zeros(slots, self.max_pools, DIM, dtype=torch.bfloat16, device=device)


def update(state: DSAState, W: DSAWeights, x: torch.Tensor, slot: torch.Tensor, pos: torch.Tensor) -> torch.Tensor:
    """Project the rows, append [k_norm | gate] to the plane ring and build the pools that these rows complete.
    Returns the per-row head weights w [rows, 32] fp32."""
    rows = x.shape[0]
    proj = W.proj.forward(x).contiguous()
    w_out = torch.empty(rows, HEADS, dtype=torch.float32, device=x.device)
    if not x.is_cuda:
        pf = proj.float()
        k = torch.nn.functional.layer_norm(pf[:, :DIM], (DIM,), W.ln_w.float(), W.ln_b.float(), 1e-6)
        w_out.copy_(pf[:, DIM:DIM + HEADS])
        for r in range(rows):
            s, p = int(slot[r]), int(pos[r])
            if s < 0:
                continue
            state.plane[s, p % PLANE_CAP, :DIM] = k[r].to(torch.bfloat16)
            state.plane[s, p % PLANE_CAP, DIM:] = proj[r, DIM + HEADS:]
            if p % POOL == POOL - 1:
                ent = state.plane[s, [(p - 3 + j) % PLANE_CAP for j in range(POOL)]].float()
                wgt = torch.softmax(ent[:, DIM:] + W.ape.float(), dim=0)
                state.pools[s, p // POOL] = (wgt * ent[:, :DIM]).sum(0).to(torch.bfloat16)
        return w_out
    for r0 in range(0, rows, PLANE_CAP - POOL):                  # a pool reads the ring before later rows wrap around it
        r1 = min(rows, r0 + PLANE_CAP - POOL)
        call("dsa_prep", "pppppppli", ptr(proj[r0:r1]), ptr(W.ln_w), ptr(W.ln_b), ptr(state.plane), ptr(w_out[r0:r1]),
             ptr(slot[r0:r1]), ptr(pos[r0:r1]), state.plane.stride(0), r1 - r0)
        call("dsa_pool_update", "ppppplli", ptr(state.plane), ptr(state.pools), ptr(W.ape), ptr(slot[r0:r1]),
             ptr(pos[r0:r1]), state.plane.stride(0), state.pools.stride(0), r1 - r0)
    return w_out


def score_reference(q_idx, w, state: DSAState, slot, pos) -> list:
    out = []
    for r in range(q_idx.shape[0]):
        bound = (int(pos[r]) + 1) // POOL
        keys = state.pools[int(slot[r]), :bound].float()
        dots = torch.relu(torch.einsum("hd,pd->hp", q_idx[r].float().reshape(HEADS, DIM), keys))
        out.append((w[r].float()[:, None] * dots).sum(0) / (DIM * HEADS) ** 0.5)
    return out


def select_reference(scores: torch.Tensor, vis: int) -> list[int]:
    """Token list of one row: pools strictly above the threshold in pool order, then the threshold ties in pool order,
    each expanded to its 4 tokens, then the raw tail; every position when at most 512 pools are complete."""
    bound = vis // POOL
    if bound <= SEL_POOLS:
        return list(range(vis))
    sc = scores[:bound]
    thr = torch.sort(sc, descending=True).values[SEL_POOLS - 1]
    gt = [p for p in range(bound) if float(sc[p]) > float(thr)]
    eq = [p for p in range(bound) if float(sc[p]) == float(thr)][: SEL_POOLS - len(gt)]
    toks = [p * POOL + j for p in gt + eq for j in range(POOL)]
    return toks + list(range(vis - vis % POOL, vis))


def select(state: DSAState, q_idx: torch.Tensor, w: torch.Tensor, slot: torch.Tensor, pos: torch.Tensor):
    """(idx int32 [rows, KPAD], nkeys int32 [rows]): the positions every row attends to."""
    rows = q_idx.shape[0]
    idx = torch.zeros(rows, KPAD, dtype=torch.int32, device=q_idx.device)
    nkeys = torch.zeros(rows, dtype=torch.int32, device=q_idx.device)
    if not q_idx.is_cuda:
        sc = score_reference(q_idx, w, state, slot, pos)
        for r in range(rows):
            if int(slot[r]) < 0:
                continue
            toks = select_reference(sc[r], int(pos[r]) + 1)
            idx[r, :len(toks)] = torch.tensor(toks, dtype=torch.int32)
            nkeys[r] = len(toks)
        return idx, nkeys
    return select_from_scores(score(state, q_idx, w, slot, pos), slot, pos, idx, nkeys)


def score(state: DSAState, q_idx, w, slot, pos) -> torch.Tensor:
    """fp32 [rows, max_pools]; entries at and beyond a row's (pos + 1) // 4 are not written."""
    rows = q_idx.shape[0]
    scores = torch.empty(rows, state.max_pools, dtype=torch.float32, device=q_idx.device)
    call("dsa_score", "pppplppliii", ptr(q_idx), ptr(w), ptr(state.pools), ptr(scores), scores.stride(0), ptr(slot), ptr(pos),
         state.pools.stride(0), rows, state.max_pools, HEADS if w is not None else QSA_HEADS)
    return scores


def select_from_scores(scores, slot, pos, idx=None, nkeys=None):
    rows = scores.shape[0]
    if idx is None:
        idx = torch.zeros(rows, KPAD, dtype=torch.int32, device=scores.device)
        nkeys = torch.zeros(rows, dtype=torch.int32, device=scores.device)
    call("dsa_select", "plppppi", ptr(scores), scores.stride(0), ptr(idx), ptr(nkeys), ptr(slot), ptr(pos), rows)
    return idx, nkeys


def gather_rows(pool: torch.Tensor, page_table: torch.Tensor, slot, idx, nkeys, scratch: torch.Tensor):
    """Copy the listed tokens' cache rows into ``scratch`` [rows * 33, 1, 64, row] (entry i of row r -> page r * 33 + i // 64)."""
    rows = idx.shape[0]
    row_elems, nkv = pool.shape[-1], pool.shape[1]
    if not pool.is_cuda:
        for r in range(rows):
            s = int(slot[r])
            for i in range(int(nkeys[r])):
                t = int(idx[r, i])
                scratch[r * PAGES_PER_ROW + i // 64, :, i % 64] = pool[int(page_table[s, t // 64]), :, t % 64]
        return scratch
    call("dsa_gather", "ppippppiiii", ptr(pool), ptr(page_table), page_table.shape[1], ptr(slot), ptr(idx), ptr(nkeys), ptr(scratch),
         PAGES_PER_ROW, row_elems, nkv, rows)
    return scratch


# ---------------------------------------------------------------------------------------------- block-sparse indexer
@dataclass
class QSAWeights:
    proj: object               # linear hidden -> 5 * 128 ([q (4 heads) | k])
    q_norm: torch.Tensor       # [128] bf16, applied as 1 + w
    k_norm: torch.Tensor
    rot: int = 64
    theta: float = 1.0e7
    eps: float = 1e-6


class QSAState:
    """Raw-key ring [slots, 1024, 128] and pooled keys [slots, max_seq / 4, 128] of one layer."""

    def __init__(self, slots: int, max_seq: int, device):
        self.max_pools = (max_seq + POOL - 1) // POOL
        self.ring = torch.zeros(slots, PLANE_CAP, DIM, dtype=torch.bfloat16, device=device)
        self.pools = torch.zeros(slots, self.max_pools, DIM, dtype=torch.bfloat16, device=device)


def _rope_rows(v: torch.Tensor, pos: torch.Tensor, rot: int, theta: float) -> torch.Tensor:
    from .reference import rope_rotate
    return rope_rotate(v[:, None, :], pos, rot, theta)[:, 0]


def qsa_update(state: QSAState, W: QSAWeights, x, slot, pos) -> torch.Tensor:
    """Project the rows, keep the raw keys in the ring, build the pools these rows complete.
    Returns the indexer queries [rows, 4 * 128] bf16 (normalised, rotated at the row's position)."""
    rows = x.shape[0]
    qk = W.proj.forward(x).contiguous()
    if not x.is_cuda:
        q = qk[:, :QSA_HEADS * DIM].float().reshape(rows, QSA_HEADS, DIM)
        q = q * torch.rsqrt(q.pow(2).mean(-1, keepdim=True) + W.eps) * (1.0 + W.q_norm.float())
        from .reference import rope_rotate
        q = rope_rotate(q, pos, W.rot, W.theta).to(torch.bfloat16)
        for r in range(rows):
            s, p = int(slot[r]), int(pos[r])
            if s < 0:
                continue
            state.ring[s, p % PLANE_CAP] = qk[r, QSA_HEADS * DIM:]
            if p % POOL == POOL - 1:
                m = state.ring[s, [(p - 3 + j) % PLANE_CAP for j in range(POOL)]].float().mean(0)
                m = m * torch.rsqrt(m.pow(2).mean() + W.eps) * (1.0 + W.k_norm.float())
                state.pools[s, p // POOL] = _rope_rows(m[None], torch.tensor([p - 3]), W.rot, W.theta)[0].to(torch.bfloat16)
        return q.reshape(rows, QSA_HEADS * DIM)
    q_out = torch.empty(rows, QSA_HEADS * DIM, dtype=torch.bfloat16, device=x.device)
    for r0 in range(0, rows, PLANE_CAP - POOL):
        r1 = min(rows, r0 + PLANE_CAP - POOL)
        call("qsa_prep", "ppppppliffi", ptr(qk[r0:r1]), ptr(W.q_norm), ptr(q_out[r0:r1]), ptr(state.ring), ptr(slot[r0:r1]),
             ptr(pos[r0:r1]), state.ring.stride(0), W.rot, float(W.theta), float(W.eps), r1 - r0)
        call("qsa_pool_update", "ppppplliffi", ptr(state.ring), ptr(state.pools), ptr(W.k_norm), ptr(slot[r0:r1]), ptr(pos[r0:r1]),
             state.ring.stride(0), state.pools.stride(0), W.rot, float(W.theta), float(W.eps), r1 - r0)
    return q_out


def qsa_score_reference(q, state: QSAState, slot, pos) -> list:
    out = []
    for r in range(q.shape[0]):
        bound = (int(pos[r]) + 1) // POOL
        keys = state.pools[int(slot[r]), :bound].float()
        dots = torch.relu(torch.einsum("hd,pd->hp", q[r].float().reshape(QSA_HEADS, DIM), keys))
        out.append(dots.sum(0) / DIM ** 0.5)
    return out


def qsa_select(state: QSAState, q, slot, pos):
    """(idx, nkeys) like ``select``: same pool size, budget, list width and order."""
    rows = q.shape[0]
    if not q.is_cuda:
        idx = torch.zeros(rows, KPAD, dtype=torch.int32)
        nkeys = torch.zeros(rows, dtype=torch.int32)
        sc = qsa_score_reference(q, state, slot, pos)
        for r in range(rows):
            if int(slot[r]) < 0:
                continue
            toks = select_reference(sc[r], int(pos[r]) + 1)
            idx[r, :len(toks)] = torch.tensor(toks, dtype=torch.int32)
            nkeys[r] = len(toks)
        return idx, nkeys
    return select_from_scores(score(state, q, None, slot, pos), slot, pos)
