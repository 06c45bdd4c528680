"""Sequence-sharded tensor parallelism for training (the Megatron "sequence parallel" form) and context-parallel
attention, both over ``torch.distributed`` (NCCL over NVLink on GPUs, gloo in the CPU tests).

Training. Every rank owns ``rows / ranks`` rows of the fp32 residual stream. A sub-layer
    all-gathers the rows  ->  column-parallel linear(s)  ->  row-parallel linear  ->  reduce-scatters the partial sums
so the activations between sub-layers are never replicated. The two collectives are each other's gradient: the backward
of the all-gather is a reduce-scatter of the row gradients and the backward of the reduce-scatter is an all-gather,
which is what ``GatherRows`` / ``ReduceScatterRows`` implement as autograd functions. Parameter gradients of the sharded
weights are local; gradients of replicated parameters (norm weights) are summed over the ranks by ``sum_replicated_grads``.
Reference: inc/engine/train/qwen4_exp.h:15-20, src/train/qwen4_exp.cpp:229-259 (gather / reduce_rows / sum_ranks).

Context-parallel attention. Every rank owns a contiguous slice of the rows (queries, keys and values) with full
weights. Keys and values of the other ranks arrive slice by slice (all-gather issued ahead on a side stream where there
is one) while attention over the slices that are already there runs; the softmax is carried across key ranges as
(running max, running sum, unnormalised output) and normalised after the last range. Causal masking skips the slices
that lie wholly in the future of the rank's rows. Reference: inc/engine/video/h3_dit_group.h:7-9,
src/video/h3_dit_group.cpp:141-180, inc/engine/video/h3_attn.h:10-17 (``h3_attention_partial``).
"""
from __future__ import annotations

import math

import torch
import torch.distributed as dist


def _world(group) -> int:
    return dist.get_world_size(group) if dist.is_initialized() else 1


class GatherRows(torch.autograd.Function):
    """[rows / ranks, ...] per rank -> [rows, ...] in rank order; backward: reduce-scatter of the row gradients."""

    @staticmethod
    def forward(ctx, x, group):
        ctx.group = group
        n = _world(group)
        if n == 1:
            return x
        out = torch.empty((n * x.shape[0],) + tuple(x.shape[1:]), dtype=x.dtype, device=x.device)
        dist.all_gather_into_tensor(out, x.contiguous(), group=group)
        return out

    @staticmethod
    def backward(ctx, g):
        n = _world(ctx.group)
        if n == 1:
            return g, None
        out = torch.empty((g.shape[0] // n,) + tuple(g.shape[1:]), dtype=g.dtype, device=g.device)
        dist.reduce_scatter_tensor(out, g.contiguous(), group=ctx.group)
        return out, None


class ReduceScatterRows(torch.autograd.Function):
    """[rows, ...] partial sums per rank -> this rank's [rows / ranks, ...] of their sum; backward: all-gather."""

    @staticmethod
    def forward(ctx, x, group):
        ctx.group = group
        n = _world(group)
        if n == 1:
            return x
        out = torch.empty((x.shape[0] // n,) + tuple(x.shape[1:]), dtype=x.dtype, device=x.device)
        dist.reduce_scatter_tensor(out, x.contiguous(), group=group)
        return out

    @staticmethod
    def backward(ctx, g):
        n = _world(ctx.group)
        if n == 1:
            return g, None
        out = torch.empty((n * g.shape[0],) + tuple(g.shape[1:]), dtype=g.dtype, device=g.device)
        dist.all_gather_into_tensor(out, g.contiguous(), group=ctx.group)
        return out, None


def gather_rows(x, group=None):
    return GatherRows.apply(x, group)


def reduce_scatter_rows(x, group=None):
    return ReduceScatterRows.apply(x, group)


def shard_rows(x: torch.Tensor, group=None) -> torch.Tensor:
    """This rank's contiguous row block of a replicated tensor (rows must divide by the rank count)."""
    n = _world(group)
    if n == 1:
        return x
    r = dist.get_rank(group)
    per = x.shape[0] // n
    assert per * n == x.shape[0], "rows must be a multiple of the rank count"
    return x[r * per:(r + 1) * per]


def sum_replicated_grads(params, group=None) -> None:
    """Gradients of parameters every rank holds in full (norm weights, biases after a row-parallel linear): each rank
    saw only its rows, so the true gradient is the sum over the ranks."""
    if _world(group) == 1:
        return
    for p in params:
        if p.grad is not None:
            dist.all_reduce(p.grad, group=group)


class SequenceParallelMLP(torch.nn.Module):
    """Gated MLP sub-layer with sequence-sharded input and output: rows [rows / ranks, H] in, the same rows out.
    ``w_gate`` / ``w_up`` hold this rank's slice of the hidden units (column parallel), ``w_down`` the matching input
    slice (row parallel); ``from_full`` cuts the slices out of full matrices."""

    def __init__(self, w_gate, w_up, w_down, norm_w, eps: float = 1e-6, group=None):
        super().__init__()
        self.w_gate, self.w_up, self.w_down = (torch.nn.Parameter(t.clone()) for t in (w_gate, w_up, w_down))
        self.norm_w = torch.nn.Parameter(norm_w.clone())
        self.eps, self.group = eps, group

    @classmethod
    def from_full(cls, w_gate, w_up, w_down, norm_w, eps: float = 1e-6, group=None):
        n = _world(group)
        r = dist.get_rank(group) if n > 1 else 0
        f = w_gate.shape[0] // n
        return cls(w_gate[r * f:(r + 1) * f], w_up[r * f:(r + 1) * f], w_down[:, r * f:(r + 1) * f], norm_w, eps, group)

    def forward(self, x):
        h = x * torch.rsqrt((x * x).mean(-1, keepdim=True) + self.eps) * self.norm_w       # local rows: no communication
        full = gather_rows(h, self.group)                                                # [rows, H]
        a = torch.nn.functional.silu(full @ self.w_gate.t()) * (full @ self.w_up.t())     # [rows, F / ranks]
        part = a @ self.w_down.t()                                                        # partial sums over the slices
        return x + reduce_scatter_rows(part, self.group)


# ------------------------------------------------------------------------------------------------ context parallel
def attention_partial(q, k, v, state, scale: float, q_pos=None, k_pos=None):
    """One key range of a softmax attention carried across calls. q [rows, heads, d], k / v [keys, kv_heads, d];
    ``state`` = (m [rows, heads], l [rows, heads], o [rows, heads, d]) or None for the first range; positions (int
    tensors) make it causal: a key is visible when k_pos <= q_pos. Returns the new state; ``attention_finish``
    normalises. fp32 arithmetic (the tensor-core form of the same recurrence is ops.kernels.attention's split merge)."""
    rows, heads, d = q.shape
    rep = heads // k.shape[1]
    kf = k.float().repeat_interleave(rep, 1) if rep > 1 else k.float()
    vf = v.float().repeat_interleave(rep, 1) if rep > 1 else v.float()
    s = torch.einsum("rhd,khd->rhk", q.float(), kf) * scale
    if q_pos is not None:
        s = s.masked_fill((k_pos[None, :] > q_pos[:, None])[:, None, :], float("-inf"))
    m_new = s.max(-1).values
    if state is not None:
        m_old, l_old, o_old = state
        m_new = torch.maximum(m_new, m_old)
    safe = torch.where(torch.isinf(m_new), torch.zeros_like(m_new), m_new)       # rows that have seen no key yet
    p = torch.exp(s - safe[..., None])
    l_new = p.sum(-1)
    o_new = torch.einsum("rhk,khd->rhd", p, vf)
    if state is not None:
        a = torch.exp(torch.where(torch.isinf(m_old), torch.full_like(m_old, float("-inf")), m_old) - safe)
        l_new = l_new + a * l_old
        o_new = o_new + a[..., None] * o_old
    return m_new, l_new, o_new


def attention_finish(state, dtype=torch.float32):
    m, l, o = state
    return (o / l.clamp(min=1e-30)[..., None]).to(dtype)


def context_parallel_attention(q, k, v, scale: float | None = None, causal: bool = False, group=None):
    """q, k, v: this rank's contiguous row slice ([rows / ranks, heads, d]); returns the attention output for the same
    rows over the keys of every rank. The slices of the other ranks are fetched one at a time, the next fetch in flight
    while the current one is used; a causal rank never fetches a slice that lies in its future."""
    n = _world(group)
    rows = q.shape[0]
    scale = scale if scale is not None else 1.0 / math.sqrt(q.shape[-1])
    r = dist.get_rank(group) if n > 1 else 0
    q_pos = torch.arange(r * rows, (r + 1) * rows, device=q.device) if causal else None

    def k_positions(src):
        return torch.arange(src * rows, (src + 1) * rows, device=q.device) if causal else None

    if n == 1:
        return attention_finish(attention_partial(q, k, v, None, scale, q_pos, k_positions(r)), q.dtype)
    # one asynchronous all-gather carries every rank's keys and values; the rank's own key range is worked on while it
    # is in flight (collectives run beside compute on NCCL)
    kv = torch.stack([k, v]).contiguous()
    flat = torch.empty((n * 2,) + tuple(kv.shape[1:]), dtype=kv.dtype, device=kv.device)
    work = dist.all_gather_into_tensor(flat, kv, group=group, async_op=True)
    state = attention_partial(q, k, v, None, scale, q_pos, k_positions(r))
    work.wait()
    every = flat.view((n, 2) + tuple(kv.shape[1:]))
    order = [(r - i) % n for i in range(1, n)]              # nearest earlier slice first
    for src in order:
        if causal and src > r:
            continue
        state = attention_partial(q, every[src, 0], every[src, 1], state, scale, q_pos, k_positions(src))
    return attention_finish(state, q.dtype)
