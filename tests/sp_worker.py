"""Child process of tests/test_sequence_parallel.py: one CPU rank of a gloo world."""
import datetime
import os
import sys

import torch
import torch.distributed as dist

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))

from volta_engine_b200.parallel import sequence_parallel as SP  # noqa: E402


def main():
    dist.init_process_group("gloo", timeout=datetime.timedelta(seconds=60))
    rank, world = dist.get_rank(), dist.get_world_size()
    g = torch.Generator().manual_seed(0)                      # the same draws on every rank
    rows, H, F = 8 * world, 32, 64
    x_full = torch.randn(rows, H, generator=g, dtype=torch.float64)
    wg, wu, wd = (torch.randn(F, H, generator=g, dtype=torch.float64) * 0.2, torch.randn(F, H, generator=g, dtype=torch.float64) * 0.2,
                  torch.randn(H, F, generator=g, dtype=torch.float64) * 0.2)
    nw = torch.rand(H, generator=g, dtype=torch.float64) + 0.5
    target = torch.randn(rows, H, generator=g, dtype=torch.float64)

    # --- the sub-layer on one rank (no process group involved): the statement
    one = SP.SequenceParallelMLP(wg, wu, wd, nw, group=None)
    one.group = "single"

    def single(x):
        h = x * torch.rsqrt((x * x).mean(-1, keepdim=True) + 1e-6) * one.norm_w
        a = torch.nn.functional.silu(h @ one.w_gate.t()) * (h @ one.w_up.t())
        return x + a @ one.w_down.t()
    xs = x_full.clone().requires_grad_(True)
    loss = ((single(xs) - target) ** 2).sum()
    loss.backward()

    # --- the same sub-layer sequence-parallel: rows sharded, hidden units sharded
    mlp = SP.SequenceParallelMLP.from_full(wg, wu, wd, nw)
    xr = SP.shard_rows(x_full).clone().requires_grad_(True)
    y = mlp(xr)
    part = ((y - SP.shard_rows(target)) ** 2).sum()
    part.backward()
    SP.sum_replicated_grads([mlp.norm_w])
    total = part.detach().clone()
    dist.all_reduce(total)
    assert torch.allclose(total, loss.detach(), rtol=1e-10), (float(total), float(loss))
    assert torch.allclose(xr.grad, SP.shard_rows(xs.grad), rtol=1e-9, atol=1e-11), "input gradient"
    f = F // world
    assert torch.allclose(mlp.w_gate.grad, one.w_gate.grad[rank * f:(rank + 1) * f], rtol=1e-9, atol=1e-11)
    assert torch.allclose(mlp.w_up.grad, one.w_up.grad[rank * f:(rank + 1) * f], rtol=1e-9, atol=1e-11)
    assert torch.allclose(mlp.w_down.grad, one.w_down.grad[:, rank * f:(rank + 1) * f], rtol=1e-9, atol=1e-11)
    assert torch.allclose(mlp.norm_w.grad, one.norm_w.grad, rtol=1e-9, atol=1e-11), "replicated parameter gradient"

    # --- the two collectives are each other's gradient
    a = torch.randn(4, 3, generator=torch.Generator().manual_seed(10 + rank), dtype=torch.float64, requires_grad=True)
    w = torch.randn(4 * world, 3, generator=g, dtype=torch.float64)
    (SP.gather_rows(a) * w).sum().backward()
    want = torch.zeros_like(a)
    want += w[rank * 4:(rank + 1) * 4] * world                # every rank's loss sees this rank's rows with the same w
    assert torch.allclose(a.grad, want)

    # --- context-parallel attention, full and causal, GQA, against the attention over all rows
    for causal in (False, True):
        heads, kvh, d, per = 4, 2, 16, 6
        q = torch.randn(per * world, heads, d, generator=g)
        k = torch.randn(per * world, kvh, d, generator=g)
        v = torch.randn(per * world, kvh, d, generator=g)
        pos = torch.arange(per * world)
        ref = SP.attention_finish(SP.attention_partial(q, k, v, None, d ** -0.5, pos if causal else None, pos if causal else None))
        sl = slice(rank * per, (rank + 1) * per)
        got = SP.context_parallel_attention(q[sl], k[sl], v[sl], causal=causal)
        assert torch.allclose(got, ref[sl], rtol=1e-4, atol=1e-5), ("context parallel", causal, float((got - ref[sl]).abs().max()))
        # the carried softmax: two key ranges equal one
        st = SP.attention_partial(q, k[:7], v[:7], None, d ** -0.5)
        st = SP.attention_partial(q, k[7:], v[7:], st, d ** -0.5)
        assert torch.allclose(SP.attention_finish(st), SP.attention_finish(SP.attention_partial(q, k, v, None, d ** -0.5)),
                              rtol=1e-5, atol=1e-6)
    dist.barrier()
    if rank == 0:
        print("SP_WORKER_OK", flush=True)
    dist.destroy_process_group()


if __name__ == "__main__":
    main()
