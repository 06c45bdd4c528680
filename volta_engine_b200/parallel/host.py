"""CPU (gloo) communicator: the tensor-parallel interface over host tensors, used by the multi-process tests of
the scheduler, the control channel and failure handling. Sums run in fp32 whatever the tensor's dtype."""
from __future__ import annotations

import torch
import torch.distributed as dist

from ..ops import kernels as K


class HostComm:
    name = "gloo"

    def __init__(self, group=None):
        self.group = group or dist.group.WORLD
        self.rank, self.size = dist.get_rank(self.group), dist.get_world_size(self.group)

    def partial_buffer(self, rows, H):
        return None

    def shard_rows(self, x):
        return x

    def rows_per_rank(self, T):
        return T

    def allreduce_(self, x):
        f = x.float()
        dist.all_reduce(f, group=self.group)
        x.copy_(f)
        return x

    def allreduce_add_norm(self, partial, residual, w, eps, wbias=0.0, out=None):
        f = partial.float()
        dist.all_reduce(f, group=self.group)
        return K.rmsnorm(f.to(partial.dtype), w, eps, wbias, residual=residual, out=out)

    def all_gather_rows(self, x):
        parts = [torch.empty_like(x) for _ in range(self.size)]
        dist.all_gather(parts, x.contiguous(), group=self.group)
        return torch.cat(parts, 0)

    def merge_argmax(self, idx, val):
        vals = [torch.empty_like(val) for _ in range(self.size)]
        idxs = [torch.empty_like(idx) for _ in range(self.size)]
        dist.all_gather(vals, val.contiguous(), group=self.group)
        dist.all_gather(idxs, idx.contiguous(), group=self.group)
        v, i = torch.stack(vals), torch.stack(idxs)
        best = v.max(dim=0).values
        cand = torch.where(v == best[None], i, torch.full_like(i, 2 ** 31 - 1))
        return cand.min(dim=0).values.int()

    def barrier(self):
        dist.barrier(self.group)
