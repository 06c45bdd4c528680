"""Tensor-parallel communicator interface and its single-GPU implementation.

The reference's ``CollectiveRing`` offers plain all-reduce plus forms fused with the residual add and
the next RMSNorm (inc/engine/core/comm.h:18-93, src/comm/all_reduce_ipc.cu:136-298). Models talk to
this small interface; multi-GPU implementations live in :mod:`volta_engine_b200.parallel.symm` (own
NVLink kernels over symmetric memory) and :mod:`volta_engine_b200.parallel.nccl` (library baseline).
"""
from __future__ import annotations

import torch

from ..ops import kernels as K


class LocalComm:
    """World of one GPU: the fused forms reduce to the fused add + RMSNorm kernel."""

    rank = 0
    size = 1
    name = "local"

    def allreduce_(self, x: torch.Tensor) -> torch.Tensor:
        return x

    def allreduce_add_norm(self, partial, residual, w, eps, wbias=0.0, out=None):
        """residual += sum_ranks(partial); returns RMSNorm(residual) * (w + wbias)."""
        return K.rmsnorm(partial, w, eps, wbias, residual=residual, out=out)

    def merge_argmax(self, idx: torch.Tensor, val: torch.Tensor):
        return idx

    def all_gather_rows(self, x: torch.Tensor) -> torch.Tensor:
        return x

    def barrier(self):
        pass
