"""Tensor-parallel communicator built on peer-mapped symmetric memory and the engine's own NVLink
kernels (csrc/cuda/comm.cu): one-shot LL all-reduce fused with residual add + RMSNorm for decode rows,
two-shot reduce-scatter + norm + all-gather (peer loads or NVLS ``multimem``) for prefill chunks, and a
device-side shard-argmax merge.

Bootstrap uses ``torch.distributed`` (NCCL process group) only to rendezvous the symmetric allocation;
the hot path issues no NCCL call. Reference counterpart: ``init_4gpu_mesh`` + ``CollectiveRing``
(src/comm/all_reduce_ipc.cu:961-987, inc/engine/core/comm.h:18-93), which caps at 4 ranks; this one
runs 2, 4 or 8.
"""
from __future__ import annotations

import ctypes
import os

import torch
import torch.distributed as dist

from .. import _lib
from ..ops import kernels as K

MAX_RANKS = 8
LL_STAGES = 4
LL_MAX_ROWS = 16


class CommArgs(ctypes.Structure):
    """Mirror of ``ve::CommArgs`` (csrc/cuda/comm.cu)."""
    _fields_ = [("peer", ctypes.c_void_p * MAX_RANKS), ("mc", ctypes.c_void_p), ("rank", ctypes.c_int),
                ("size", ctypes.c_int), ("seq", ctypes.c_void_p), ("status", ctypes.c_void_p),
                ("budget_ns", ctypes.c_ulonglong), ("off_ll", ctypes.c_size_t), ("ll_row_bytes", ctypes.c_size_t),
                ("off_flags", ctypes.c_size_t), ("off_part", ctypes.c_size_t), ("off_xout", ctypes.c_size_t)]


def _round_up(x, m):
    return (x + m - 1) // m * m


class SymmComm:
    name = "symm"

    def __init__(self, device, hidden_max: int = 8192, chunk_rows: int = 4096, use_nvls: bool | None = None,
                 budget_ms: float = 1000.0, group=None):
        import torch.distributed._symmetric_memory as symm_mem
        self.device = torch.device(device)
        self.group = group or dist.group.WORLD
        self.rank, self.size = dist.get_rank(self.group), dist.get_world_size(self.group)
        assert self.size <= MAX_RANKS
        self.hidden_max, self.chunk_rows = hidden_max, _round_up(chunk_rows, self.size)
        self.max_ctas = 512
        off_flags = 0
        off_ll = 64 * 1024
        ll_row_bytes = hidden_max * 4
        ll_bytes = LL_STAGES * MAX_RANKS * LL_MAX_ROWS * ll_row_bytes
        off_part = _round_up(off_ll + ll_bytes, 1 << 16)
        part_bytes = self.chunk_rows * hidden_max * 2
        off_xout = off_part + _round_up(part_bytes, 1 << 16)
        total = off_xout + _round_up(part_bytes, 1 << 16)
        self.buf = symm_mem.empty(total, dtype=torch.uint8, device=self.device)
        self.buf.zero_()
        torch.cuda.synchronize(self.device)
        self.hdl = symm_mem.rendezvous(self.buf, self.group)
        mc = int(getattr(self.hdl, "multicast_ptr", 0) or 0)
        if use_nvls is None:
            use_nvls = os.environ.get("VOLTA_NVLS", "1") != "0"
        self.use_nvls = bool(use_nvls and mc)
        self.seq = torch.ones(4, dtype=torch.int32, device=self.device)
        self.seq[1] = 0
        self.seq[3] = 0
        self.status = K.status_word(self.device)
        a = CommArgs()
        for i, p in enumerate(self.hdl.buffer_ptrs):
            a.peer[i] = p
        a.mc = mc if self.use_nvls else 0
        a.rank, a.size = self.rank, self.size
        a.seq, a.status = self.seq.data_ptr(), self.status.data_ptr()
        a.budget_ns = int(budget_ms * 1e6)
        a.off_ll, a.ll_row_bytes, a.off_flags, a.off_part, a.off_xout = off_ll, ll_row_bytes, off_flags, off_part, off_xout
        self.args = a
        self._args_ptr = ctypes.addressof(a)
        self.off_part, self.off_xout = off_part, off_xout
        assert _lib.kernels().ve_comm_args_size() == ctypes.sizeof(CommArgs)
        self._arg_idx = torch.empty(LL_MAX_ROWS, dtype=torch.int32, device=self.device)
        self.pushed = False        # set by a linear whose epilogue already sent its rows (see push_target)
        self.fuse_push = os.environ.get("VOLTA_FUSE_PUSH", "1") != "0"
        # False (launch option ar_ll = false): decode rows take the two-shot collective too, followed by the add + norm
        # kernel; an A/B switch for the one-shot low-latency form
        self.use_ll = True
        dist.barrier(self.group)
        torch.cuda.synchronize(self.device)

    # ---- symmetric views -----------------------------------------------------------------------
    def partial_buffer(self, rows: int, H: int) -> torch.Tensor:
        """[rows, H] bf16 view of the two-shot input region: row-parallel GEMMs write here directly."""
        assert rows <= self.chunk_rows and H <= self.hidden_max
        return self.buf[self.off_part: self.off_part + rows * H * 2].view(torch.bfloat16).view(rows, H)

    def _xout(self, rows: int, H: int) -> torch.Tensor:
        return self.buf[self.off_xout: self.off_xout + rows * H * 2].view(torch.bfloat16).view(rows, H)

    def rows_per_rank(self, T: int) -> int:
        return (T + self.size - 1) // self.size

    def shard_rows(self, x: torch.Tensor) -> torch.Tensor:
        """This rank's row slice of a replicated [T, H] tensor (zero padded), for the sharded residual."""
        T, H = x.shape
        Tl = self.rows_per_rank(T)
        out = torch.zeros(Tl, H, dtype=x.dtype, device=x.device)
        lo = self.rank * Tl
        hi = min(T, lo + Tl)
        if hi > lo:
            out[: hi - lo] = x[lo:hi]
        return out

    def push_target(self, rows: int, H: int) -> int:
        """Address of the argument block for a producer kernel that sends its [rows, H] result into the peers' low-latency
        staging area itself (decode rows only), or 0 when the fused send does not apply."""
        if not self.fuse_push or not self.use_ll or rows > LL_MAX_ROWS or H * 4 > self.args.ll_row_bytes or H % 4:
            return 0
        return self._args_ptr

    # ---- collectives ---------------------------------------------------------------------------
    def allreduce_(self, x: torch.Tensor) -> torch.Tensor:
        rows, H = x.shape
        if rows <= LL_MAX_ROWS and self.use_ll:
            out = torch.empty_like(x)
            _lib.call("ll_allreduce", "piplpppliiff", self._args_ptr, 0, x.data_ptr(), x.stride(0), 0, 0,
                      out.data_ptr(), out.stride(0), rows, H, 0.0, 0.0)
            x.copy_(out)
            return x
        part = self.partial_buffer(rows, H)
        if x.data_ptr() != part.data_ptr():
            part.copy_(x)
        self._two_shot(None, None, rows, H, 0.0, 0.0, 0)
        x.copy_(self._xout(rows, H))
        return x

    def _two_shot(self, res_shard, w, T, H, eps, wbias, mode):
        Tl = self.rows_per_rank(T)
        ctas = min(self.max_ctas, max(1, min(Tl, 148 * 2)))
        _lib.call("rs_norm_ag", "pppiiiffiii", self._args_ptr, _lib.ptr(res_shard), _lib.ptr(w), T, Tl, H,
                  float(eps), float(wbias), mode, 1 if self.use_nvls else 0, ctas)

    def allreduce_add_norm(self, partial, residual, w, eps, wbias=0.0, out=None):
        """Decode rows (<= 16): ``residual`` is replicated [rows, H]. Prefill chunks: ``residual`` is this
        rank's row shard [ceil(rows/size), H] and ``partial`` should be ``partial_buffer(rows, H)``.
        Returns the normalised activations [rows, H] (replicated)."""
        rows, H = partial.shape
        pushed, self.pushed = self.pushed, False
        if rows <= LL_MAX_ROWS and not self.use_ll:
            part = self.partial_buffer(rows, H)
            part.copy_(partial)
            self._two_shot(None, None, rows, H, 0.0, 0.0, 0)
            return K.rmsnorm(self._xout(rows, H), w, eps, wbias, residual=residual, out=out)
        if rows <= LL_MAX_ROWS:
            if out is None:
                out = torch.empty_like(partial)
            _lib.call("ll_allreduce", "piplpppliiff", self._args_ptr, 3 if pushed else 1, partial.data_ptr(), partial.stride(0),
                      residual.data_ptr(), w.data_ptr(), out.data_ptr(), out.stride(0), rows, H, float(eps),
                      float(wbias))
            return out
        part = self.partial_buffer(rows, H)
        if partial.data_ptr() != part.data_ptr():
            part.copy_(partial)
        self._two_shot(residual, w, rows, H, eps, wbias, 1)
        return self._xout(rows, H)

    def allreduce_epilogue(self, mode: int, partial: torch.Tensor, epi_args: tuple) -> None:
        """All-reduce of <= 16 decode rows with a stream epilogue (ops/streams.py: 2 sandwich norm, 3 gated streams,
        4 hyper-connection update) applied to the reduced rows in the same launch; ``epi_args`` as packed there."""
        from ..ops.streams import LL_EPI_SIG
        pushed, self.pushed = self.pushed, False
        _lib.call("ll_allreduce_epi", LL_EPI_SIG, self._args_ptr, mode, 1 if pushed else 0, partial.data_ptr(),
                  partial.stride(0), *epi_args)

    def merge_argmax(self, idx: torch.Tensor, val: torch.Tensor) -> torch.Tensor:
        rows = idx.numel()
        _lib.call("ll_argmax_merge", "ppppi", self._args_ptr, idx.data_ptr(), val.data_ptr(),
                  self._arg_idx.data_ptr(), rows)
        return self._arg_idx[:rows]

    def all_gather_rows(self, x: torch.Tensor) -> torch.Tensor:
        """[n, ...] per rank -> [size * n, ...] (sampling path only; not on the greedy hot path)."""
        out = torch.empty((self.size * x.shape[0],) + tuple(x.shape[1:]), dtype=x.dtype, device=x.device)
        dist.all_gather_into_tensor(out, x.contiguous(), group=self.group)
        return out

    def barrier(self):
        dist.barrier(self.group)


class NcclComm:
    """Library baseline: NCCL all-reduce followed by the fused add + RMSNorm kernel (A/B reference for the
    engine's own collectives; also what the reference's video / training paths use NCCL for)."""
    name = "nccl"

    def __init__(self, device, group=None):
        self.device = torch.device(device)
        self.group = group or dist.group.WORLD
        self.rank, self.size = dist.get_rank(self.group), dist.get_world_size(self.group)

    def partial_buffer(self, rows, H):
        return None

    def shard_rows(self, x):
        return x

    def rows_per_rank(self, T):
        return T

    def allreduce_(self, x):
        dist.all_reduce(x, group=self.group)
        return x

    def allreduce_add_norm(self, partial, residual, w, eps, wbias=0.0, out=None):
        dist.all_reduce(partial, group=self.group)
        return K.rmsnorm(partial, w, eps, wbias, residual=residual, out=out)

    def all_gather_rows(self, x):
        out = torch.empty((self.size * x.shape[0],) + tuple(x.shape[1:]), dtype=x.dtype, device=x.device)
        dist.all_gather_into_tensor(out, x.contiguous(), group=self.group)
        return out

    def merge_argmax(self, idx, val):
        vals = [torch.empty_like(val) for _ in range(self.size)]
        idxs = [torch.empty_like(idx) for _ in range(self.size)]
        dist.all_gather(vals, val, group=self.group)
        dist.all_gather(idxs, idx, group=self.group)
        v, i = torch.stack(vals), torch.stack(idxs)
        best = v.max(dim=0).values
        cand = torch.where(v == best[None], i, torch.full_like(i, 2 ** 31 - 1))
        return cand.min(dim=0).values.int()

    def barrier(self):
        dist.barrier(self.group)
