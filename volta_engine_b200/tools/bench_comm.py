"""Device-timed latency of the engine's tensor-parallel collectives (run under torchrun, one rank per GPU):

    python -m torch.distributed.run --nnodes=1 --nproc-per-node N --master-addr 127.0.0.1 --master-port P \
        -m volta_engine_b200.tools.bench_comm [--hidden 5120] [--iters 200] [--step-layers 8]

Measured, CUDA events around CUDA-graph replays, warm-up first, max over ranks:
  * one-shot LL all-reduce of 1 / 4 / 16 rows x H: plain, fused with residual add + RMSNorm, and the pair
    "decode linear that sends its rows from its own epilogue + all-reduce that only waits, adds and normalises";
  * two-shot reduce-scatter + norm + all-gather of a 2048-row chunk with plain peer loads and with ``multimem``;
  * the NCCL all-reduce of the same payloads (library A/B);
  * (``--step-layers L``) one decode step of an L-layer 27B-shaped model: time per step and the launch count.
Roofline column: bytes every rank must receive over NVLink (LL lines carry 8 payload bytes per 16) divided by the time,
against the measured 770 GB/s per direction; for these small payloads the number shows how far from bandwidth (that is:
how latency-bound) each form is. Waiting kernels are never run under a multi-pass profiler.
Reference counterpart: tests/3_bench/bench_all_reduce.cpp, bench_allreduce.cpp (NCCL vs own collective).
"""
from __future__ import annotations

import argparse
import json
import os

import torch
import torch.distributed as dist

NVLINK_GBS = 770.0


def _time_graph(fn, iters: int, inner: int, dev) -> float:
    """Microseconds per call of ``fn``: a graph of ``inner`` calls replayed ``iters`` times."""
    for _ in range(3):
        fn()
    torch.cuda.synchronize(dev)
    dist.barrier()
    g = torch.cuda.CUDAGraph()
    with torch.cuda.graph(g):
        for _ in range(inner):
            fn()
    for _ in range(3):
        g.replay()
    torch.cuda.synchronize(dev)
    dist.barrier()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    for _ in range(iters):
        g.replay()
    e1.record()
    torch.cuda.synchronize(dev)
    us = e0.elapsed_time(e1) * 1e3 / (iters * inner)
    t = torch.tensor([us], dtype=torch.float64, device=dev)
    dist.all_reduce(t, op=dist.ReduceOp.MAX)
    return float(t.item())


def _time_eager(fn, iters: int, dev) -> float:
    for _ in range(5):
        fn()
    torch.cuda.synchronize(dev)
    dist.barrier()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    for _ in range(iters):
        fn()
    e1.record()
    torch.cuda.synchronize(dev)
    t = torch.tensor([e0.elapsed_time(e1) * 1e3 / iters], dtype=torch.float64, device=dev)
    dist.all_reduce(t, op=dist.ReduceOp.MAX)
    return float(t.item())


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--hidden", type=int, default=5120)
    ap.add_argument("--iters", type=int, default=200)
    ap.add_argument("--chunk", type=int, default=2048)
    ap.add_argument("--step-layers", type=int, default=0)
    ap.add_argument("--json", default="")
    args = ap.parse_args()
    local = int(os.environ.get("LOCAL_RANK", "0"))
    torch.cuda.set_device(local)
    dev = torch.device("cuda", local)
    dist.init_process_group("nccl", device_id=dev)
    rank, size = dist.get_rank(), dist.get_world_size()
    from ..ops import kernels as K
    from ..ops.linear import LinearNVFP4
    from ..parallel.symm import SymmComm
    H = args.hidden
    rows_out = []

    def emit(name, rows, us, recv_bytes, note=""):
        gbs = recv_bytes / us / 1e3 if us > 0 else 0.0
        rows_out.append({"form": name, "rows": rows, "us": round(us, 2), "recv_bytes": recv_bytes,
                         "gbs": round(gbs, 1), "frac_of_nvlink": round(gbs / NVLINK_GBS, 4), "note": note})
        if rank == 0:
            print(f"{name:34s} rows {rows:5d}  {us:8.2f} us  recv {recv_bytes/1024:8.1f} KiB  {gbs:7.1f} GB/s  "
                  f"{gbs / NVLINK_GBS:6.3f} of NVLink  {note}", flush=True)

    comm = SymmComm(dev, hidden_max=max(8192, H), chunk_rows=max(args.chunk, 512), use_nvls=True)
    w = torch.ones(H, dtype=torch.bfloat16, device=dev)
    for rows in (1, 4, 16):
        x = torch.randn(rows, H, device=dev).bfloat16()
        res = torch.zeros(rows, H, dtype=torch.bfloat16, device=dev)
        line_bytes = (size - 1) * rows * H * 4          # 16 B lines carry 8 payload bytes
        emit("ll_allreduce", rows, _time_graph(lambda: comm.allreduce_(x), args.iters, 16, dev), line_bytes)
        emit("ll_allreduce + add + rmsnorm", rows,
             _time_graph(lambda: comm.allreduce_add_norm(x, res, w, 1e-6, 0.0), args.iters, 16, dev), line_bytes)
        lin = LinearNVFP4.from_dense(torch.randn(H, 2176, device=dev) * 0.02, search=False).prepare()
        xin = torch.randn(rows, 2176, device=dev).bfloat16()

        def pair():
            y = lin.forward(xin, push=comm)
            comm.allreduce_add_norm(y, res, w, 1e-6, 0.0)

        t_pair = _time_graph(pair, args.iters, 8, dev)
        t_lin = _time_graph(lambda: lin.forward(xin), args.iters, 8, dev)
        emit("linear(send) + allreduce(norm)", rows, t_pair, line_bytes, f"linear alone {t_lin:.2f} us")
        xn = x.clone()
        emit("nccl all_reduce (eager)", rows, _time_eager(lambda: dist.all_reduce(xn), args.iters, dev),
             2 * (size - 1) * rows * H * 2 // size, "library A/B")
    T = args.chunk
    rs_bytes = (size - 1) * (T // size) * H * 2 * 2          # pull the shard from the peers + receive the gathered rows
    for c2 in ((comm, SymmComm(dev, hidden_max=max(8192, H), chunk_rows=max(args.chunk, 512), use_nvls=False))
               if comm.use_nvls else (comm,)):
        part = c2.partial_buffer(T, H)
        part.copy_(torch.randn(T, H, device=dev).bfloat16())
        shard = torch.zeros(c2.rows_per_rank(T), H, dtype=torch.bfloat16, device=dev)
        emit(f"rs + norm + ag ({'multimem' if c2.use_nvls else 'peer loads'})", T,
             _time_graph(lambda: c2.allreduce_add_norm(part, shard, w, 1e-6, 0.0), max(20, args.iters // 10), 4, dev), rs_bytes)
    big = torch.randn(T, H, device=dev).bfloat16()
    emit("nccl all_reduce (eager)", T, _time_eager(lambda: dist.all_reduce(big), max(20, args.iters // 10), dev),
         2 * (size - 1) * T * H * 2 // size, "library A/B")
    last_comm = comm

    if args.step_layers > 0:
        from .. import _lib
        from ..models.dense import DenseConfig, DenseModel
        from ..runtime.engine import Engine
        from ..runtime.kv_cache import PagedKVCache
        cfg = DenseConfig.baseline_27b()
        cfg.n_layers = args.step_layers
        model = DenseModel(cfg, dev, last_comm).init_random(seed=1, search=False)
        plen = 2048
        kv = PagedKVCache(cfg.n_layers, model.nkv, cfg.head_dim, plen // 64 + 8, 1, plen + 512, dev)
        eng = Engine(model, kv, prefill_chunk=2048)
        prompt = torch.randint(0, cfg.vocab, (plen,), generator=torch.Generator().manual_seed(0)).tolist()
        tok = eng.prefill(0, prompt)
        l0 = _lib.launch_count
        eng.decode_chain([tok], [plen], [0], 1)
        launches = _lib.launch_count - l0
        eng.decode_chain([tok], [plen + 1], [0], 4)
        eng.kv.reserve(0, plen + 300)
        eng.set_rows([tok], [plen + 5], [0])
        torch.cuda.synchronize(dev)
        dist.barrier()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        for _ in range(64):
            eng._run_rows(1)
        e1.record()
        torch.cuda.synchronize(dev)
        t = torch.tensor([e0.elapsed_time(e1) * 1e3 / 64], dtype=torch.float64, device=dev)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        if rank == 0:
            us = float(t.item())
            print(f"decode step, {args.step_layers} layers of the 27B shape, tp{size}: {us:.1f} us / step, {launches} launches / step, "
                  f"{us / args.step_layers:.1f} us / layer, device status {K.check_status(dev)}", flush=True)
            rows_out.append({"form": "decode step", "layers": args.step_layers, "us": round(us, 1), "launches": launches})
    if rank == 0 and args.json:
        with open(args.json, "w") as f:
            json.dump({"world": size, "hidden": H, "rows": rows_out}, f, indent=1)
    dist.barrier()
    dist.destroy_process_group()


if __name__ == "__main__":
    main()
