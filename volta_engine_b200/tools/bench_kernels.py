"""Kernel micro-benchmarks: CSV of (kernel, shape, rows, microseconds, GB/s or TFLOP/s, fraction of the measured peak).

Timing: CUDA events around one CUDA-graph replay that holds ``reps`` back-to-back launches over different weight
copies (so every launch streams from HBM, not L2), after warm-up; the L2 is also flushed before each replay.
``--iters N --no-graph`` launches N times eagerly instead (the form used under a profiler).
Reference: tests/3_bench/bench_kernels (CSV sweep compared against tests/baselines/kernels.csv).
"""
from __future__ import annotations

import argparse
import json
import os
import sys

import torch


def _peaks():
    p = os.path.join(os.path.dirname(os.path.dirname(os.path.dirname(os.path.abspath(__file__)))), "MEASURED_PEAKS.json")
    try:
        with open(p) as f:
            d = json.load(f)
        return float(d.get("hbm_gbs", 6650.0)), float(d.get("bf16_tflops", 1590.0)), "measured"
    except (OSError, ValueError):
        return 6650.0, 1590.0, "fallback"


def graph_time(fn, reps: int, flush: torch.Tensor, rounds: int = 5) -> float:
    """Median milliseconds per launch."""
    fn()
    torch.cuda.synchronize()
    g = torch.cuda.CUDAGraph()
    with torch.cuda.graph(g):
        for _ in range(reps):
            fn()
    for _ in range(3):
        g.replay()
    torch.cuda.synchronize()
    ts = []
    for _ in range(rounds):
        flush.zero_()
        torch.cuda.synchronize()
        a, b = torch.cuda.Event(True), torch.cuda.Event(True)
        a.record()
        g.replay()
        b.record()
        torch.cuda.synchronize()
        ts.append(a.elapsed_time(b) / reps)
    ts.sort()
    return ts[len(ts) // 2]


def main(argv=None) -> int:
    ap = argparse.ArgumentParser(prog="bench_kernels")
    ap.add_argument("--only", default="", help="comma list: decode_w4a4,nvfp4_gemv,exl3_gemv,gemm_w4a4,gemm_w4a16,gemm_bf16,attention")
    ap.add_argument("--shape", action="append", default=[], help="NxK (repeatable); default: the 27B layer shapes")
    ap.add_argument("--rows", default="1,4,16")
    ap.add_argument("--tokens", type=int, default=4096, help="rows of the GEMM benchmarks")
    ap.add_argument("--iters", type=int, default=0, help="with --no-graph: eager launches per case")
    ap.add_argument("--no-graph", action="store_true")
    ap.add_argument("--nsplit", type=int, default=0, help="attention: key splits per kv head (0 = the engine's choice)")
    a = ap.parse_args(argv)
    from ..ops import kernels as K
    from ..ops import linear_exl3 as LX
    from ..quant import nvfp4 as qn
    dev = torch.device("cuda:0")
    hbm, tfl, src = _peaks()
    only = set(x for x in a.only.split(",") if x)
    shapes = [tuple(int(v) for v in s.lower().split("x")) for s in a.shape] or \
        [(7168, 5120), (5120, 5120), (34816, 5120), (5120, 17408)]
    if only == {"attention"}:
        shapes = []
    rows = [int(r) for r in a.rows.split(",")]
    flush = torch.empty(256 << 20, dtype=torch.uint8, device=dev)
    print(f"kernel,N,K,rows,us,rate,unit,frac_of_{src}_peak")

    def run(name, fn, reps, nbytes=0, flops=0):
        if a.no_graph:
            for _ in range(max(1, a.iters)):
                fn()
            torch.cuda.synchronize()
            return None
        ms = graph_time(fn, reps, flush)
        if flops:
            rate = flops / ms / 1e9
            return f"{ms * 1e3:.1f},{rate:.0f},TFLOP/s,{rate / tfl:.3f}"
        rate = nbytes / ms / 1e6
        return f"{ms * 1e3:.1f},{rate:.0f},GB/s,{rate / hbm:.3f}"

    for (N, Kd) in shapes:
        copies = 1 if a.no_graph else max(2, min(12, (300 << 20) // (N * Kd // 2)))
        packed = [torch.randint(0, 255, (N, Kd // 2), dtype=torch.uint8, device=dev) for _ in range(copies)]
        scales = torch.randint(40, 60, (N, Kd // 16), dtype=torch.uint8, device=dev)
        atoms = qn.scales_atoms_512(scales) if N % 128 == 0 else None
        wbytes = N * Kd // 2 + N * Kd // 16
        idx = [0]

        def nxt():
            idx[0] = (idx[0] + 1) % copies
            return packed[idx[0]]
        for M in rows:
            x = torch.randn(M, Kd, device=dev).to(torch.bfloat16)
            out = torch.empty(M, N, dtype=torch.bfloat16, device=dev)
            if (not only or "decode_w4a4" in only) and atoms is not None and Kd % 256 == 0 and M <= 16:
                r = run("decode_w4a4", lambda: K.decode_w4a4(nxt(), atoms, 1.0, x, out=out), copies, wbytes)
                if r:
                    print(f"decode_w4a4,{N},{Kd},{M},{r}", flush=True)
            if (not only or "nvfp4_gemv" in only) and M <= 4:
                r = run("nvfp4_gemv", lambda: K.nvfp4_gemv(nxt(), scales, 1.0, x, out=out), copies, wbytes)
                if r:
                    print(f"nvfp4_gemv,{N},{Kd},{M},{r}", flush=True)
            if (not only or "exl3_gemv" in only) and N % 16 == 0 and Kd % 16 == 0 and M <= 16:
                codes = torch.randint(-32768, 32767, (Kd // 16, N // 16, 64), dtype=torch.int16, device=dev)
                xh = x.to(torch.float16)
                acc = torch.empty(M, N, dtype=torch.float32, device=dev)
                r = run("exl3_gemv", lambda: LX.exl3_gemv(codes, xh, M, Kd, N, 4, 2, out=acc), 1 if a.no_graph else 4,
                        codes.numel() * 2)
                if r:
                    print(f"exl3_gemv_4bit,{N},{Kd},{M},{r}", flush=True)
        T = a.tokens
        xt = torch.randn(T, Kd, device=dev).to(torch.bfloat16)
        fl = 2.0 * T * N * Kd
        if (not only or "gemm_w4a16" in only) and N % 128 == 0 and Kd % 128 == 0:
            sf = qn.scales_blocked_k128(scales)
            r = run("gemm_w4a16", lambda: K.gemm_w4a16(packed[0], sf, 1.0, xt), 1 if a.no_graph else 3, flops=fl)
            if r:
                print(f"gemm_w4a16,{N},{Kd},{T},{r}", flush=True)
        if (not only or "gemm_w4a4" in only) and atoms is not None and Kd % 256 == 0:
            xp, xs = K.nvfp4_quant_rows(xt, blocked=True)
            r = run("gemm_w4a4", lambda: K.gemm_w4a4(packed[0], atoms, 1.0, xp, xs, T), 1 if a.no_graph else 3, flops=fl)
            if r:
                print(f"gemm_w4a4,{N},{Kd},{T},{r}", flush=True)
        if not only or "gemm_bf16" in only:
            wb = torch.randn(N, Kd, device=dev).to(torch.bfloat16)
            r = run("gemm_bf16", lambda: K.gemm_bf16(wb, xt), 1 if a.no_graph else 3, flops=fl)
            if r:
                print(f"gemm_bf16,{N},{Kd},{T},{r}", flush=True)
            del wb
        del packed
    if not only or "attention" in only:
        # decode attention of the 27B shape: 40 q / 8 kv heads, head_dim 128, one row, `ctx` keys in 64-token pages
        import math
        nq, nkv, hd = 40, 8, 128
        for ctx in (4096, 16384, 65536):
            pages = ctx // 64 + 2
            kpool = torch.randn(pages, nkv, 64, hd, device=dev).to(torch.bfloat16)
            vpool = torch.randn(pages, nkv, 64, hd, device=dev).to(torch.bfloat16)
            table = torch.arange(1, pages, dtype=torch.int32, device=dev)[None].contiguous()
            pos = torch.tensor([ctx - 1], dtype=torch.int32, device=dev)
            slot = torch.zeros(1, dtype=torch.int32, device=dev)
            q = torch.randn(1, (nq + 2 * nkv) * hd, device=dev).to(torch.bfloat16)
            ws = K.AttnWorkspace(1, nq, hd, 64, dev)
            out = torch.empty(1, nq * hd, dtype=torch.bfloat16, device=dev)
            nsplit = a.nsplit or min(32, max(1, 148 * 3 // nkv))
            fn = lambda: K.attention(q, pos, slot, table, kpool, vpool, nq, nkv, hd, 1 / math.sqrt(hd), out=out,
                                     nsplit=nsplit, ws=ws)
            r = run("attention", fn, 1 if a.no_graph else 4, nbytes=2 * ctx * nkv * hd * 2)
            if r:
                print(f"attention_decode_ctx,{ctx},{hd},1,{r}", flush=True)
            del kpool, vpool
    st = K.check_status(dev)
    print(f"# device_status {st}")
    return 0 if st == 0 else 1


if __name__ == "__main__":
    sys.exit(main())
