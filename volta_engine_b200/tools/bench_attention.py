"""Device-timed prefill attention: the tcgen05 kernel (128-row query tiles, accumulators in TMEM) against the mma.sync
kernel (64-row tiles) on the same paged cache, plus a check of both against the fp32 oracle on a small case.

    python -m volta_engine_b200.tools.bench_attention [--ctx 16384] [--rows 4096] [--heads 40] [--kv-heads 8]
                                                      [--iters 10] [--only tc|mma] [--no-check]

One launch = the last ``--rows`` tokens of a ``--ctx``-token sequence attending causally to everything before them
(what one prefill chunk of a long prompt costs). FLOPs counted = 4 x head_dim x heads x sum over rows of (position + 1)
(QK^T and PV, causal); the K / V pages of the sequence (ctx x kv_heads x 128 x 2 x 2 bytes) stay in L2 between tiles,
so the roofline is the tensor core, not HBM. CUDA events around ``--iters`` launches after three warm-up launches.
Reference counterpart: src/backend/cuda/modules/attention.cu:817-822 (prefill attention dispatch).
"""
from __future__ import annotations

import argparse
import json
import math

import torch


def _rnd(*shape, seed=0, dev="cuda"):
    g = torch.Generator(device=dev).manual_seed(seed)
    return torch.randn(*shape, generator=g, device=dev).to(torch.bfloat16)


def _cache(nkv, hd, max_seq, dev, seed=0):
    npages = (max_seq + 63) // 64
    kpool, vpool = _rnd(npages + 2, nkv, 64, hd, seed=seed + 1, dev=dev), _rnd(npages + 2, nkv, 64, hd, seed=seed + 2, dev=dev)
    table = (torch.randperm(npages + 1, generator=torch.Generator().manual_seed(seed)) + 1)[:npages].int().view(1, -1).to(dev)
    return kpool, vpool, table


def main(argv=None) -> int:
    from ..ops import kernels as K
    from ..ops import reference as ref
    ap = argparse.ArgumentParser()
    ap.add_argument("--ctx", type=int, default=16384)
    ap.add_argument("--rows", type=int, default=4096)
    ap.add_argument("--heads", type=int, default=40)
    ap.add_argument("--kv-heads", type=int, default=8)
    ap.add_argument("--iters", type=int, default=10)
    ap.add_argument("--only", choices=("tc", "mma"), default=None)
    ap.add_argument("--no-check", action="store_true")
    a = ap.parse_args(argv)
    dev, hd, nq, nkv = "cuda", 128, a.heads, a.kv_heads
    scale = 1 / math.sqrt(hd)
    out = {"head_dim": hd, "heads": nq, "kv_heads": nkv, "ctx": a.ctx, "rows": a.rows}

    def run(tc, q, pos, slot, table, kp, vp, tiles, o=None):
        K.ATTN_PREFILL_TC = tc
        return K.attention(q, pos, slot, table, kp, vp, nq, nkv, hd, scale, tiles=tiles, out=o)

    if not a.no_check:
        n, start = 300, 700
        kp, vp, table = _cache(nkv, hd, start + n + 64, dev)
        pos = torch.arange(start, start + n, dtype=torch.int32, device=dev)
        slot = torch.zeros(n, dtype=torch.int32, device=dev)
        q = _rnd(n, (nq + 2 * nkv) * hd, seed=13, dev=dev)
        tiles = K.make_prefill_tiles([0] * n, nq // nkv, dev)
        want = ref.attention(q.cpu().float(), pos.cpu(), slot.cpu(), table.cpu(), kp.cpu(), vp.cpu(), nq, nkv, hd, scale).double()
        for name, tc in (("tc", True), ("mma", False)):
            got = run(tc, q, pos, slot, table, kp, vp, tiles).double().cpu()
            out[f"check_{name}"] = {"cos": round(float(torch.nn.functional.cosine_similarity(got.flatten(), want.flatten(), dim=0)), 7),
                                    "max_abs_err": round(float((got - want).abs().max()), 5), "ref_abs_max": round(float(want.abs().max()), 4)}
    kp, vp, table = _cache(nkv, hd, a.ctx + 64, dev)
    pos = torch.arange(a.ctx - a.rows, a.ctx, dtype=torch.int32, device=dev)
    slot = torch.zeros(a.rows, dtype=torch.int32, device=dev)
    q = _rnd(a.rows, (nq + 2 * nkv) * hd, seed=13, dev=dev)
    tiles = K.make_prefill_tiles([0] * a.rows, nq // nkv, dev)
    o = torch.empty(a.rows, nq * hd, dtype=torch.bfloat16, device=dev)
    flops = 4 * hd * nq * sum(range(a.ctx - a.rows + 1, a.ctx + 1))
    for name, tc in (("tc", True), ("mma", False)):
        if a.only and a.only != name:
            continue
        for _ in range(3):
            run(tc, q, pos, slot, table, kp, vp, tiles, o)
        torch.cuda.synchronize()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        for _ in range(a.iters):
            run(tc, q, pos, slot, table, kp, vp, tiles, o)
        e1.record()
        torch.cuda.synchronize()
        ms = e0.elapsed_time(e1) / a.iters
        out[name] = {"ms": round(ms, 4), "tflops": round(flops / ms / 1e9, 1), "tiles": int(tiles[3][2] if tc else tiles[2])}
    out["device_status"] = K.check_status(torch.device(dev))
    print(json.dumps(out))
    return 0


if __name__ == "__main__":
    raise SystemExit(main())
