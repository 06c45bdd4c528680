"""Device-timed prompt pieces through tiered MoE layers: cold experts read in place from pinned host memory for every
route, against cold experts copied once per layer into device scratch a layer ahead (``expert_stage``).

    python -m volta_engine_b200.tools.bench_expert_stage [--layers 4] [--experts 128] [--top-k 8] [--hidden 2048]
                                                         [--expert-ffn 768] [--resident 0.5] [--rows 1024] [--iters 3]

One iteration = the routed FFN blocks of all layers on ``--rows`` random rows (attention is left out: it does not touch the
experts). The two arms run the same route-indexed kernel on the same codes, so their outputs are compared bit for bit
before anything is timed. CUDA events around ``--iters`` iterations after two warm-up iterations.
Reference counterpart: src/backend/cuda/modules/expert_tier.cu:126 (staging a layer ahead), docs/CONFIG.md:91.
"""
from __future__ import annotations

import argparse
import json

import torch


def main(argv=None) -> int:
    from ..models.moe import MoEConfig, MoEModel
    ap = argparse.ArgumentParser()
    ap.add_argument("--layers", type=int, default=4)
    ap.add_argument("--experts", type=int, default=128)
    ap.add_argument("--top-k", type=int, default=8)
    ap.add_argument("--hidden", type=int, default=2048)
    ap.add_argument("--expert-ffn", type=int, default=768)
    ap.add_argument("--resident", type=float, default=0.5)
    ap.add_argument("--rows", type=int, default=1024)
    ap.add_argument("--iters", type=int, default=3)
    a = ap.parse_args(argv)
    dev = "cuda"
    cfg = MoEConfig(n_layers=a.layers, hidden=a.hidden, n_q=16, n_kv=2, head_dim=128, ffn=0, vocab=1024, n_experts=a.experts,
                    top_k=a.top_k, expert_ffn=a.expert_ffn, shared_ffn=0, router="softmax", expert_quant="nvfp4_random")
    m = MoEModel(cfg, dev).init_random(seed=3)
    hot = max(1, int(a.experts * a.resident))
    tiers = m.enable_expert_tier(hot)
    idx = [li for li, _ in tiers]
    g = torch.Generator(device=dev).manual_seed(1)
    x = torch.randn(a.rows, a.hidden, generator=g, device=dev).to(torch.bfloat16)

    def step():
        y = None
        for li in idx:
            y = m.ffn_block(li, m.layers[li], x, None, None)
        return y

    def timed():
        for _ in range(2):
            step()
        torch.cuda.synchronize()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        for _ in range(a.iters):
            step()
        e1.record()
        torch.cuda.synchronize()
        return e0.elapsed_time(e1) / a.iters

    want = step().clone()
    in_place_ms = timed()
    st = m.enable_expert_staging()
    if st is None:
        print(json.dumps({"error": "staging scratch does not fit in free device memory"}))
        return 1
    same = bool(torch.equal(step(), want))
    c0, b0 = st.copies, st.bytes_staged
    staged_ms = timed()
    per_iter = (st.bytes_staged - b0) / (a.iters + 2)
    t0 = tiers[0][1]
    per_expert = sum(t0.cold[n][0].numel() * t0.cold[n].element_size() for n in t0.NAMES)
    print(json.dumps({"layers": len(idx), "experts": a.experts, "resident": hot, "top_k": a.top_k, "rows": a.rows,
                      "expert_mib": round(per_expert / 2**20, 3), "bit_equal": same,
                      "in_place_ms": round(in_place_ms, 3), "staged_ms": round(staged_ms, 3),
                      "speedup": round(in_place_ms / staged_ms, 2), "staged_mib_per_iter": round(per_iter / 2**20, 1),
                      "staged_gb_per_s_over_iteration": round(per_iter / (staged_ms * 1e-3) / 1e9, 1),
                      "layer_copies_per_iter": (st.copies - c0) / (a.iters + 2)}))
    return 0 if same else 1


if __name__ == "__main__":
    raise SystemExit(main())
