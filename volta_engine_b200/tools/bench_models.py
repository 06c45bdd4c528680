"""``volta_bench_models``: single-stream decode rate of the other model families at a chosen shape (random weights).

  volta_bench_models --family dsv4 [--layers 6] [--experts 32] [--prompt 8192] [--steps 64] [--warmup 8] [--no-graphs]

The model is built from the family's published shape with ``--layers`` layers and ``--experts`` routed experts (the full
expert count of the large families does not fit one GPU with random initialisation in reasonable time), prefilled with
``--prompt`` random tokens, then decoded greedily; the decode steps are timed on the device. One JSON line is printed.
The flagship dense benchmark is ``bench.py`` at the repository root; this tool is for the per-family numbers beside it.
"""
from __future__ import annotations

import argparse
import json
import sys

import torch


def build(family: str, layers: int, experts: int, device):
    if family == "dsv4":
        from ..models.dsv4 import DSV4Config, DSV4Model
        cfg = DSV4Config.baseline_dsv41()
        ratios = ((0, 2, 2, 1, 1, 1) * ((layers + 5) // 6))[:layers]
        src = tuple(i for i in (1, 3) if i < layers)
        cfg.n_layers, cfg.compress_ratios, cfg.kv_sources = layers, ratios, src
        cfg.index_sources = tuple(i for i in range(layers) if ratios[i] > 0 and (i in src or i % 4 == 0))
        cfg.candidate_source = 3 if layers > 3 else -1
        cfg.engram_layers = (1,) if layers > 1 else ()
        cfg.n_experts, cfg.rms_eps = experts, 1e-6
        return DSV4Model(cfg, device).init_random(seed=1), cfg
    if family == "moe":
        from ..models.moe import MoEConfig, MoEModel
        cfg = MoEConfig.baseline_moe()
        cfg.n_layers, cfg.n_experts = layers, experts
        return MoEModel(cfg, device).init_random(seed=1), cfg
    if family == "mla":
        from ..models.mla import MLAConfig, MLAModel
        cfg = MLAConfig.baseline_mla_mtp()
        cfg.n_layers, cfg.n_experts, cfg.mtp_layers = layers, experts, 0
        return MLAModel(cfg, device).init_random(seed=1), cfg
    raise ValueError(f"unknown family {family!r}")


def main(argv=None) -> int:
    ap = argparse.ArgumentParser(prog="volta_bench_models", description=__doc__.split("\n\n")[0])
    ap.add_argument("--family", default="dsv4", choices=["dsv4", "moe", "mla"])
    ap.add_argument("--layers", type=int, default=6)
    ap.add_argument("--experts", type=int, default=32)
    ap.add_argument("--prompt", type=int, default=8192)
    ap.add_argument("--steps", type=int, default=64)
    ap.add_argument("--warmup", type=int, default=8)
    ap.add_argument("--chunk", type=int, default=512)
    ap.add_argument("--no-graphs", action="store_true")
    ap.add_argument("--profiler-range", action="store_true",
                    help="bracket the timed steps with cudaProfilerStart / Stop (for a profiler started with capture off)")
    a = ap.parse_args(argv)
    if not torch.cuda.is_available():
        print("volta_bench_models: needs a GPU", file=sys.stderr)
        return 1
    from ..runtime.engine import Engine
    from ..runtime.kv_cache import PagedKVCache
    dev = torch.device("cuda", 0)
    model, cfg = build(a.family, a.layers, a.experts, dev)
    total = a.prompt + a.steps + a.warmup + 64
    kv = PagedKVCache(getattr(model, "kv_layers", cfg.n_layers), model.nkv, model.hd if a.family == "dsv4" else cfg.head_dim,
                      (total + 63) // 64 + 2, 1, total, dev)
    eng = Engine(model, kv, use_graphs=not a.no_graphs, prefill_chunk=a.chunk)
    g = torch.Generator().manual_seed(0)
    prompt = torch.randint(0, cfg.vocab, (a.prompt,), generator=g).tolist()
    t0, t1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    t0.record()
    tok = eng.prefill(0, prompt)
    t1.record()
    torch.cuda.synchronize()
    prefill_ms = t0.elapsed_time(t1)
    pos = a.prompt
    for _ in range(a.warmup):
        tok = eng.step([tok], [pos], [0])[0]
        pos += 1
    torch.cuda.synchronize()
    if a.profiler_range:
        torch.cuda.profiler.start()
    t0.record()
    for _ in range(a.steps):
        tok = eng.step([tok], [pos], [0])[0]
        pos += 1
    t1.record()
    torch.cuda.synchronize()
    if a.profiler_range:
        torch.cuda.profiler.stop()
    ms = t0.elapsed_time(t1) / a.steps
    print(json.dumps({"family": a.family, "layers": a.layers, "experts": a.experts, "prompt": a.prompt, "graphs": not a.no_graphs,
                      "decode_tok_s": round(1e3 / ms, 2), "ms_per_step": round(ms, 4), "ms_per_layer": round(ms / a.layers, 4),
                      "prefill_tok_s": round(a.prompt / prefill_ms * 1e3, 1), "decode_gb_per_token": round(model.decode_bytes_per_token() / 1e9, 3)}))
    return 0


if __name__ == "__main__":
    sys.exit(main())
