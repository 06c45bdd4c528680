"""CPU-backend benchmark configuration: tiny dense GQA decoder, GGUF Q8_0 weights, batch 1, greedy decode of 128
tokens after a 64-token prompt (4 layers, hidden 512, 8 q / 2 kv heads of 64, RoPE theta 1e6, RMSNorm eps 1e-6,
SwiGLU 1408, vocab 32000, untied embeddings, weights N(0, 0.02) seed 0, prompt ids uniform seed 0).

Two activation semantics are run and compared token for token:
  * ``fp32``  fp32 activations against dequantised Q8_0 weights;
  * ``q8``    the reference CPU backend's arithmetic: activation rows quantised to Q8_0 before every product,
              integer block dots (src/backend/cpu/linear_gguf.cpp:65-113).
The reference's own CPU binary cannot be built offline (needs slangc and nlohmann-json), so this restatement is the
oracle and the timed CPU baseline.

    python -m volta_engine_b200.tools.bench_cpu_q8 [--tokens 128]
"""
from __future__ import annotations

import argparse
import json
import time

import torch

from ..models.dense import DenseConfig, DenseModel
from ..runtime.engine import Engine
from ..runtime.kv_cache import PagedKVCache


def config() -> DenseConfig:
    return DenseConfig(n_layers=4, hidden=512, n_q=8, n_kv=2, head_dim=64, ffn=1408, vocab=32000, rope_theta=1e6,
                       rms_eps=1e-6, quant="gguf_q8_0", gemm_mode="fp32")


def run(mode: str, tokens: int, device: str = "cpu"):
    cfg = config()
    cfg.gemm_mode = "q8_act" if mode == "q8" else "fp32"
    model = DenseModel(cfg, device).init_random(seed=0)
    kv = PagedKVCache(cfg.n_layers, model.nkv, cfg.head_dim, 8, 1, 64 + tokens + 64, device)
    eng = Engine(model, kv, use_graphs=device != "cpu", prefill_chunk=64)
    prompt = torch.randint(0, cfg.vocab, (64,), generator=torch.Generator().manual_seed(0)).tolist()
    t0 = time.perf_counter()
    out, st = eng.generate(prompt, tokens)
    return out, st, time.perf_counter() - t0


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--tokens", type=int, default=128)
    ap.add_argument("--device", default="cpu")
    a = ap.parse_args()
    o32, s32, t32 = run("fp32", a.tokens, a.device)
    oq8, sq8, tq8 = run("q8", a.tokens, a.device)
    agree = next((i for i, (x, y) in enumerate(zip(o32, oq8)) if x != y), len(o32))
    print(json.dumps({"config": "cpu tiny dense q8_0", "device": a.device, "tokens": a.tokens,
                      "fp32": {"decode_tok_s": round(s32.decode_tok_s, 2), "prefill_tok_s": round(s32.prefill_tok_s, 1)},
                      "q8_act": {"decode_tok_s": round(sq8.decode_tok_s, 2), "prefill_tok_s": round(sq8.prefill_tok_s, 1)},
                      "first_divergence": agree, "tokens_fp32_head": o32[:8], "tokens_q8_head": oq8[:8]}))


if __name__ == "__main__":
    main()
