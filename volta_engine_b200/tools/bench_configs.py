"""The other headline configurations behind ``bench.py --config``: full layer and expert counts, random weights drawn
directly in their storage format (so a 77 B-parameter model initialises in seconds), synthetic token ids.

  moe80b     48 layers, hidden 2048, 512 routed experts top-10 + shared expert, GQA attention; experts sharded over the
             ranks (expert parallel) with tensor-parallel attention. The routed experts are NVFP4 (4.5 bpw), this engine's
             native format; the reference's row runs EXL3 4.0 bpw experts (next entry).
  moe80b_exl3  the same model with the routed experts as EXL3 4.0 bpw trellis codes (the reference row's format).
  mla_mtp    46 layers MLA attention + 128 experts top-8 + shared, one MTP layer drafting 3 tokens per round. NVFP4.
  flash_next the Flash-Next assembly (48 layers, GDN + block-sparse attention, 512 experts, gated residual streams, MTP).
  qwen3_5    the 27B hybrid assembly (48 GDN + 16 gated attention layers, dense FFN, MTP head).
  glm5_next  the GLM-5-Next assembly (45 layers: 34 KDA mixers + 11 latent-attention layers with the sparse indexer, 288
             experts top-8 + shared, hyper-connection streams, MTP head).
  dsv3_gguf  DeepSeek-V3 shape (61 layers, 3 dense, 256 experts sigmoid top-8 in 8 groups / top-4), dense linears Q4_K,
             routed experts IQ2_XXS (gate / up) + Q4_K (down) as GGUF blocks. Needs the memory of 4 or more GPUs.

Measured, all on the device with CUDA events, max over ranks: prefill of ``--prompt-len`` tokens, single-stream greedy
decode (CUDA-graph replays chained on the device), a 16-stream decode step, the latency of verify blocks of 1 / 2 / 4 / 8
/ 16 rows, the end-to-end rate through ``Engine.step`` (pinned H2D row descriptor, D2H token, every step) and, for
``mla_mtp``, speculative rounds with the MTP head (rounds per second, accepted drafts per round; random weights accept
almost nothing, so tokens per second at a real acceptance rate is rounds/s x (1 + accepted)).
Reference rows: docs/PERFORMANCE.md:77-87 (EP scaling of the 512-expert model), :126-133 (MTP verify and decode rates).
"""
from __future__ import annotations

import json
import os
import time

import torch

CONFIGS = ("moe80b", "moe80b_exl3", "mla_mtp", "dsv3_gguf", "flash_next", "qwen3_5", "glm5_next")


def build(name: str, dev, comm, layers: int):
    if name == "moe80b":
        from ..models.moe import MoEConfig, MoEModel
        cfg = MoEConfig.baseline_moe()
        cfg.expert_quant = "nvfp4_random"
        klass, note = MoEModel, "routed experts NVFP4 4.5 bpw (reference row: EXL3 4.0 bpw, see moe80b_exl3)"
    elif name == "moe80b_exl3":
        from ..models.moe import MoEConfig, MoEModel
        cfg = MoEConfig.baseline_moe()
        cfg.expert_quant = "exl3_4"
        klass, note = MoEModel, "routed experts EXL3 4.0 bpw (trellis codes drawn at random), dense linears NVFP4"
    elif name == "mla_mtp":
        from ..models.mla import MLAConfig, MLAModel
        cfg = MLAConfig.baseline_mla_mtp()
        cfg.expert_quant = "nvfp4_random"
        klass, note = MLAModel, "NVFP4 weights (reference row: EXL3 3.05 bpw)"
    elif name in ("flash_next", "qwen3_5"):
        from ..models.hybrid import HybridConfig, HybridModel
        cfg = HybridConfig.flash_next() if name == "flash_next" else HybridConfig.qwen3_5_27b()
        cfg.expert_quant = "nvfp4_random"
        klass = HybridModel
        note = ("GDN + QSA attention, 512 NVFP4 experts + gated shared expert, gated residual streams, MTP head" if name == "flash_next"
                else "48 GDN + 16 gated attention layers, dense FFN, NVFP4, MTP head")
    elif name == "glm5_next":
        from ..models.glm5 import Glm5NextConfig, Glm5NextModel
        cfg = Glm5NextConfig.glm5_next()
        cfg.expert_quant = "nvfp4_random"
        klass, note = Glm5NextModel, "KDA mixers + latent attention with the sparse indexer, 288 NVFP4 experts + shared, hyper-connection streams, MTP head"
    elif name == "dsv3_gguf":
        from ..models.mla import MLAConfig, MLAModel
        cfg = MLAConfig.baseline_dsv3()
        cfg.quant = "gguf_q4_k"
        cfg.expert_quant = "gguf_iq2_xxs+q4_k"
        klass, note = MLAModel, "dense linears Q4_K, experts IQ2_XXS gate/up + Q4_K down (GGUF blocks drawn at random)"
    else:
        raise ValueError(name)
    if layers:
        cfg.n_layers = layers
        cfg.first_dense_layers = min(cfg.first_dense_layers, max(0, layers - 1))
    model = klass(cfg, dev, comm).init_random(seed=1)
    if getattr(cfg, "residual", "plain") != "plain":
        model.init_stream_weights()
    return model, cfg, note


def run(args, ClockSampler) -> int:
    import torch.distributed as dist
    from .. import _lib
    from ..ops import kernels as K
    from ..runtime.engine import Engine
    from ..runtime.kv_cache import PagedKVCache
    world = int(os.environ.get("WORLD_SIZE", "1"))
    rank = int(os.environ.get("RANK", "0"))
    local = int(os.environ.get("LOCAL_RANK", "0"))
    torch.cuda.set_device(local)
    dev = torch.device("cuda", local)
    comm = None
    if world > 1:
        os.environ.setdefault("MASTER_ADDR", "127.0.0.1")
        dist.init_process_group("nccl", device_id=dev)
        from ..parallel import make_comm
        comm = make_comm(args.comm, dev)

    def barrier():
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()

    def mx(ms: float) -> float:
        if world == 1:
            return ms
        t = torch.tensor([ms], dtype=torch.float64, device=dev)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        return float(t.item())

    t0 = time.time()
    model, cfg, note = build(args.config, dev, comm, args.layers)
    torch.cuda.synchronize()
    init_s = time.time() - t0
    steps, warm = args.steps, max(3, args.warmup)
    plen = min(args.prompt_len, 8192)
    streams = 16
    max_seq = plen + 4 * (steps + warm) + 256
    mla = hasattr(cfg, "q_lora_rank")
    n_cache = model.kv_layers if hasattr(type(model), "kv_layers") and isinstance(getattr(type(model), "kv_layers"), property) \
        else cfg.n_layers + getattr(cfg, "mtp_layers", 0)
    pages = streams * ((max_seq + 63) // 64 + 2)
    if mla:
        kv = PagedKVCache(n_cache, 1, 576, pages, streams, max_seq, dev, v_head_dim=8)
    else:
        kv = PagedKVCache(n_cache, model.nkv, cfg.head_dim, pages, streams, max_seq, dev)
    eng = Engine(model, kv, prefill_chunk=min(args.prefill_chunk, 2048), feedback=True)
    prompt = torch.randint(0, cfg.vocab, (plen,), generator=torch.Generator().manual_seed(0)).tolist()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)

    eng.prefill(0, prompt[:512])
    kv.release(0)
    barrier()
    e0.record()
    first = eng.prefill(0, prompt)
    e1.record()
    barrier()
    prefill_ms = mx(e0.elapsed_time(e1))

    # single-stream decode: graph replays chained on the device
    pos = plen
    l1 = _lib.launch_count
    eng.decode_chain([first], [pos], [0], 1)
    per_step = _lib.launch_count - l1
    pos += 1
    toks = eng.decode_chain([int(eng.s_tok[0].item())], [pos], [0], warm)
    pos += warm
    eng.kv.reserve(0, pos + steps + 2)
    eng.set_rows([int(toks[-1, 0].item())], [pos], [0])
    barrier()
    sampler = ClockSampler(local)
    sampler.start()
    e0.record()
    for _ in range(steps):
        eng._run_rows(1)
    e1.record()
    barrier()
    dec_ms = mx(e0.elapsed_time(e1))
    clocks = sampler.stop()
    pos += steps

    # verify blocks of 1..16 rows of the same sequence (what a speculative round costs), graph replays
    verify = {}
    eng.feedback = False
    for rows in (1, 2, 4, 8, 16):
        ids = [5 + i for i in range(rows)]
        for _ in range(3):
            eng.step(ids, [pos + i for i in range(rows)], [0] * rows)
        barrier()
        e0.record()
        for _ in range(16):
            eng._run_rows(rows)
        e1.record()
        barrier()
        verify[str(rows)] = round(mx(e0.elapsed_time(e1)) / 16, 4)

    # 16 concurrent streams: short prompts in the other slots, then one batched step
    for s in range(1, streams):
        eng.prefill(s, prompt[:256])
    ids, poss, slots = [7] * streams, [pos] + [256] * (streams - 1), list(range(streams))
    for _ in range(3):
        eng.step(ids, poss, slots)
    barrier()
    e0.record()
    for _ in range(16):
        eng._run_rows(streams)
    e1.record()
    barrier()
    batch_ms = mx(e0.elapsed_time(e1)) / 16

    # end to end: host round trip every step
    tok = 9
    for _ in range(3):
        tok = eng.step([tok], [pos], [0])[0]
        pos += 1
    barrier()
    e0.record()
    for _ in range(steps):
        tok = eng.step([tok], [pos], [0])[0]
        pos += 1
    e1.record()
    barrier()
    e2e_ms = mx(e0.elapsed_time(e1))

    spec = None
    if getattr(model, "mtp", None) is not None and world == 1:
        from ..runtime.mtp_runner import MtpRunner
        run_ = MtpRunner(eng, depth=3)
        kv.release(1)
        t = run_.prefill_rows(1, prompt[:1024], 0, 1024, True)
        p = 1024
        for _ in range(4):
            new = run_.round(1, t, p)
            t, p = new[-1], p + len(new)
        barrier()
        n0, a0 = run_.stats["rounds"], run_.stats["accepted"]
        e0.record()
        for _ in range(32):
            new = run_.round(1, t, p)
            t, p = new[-1], p + len(new)
        e1.record()
        barrier()
        ms = e0.elapsed_time(e1) / 32
        spec = {"depth": 3, "round_ms": round(ms, 4), "rounds_per_s": round(1e3 / ms, 1),
                "accepted_per_round": round((run_.stats["accepted"] - a0) / max(1, run_.stats["rounds"] - n0), 3),
                "note": "random weights: the head's drafts are almost never accepted; tok/s = rounds/s x (1 + accepted)"}

    status = K.check_status(dev)
    if rank == 0:
        tok_s = steps / (dec_ms / 1e3)
        out = {"metric": "decode_tok_s_1stream", "value": round(tok_s, 2), "unit": "tok/s", "n_gpus": world, "steps": steps,
               "warmup": warm, "ms_per_step": round(dec_ms / steps, 4), "higher_is_better": True, "scaling": "strong",
               "vs_baseline": None, "dtype": "bf16", "data": "synthetic (random token ids; weights drawn at random in their storage format)",
               "config": {"model": args.config, "layers": cfg.n_layers, "experts": cfg.n_experts, "top_k": cfg.top_k,
                          "hidden": cfg.hidden, "global_batch": 1, "seq_len": plen, "parallelism": f"tp{world}+ep{world}",
                          "weights": note, "l2": "inputs larger than L2 (weights streamed per step >> 126 MB)"},
               "prefill_tok_s": round(plen / (prefill_ms / 1e3), 1), "verify_ms_by_rows": verify,
               "decode_16_streams": {"ms_per_step": round(batch_ms, 4), "tok_s": round(streams / (batch_ms / 1e3), 1)},
               "e2e": {"value": round(steps / (e2e_ms / 1e3), 2), "unit": "tok/s", "h2d_bytes_per_step": 12,
                       "d2h_bytes_per_step": 4},
               "gpu_launches": per_step * steps, "launches_per_step": per_step, "clocks": clocks, "device_status": status,
               "init_s": round(init_s, 1)}
        if spec:
            out["mtp"] = spec
        print(json.dumps(out))
    if world > 1:
        dist.barrier()
        dist.destroy_process_group()
    return 0
