"""``volta_server``: launch configuration and process start-up.

Precedence: command-line flags > JSON launch file > ``ENGINE_*`` environment > defaults; unknown keys are fatal;
the model type is never configured (``config.json`` of the model directory decides).
One process per GPU: with ``tp_size`` > 1 and no rank environment the launcher re-executes itself under
``torch.distributed.run`` on 127.0.0.1; rank 0 then hosts the HTTP front end and the scheduler, the other ranks
mirror its engine calls (runtime/tp_control.py).
Reference: inc/engine/server/config.h:21-52 (launch struct), src/server/config.cpp, docs/CONFIG.md:5-26,
src/server/main.cpp (start-up order: config -> cluster -> tokenizer / template -> generator -> HTTP).
"""
from __future__ import annotations

import argparse
import json
import os
import signal
import sys
import logging
import threading
from dataclasses import asdict, dataclass, field

from ..runtime.options import Options, config_docs

log = logging.getLogger("volta")

_TOP_KEYS = {
    "model_dir": (str, ""), "draft_model_dir": (str, ""), "use_speculation": (bool, False), "tui": (bool, False),
    "tp_size": (int, 1), "host": (str, "127.0.0.1"), "port": (int, 8080), "api_key": (str, ""),
    "max_batch_size": (int, 8), "default_max_tokens": (int, 1024), "default_temperature": (float, 0.7),
    "default_top_p": (float, 0.95), "default_top_k": (int, 0), "default_enable_thinking": (bool, True),
    "request_timeout_s": (int, 300), "model_name": (str, ""), "video": (dict, None), "options": (dict, None),
}


@dataclass
class LaunchConfig:
    model_dir: str = ""
    draft_model_dir: str = ""
    use_speculation: bool = False
    tui: bool = False
    tp_size: int = 1
    host: str = "127.0.0.1"
    port: int = 8080
    api_key: str = ""
    max_batch_size: int = 8
    default_max_tokens: int = 1024
    default_temperature: float = 0.7
    default_top_p: float = 0.95
    default_top_k: int = 0
    default_enable_thinking: bool = True
    request_timeout_s: int = 300
    model_name: str = ""
    video: dict = field(default_factory=dict)
    options: Options = None

    def to_dict(self):
        d = asdict(self)
        d["options"] = dict(self.options.values)
        return d


def _coerce(key, val):
    t = _TOP_KEYS[key][0]
    if t is bool and not isinstance(val, bool):
        return str(val).strip().lower() in ("1", "true", "yes", "on")
    if t is dict:
        if not isinstance(val, dict):
            raise ValueError(f"'{key}' must be an object")
        return val
    return t(val)


def build_parser() -> argparse.ArgumentParser:
    p = argparse.ArgumentParser(prog="volta_server", description="OpenAI / Anthropic compatible LLM server for B200")
    p.add_argument("config", nargs="?", help="JSON launch file")
    p.add_argument("--config", dest="config_flag", help="JSON launch file")
    p.add_argument("--model-dir")
    p.add_argument("--draft-model-dir")
    p.add_argument("--use-speculation", action="store_true", default=None)
    p.add_argument("--tui", action="store_true", default=None)
    p.add_argument("--tp", "--tp-size", dest="tp_size", type=int)
    p.add_argument("--host")
    p.add_argument("--port", type=int)
    p.add_argument("--api-key")
    p.add_argument("--max-batch-size", type=int)
    p.add_argument("--default-max-tokens", type=int)
    p.add_argument("--model-name")
    p.add_argument("--request-timeout-s", type=int)
    p.add_argument("--set", action="append", default=[], metavar="KEY=VALUE", help="runtime option (repeatable)")
    p.add_argument("--print-config", action="store_true", help="print the resolved configuration and exit")
    p.add_argument("--print-config-docs", action="store_true", help="print the option reference (markdown) and exit")
    return p


def resolve_config(argv: list[str], env=None) -> tuple[LaunchConfig, argparse.Namespace]:
    env = os.environ if env is None else env
    args = build_parser().parse_args(argv)
    vals = {k: d for k, (t, d) in _TOP_KEYS.items()}
    for k in vals:                                     # environment (lowest)
        raw = env.get("ENGINE_" + k.upper())
        if raw is not None and _TOP_KEYS[k][0] is not dict:
            vals[k] = _coerce(k, raw)
    path = args.config_flag or args.config
    json_options = None
    if path:
        with open(path) as f:
            doc = json.load(f)
        for k, v in doc.items():
            if k not in _TOP_KEYS:
                raise KeyError(f"unknown key '{k}' in {path}")
            vals[k] = _coerce(k, v)
        json_options = vals.get("options")
    for k in ("model_dir", "draft_model_dir", "use_speculation", "tui", "tp_size", "host", "port", "api_key",
              "max_batch_size", "default_max_tokens", "model_name", "request_timeout_s"):
        v = getattr(args, k, None)
        if v is not None:
            vals[k] = v
    sets = list(args.set)
    if not any(s.startswith("tp=") for s in sets) and (args.tp_size is not None or "tp" not in (json_options or {})):
        sets.append(f"tp={vals['tp_size']}")
    opts = Options.resolve(json_options, sets, env)
    vals["tp_size"] = opts.tp
    vals["options"] = opts
    vals["video"] = vals["video"] or {}
    if vals["use_speculation"] and opts.speculator == "none":
        opts.values["speculator"] = "draft" if vals["draft_model_dir"] else "mtp"
    return LaunchConfig(**vals), args


def load_drafter(engine, draft_dir: str):
    """Block drafter from a checkpoint directory: ``config.json`` carries the geometry under ``dflash_config`` (block size,
    target layer ids, mask token) beside the usual decoder keys; tensors use the dense decoder names plus ``fc`` and
    ``hidden_norm``."""
    from ..models.factory import TensorSource
    from ..runtime.dflash_runner import DFlashConfig, DFlashRunner
    with open(os.path.join(draft_dir, "config.json")) as f:
        hf = json.load(f)
    if hf.get("model_type") == "deepseek_v41":
        # the DeepSeek-V4.1 drafter ("DSpark") is described by the trunk's own config keys; like the trunk, only the
        # synthetic form (random weights) is built
        from ..runtime.dspark_runner import DSparkConfig, DSparkRunner
        if "synthetic_weights" not in hf:
            raise NotImplementedError("deepseek_v41 drafter: loading checkpoint tensors is not built")
        return DSparkRunner(engine, DSparkConfig.from_hf(hf), seed=int(hf["synthetic_weights"]) + 100)
    d = hf.get("dflash_config", {})
    cfg = DFlashConfig(block_size=int(hf.get("block_size", d.get("block_size", 8))), n_layers=int(hf["num_hidden_layers"]),
                       hidden=int(hf["hidden_size"]), n_q=int(hf["num_attention_heads"]), n_kv=int(hf["num_key_value_heads"]),
                       head_dim=int(hf.get("head_dim", hf["hidden_size"] // hf["num_attention_heads"])),
                       ffn=int(hf["intermediate_size"]), target_layer_ids=tuple(d.get("target_layer_ids", hf.get("target_layer_ids", ()))),
                       sliding_window=int(hf.get("sliding_window") or 2048), rope_theta=float(hf.get("rope_theta", 1e7)),
                       rms_eps=float(hf.get("rms_norm_eps", 1e-6)), mask_token_id=int(d.get("mask_token_id", hf.get("mask_token_id", 0))),
                       version=int(d.get("version", hf.get("dflash_version", 1))),
                       conv_kernel_size=int(d.get("conv_kernel_size", 2)), conv_group_size=int(d.get("conv_group_size", 16)),
                       selector_rank=int(d.get("selector_rank", 256)), selector_top_k=int(d.get("selector_top_k", 16)))
    runner = DFlashRunner(engine, cfg)
    runner.load(TensorSource(draft_dir))
    return runner


def build_engine(cfg: LaunchConfig, device=None, comm=None, agree=None):
    """Model directory -> (model, hf_config, Engine, kv pool tokens) on this rank. ``agree(n)`` returns the value all
    ranks settle on for the KV pool size (minimum over ranks); ``None`` for a single rank."""
    import torch
    from ..models.factory import load_model
    from ..runtime.engine import Engine
    from ..runtime.kv_cache import PagedKVCache
    o = cfg.options
    device = device or ("cuda:0" if torch.cuda.is_available() else "cpu")
    overlay = {k: getattr(o, k) for k in ("nvfp4_experts", "nvfp4_expert_layers", "mtp_head_dir", "mtp_nvfp4", "nvfp4_dense_dir", "nvfp4_dense_src")
               if getattr(o, k)}
    model, hf = load_model(cfg.model_dir, device, comm, gemm_mode=o.gemm_mode, overlay=overlay or None, nvfp4_dense=o.nvfp4_dense)
    mcfg = model.cfg
    model.side_streams = bool(o.side_streams)
    if o.trace_layers:
        from ..utils.trace import enable_layer_trace
        enable_layer_trace(model)
    configure_expert_tier(model, o, getattr(comm, "rank", 0) if comm is not None else 0)
    configure_cpu_experts(model, o)
    from ..runtime.kv_cache import KV_FORMATS
    if o.kv_format not in KV_FORMATS:
        raise ValueError(f"kv_format '{o.kv_format}': this build has {sorted(KV_FORMATS)}")
    # bytes per cached element, scales included: bf16 2, E5M2 1, k8v4 (1 + 1/32 + 1/2 + 1/32) / 2, nvfp4 1/2 + 1/16
    kv_bytes = {"fp8": 1.0, "k8v4": 0.78125, "nvfp4": 0.5625}.get(o.kv_format, 2.0)
    bpt = int(getattr(model, "kv_layers", mcfg.n_layers) * model.nkv * 2 * mcfg.head_dim * kv_bytes)
    on_gpu = torch.device(device).type == "cuda"
    scratch_bytes = max(0, o.scratch_mib) << 20
    budget = None
    if on_gpu:
        free, _ = torch.cuda.mem_get_info(torch.device(device))
        # the arena holds the KV pools and the kernels' workspaces: arena_gib fixes its size, otherwise it takes what
        # is free after the weights minus the reserve (graphs, library workspaces, prefill activations)
        budget = (o.arena_gib << 30) if o.arena_gib > 0 else int((free - (o.vram_reserve_mib << 20)) * 0.9)
        budget = min(budget, free - (256 << 20))
    if o.kv_pool:
        pool_tokens = o.kv_pool
    elif on_gpu:
        pool_tokens = max(4096, (budget - scratch_bytes) // bpt)
    else:
        pool_tokens = min(o.max_seq * 2, 16384)
    pool_tokens = min(pool_tokens, o.max_seq * o.max_slots)
    if agree is not None:
        pool_tokens = agree(pool_tokens)
    kv_layers = getattr(model, "kv_layers", mcfg.n_layers)       # hybrid models keep KV only for their attention layers
    pages = max(2, pool_tokens // 64)
    arena = scratch = None
    if on_gpu:
        from ..ops import kernels as K
        from ..runtime.arena import Arena, ScratchRegistry
        arena = Arena(PagedKVCache.pool_bytes(kv_layers, model.nkv, mcfg.head_dim, pages, o.kv_format) + scratch_bytes
                      + (1 << 20), device)
        scratch = ScratchRegistry(arena, overflow=True)
        K.use_scratch(scratch, device)
    kv = PagedKVCache(kv_layers, model.nkv, mcfg.head_dim, pages, o.max_slots, o.max_seq, device,
                      dtype=o.kv_format, arena=arena)
    engine = Engine(model, kv, use_graphs=not o.no_graphs and torch.device(device).type == "cuda",
                    prefill_chunk=o.prefill_chunk)
    engine.arena, engine.scratch = arena, scratch
    if o.mem_log and on_gpu:
        free, total = torch.cuda.mem_get_info(torch.device(device))
        log.info("memory: device %.1f GiB used of %.1f; arena %.2f GiB (%s); KV pool %d tokens", (total - free) / 2**30,
                 total / 2**30, arena.capacity / 2**30,
                 ", ".join(f"{k} {v / 2**20:.0f} MiB" for k, v in arena.report()["by_name"].items()), pool_tokens)
    if hasattr(model, "set_prefill_truncate"):
        model.set_prefill_truncate(o.prefill_truncate)
    if o.hessian_dir and hasattr(model, "enable_hessians"):
        from ..ops.hessian import parse_layer_range
        model.enable_hessians(parse_layer_range(o.hessian_layers, mcfg.n_layers))
    if o.route_dump and hasattr(model, "heat"):
        from ..runtime.route_dump import RouteRecorder
        n_all = mcfg.n_layers + int(getattr(mcfg, "mtp_layers", 0) or 0)
        # route_dump_from: only the layers from this index on (n_layers = the MTP head's block only)
        model.route_recorder = RouteRecorder(layers=range(o.route_dump_from, n_all) if o.route_dump_from > 0 else None)
    apply_model_switches(model, o)
    return model, hf, engine, pool_tokens


def load_vision_frontend(model_dir: str, hf: dict, o, device):
    """The vision tower of a multimodal checkpoint -> ``MultimodalFrontend`` (or None for a text-only model or with
    ``max_image_tokens`` = 0). ``vision_dir`` names the directory that holds the tower (its ``config.json`` with
    ``vision_config``, ``preprocessor_config.json`` and ``model.visual.*`` tensors) when it is not the model directory;
    ``max_image_tokens`` caps an image's size in language-model tokens (it bounds the resize)."""
    vdir = o.vision_dir or model_dir
    vcfg = hf.get("vision_config")
    if o.vision_dir:
        with open(os.path.join(vdir, "config.json")) as f:
            vcfg = json.load(f).get("vision_config", vcfg)
    if not vcfg or int(o.max_image_tokens) <= 0:
        return None
    from ..loader.image import VisionParams
    from ..models.factory import TensorSource
    from ..models.vision import VisionConfig, VisionTower
    from ..runtime.multimodal import MultimodalFrontend
    cfg = VisionConfig.from_hf(vcfg)
    mm = getattr(o, "vision_mmproj", "") or ""
    if mm:
        # vision_mmproj: a directory holding a llama.cpp projector file (*mmproj*.gguf) to take the tower's weights from
        import glob
        from ..loader.gguf_file import GGUFFile
        files = sorted(glob.glob(os.path.join(mm, "*mmproj*.gguf"))) if os.path.isdir(mm) else [mm]
        if not files:
            raise FileNotFoundError(f"vision_mmproj: no *mmproj*.gguf in {mm}")
        tower = VisionTower(cfg, device).load_mmproj(GGUFFile(files[0]))
    else:
        src = TensorSource(vdir)
        if not src.has("model.visual.patch_embed.proj.weight"):
            log.warning("vision: %s has a vision_config but no model.visual.* tensors; image input stays off", vdir)
            return None
        tower = VisionTower(cfg, device).load(src)
    pre = {}
    for fn in ("preprocessor_config.json", "processor_config.json"):
        if os.path.exists(os.path.join(vdir, fn)):
            with open(os.path.join(vdir, fn)) as f:
                pre = json.load(f)
            pre = pre.get("image_processor", pre)
            break
    params = VisionParams.from_config(pre, vcfg)
    per_token = (params.patch_size * params.merge_size) ** 2           # pixels behind one language-model token
    params.max_pixels = min(params.max_pixels, int(o.max_image_tokens) * per_token)
    params.min_pixels = min(params.min_pixels, params.max_pixels)
    image_token = int(hf.get("image_token_id", hf.get("image_token_index", 151655)))
    log.info("vision tower: %d blocks of %d, images up to %d tokens", cfg.depth, cfg.hidden, o.max_image_tokens)
    return MultimodalFrontend(tower, params, image_token)


def apply_model_switches(model, o) -> None:
    """Launch options that turn parts of a loaded model off: ``expert_stats`` (routing histogram for the monitor),
    ``dsa`` / ``qsa_off`` (the sparse-attention indexers: without them every row attends densely)."""
    mcfg = model.cfg
    if not o.expert_stats and getattr(model, "heat", None) is not None and not getattr(model, "tiers", None):
        model.heat = None                 # (the expert tier needs the histogram and keeps it)
    if (not o.dsa or o.qsa_off) and hasattr(model, "layers"):
        blocks = list(model.layers) + ([model.mtp["layer"]] if getattr(model, "mtp", None) else [])
        for L in blocks:
            if not o.dsa and getattr(L, "dsa", None) is not None:
                L.dsa = None
            if o.qsa_off and getattr(L, "qsa", None) is not None:
                L.qsa = None
        if not o.dsa and hasattr(mcfg, "dsa"):
            mcfg.dsa = False
        if o.qsa_off and hasattr(mcfg, "qsa"):
            mcfg.qsa = False


def configure_cpu_experts(model, o):
    """``cpu_experts`` = f in (0, 1): that share of every layer's routed experts lives in host memory in its packed form
    and is computed by the host pool while the GPU runs the rest of the layer. ``cpu_expert_cpus`` ("0-7,16") pins the
    pool's workers, ``cpu_expert_node`` takes the CPU list of a NUMA node instead, ``cpu_expert_spin_us`` is how long an
    idle worker spins before it sleeps. Returns the service (None when off)."""
    share = float(getattr(o, "cpu_experts", 0.0) or 0.0)
    if share <= 0 or not hasattr(model, "layers") or not any(getattr(L, "bank", None) is not None for L in model.layers):
        return None
    if getattr(model, "tiers", None):
        raise ValueError("cpu_experts and expert_cache (the host-resident tier) cannot both own the same experts")
    from ..runtime.cpu_experts import CpuExpertService, attach_cpu_experts, numa_node_cpus, parse_cpu_list
    cpus = parse_cpu_list(o.cpu_expert_cpus) if o.cpu_expert_cpus else (numa_node_cpus(o.cpu_expert_node) if o.cpu_expert_node >= 0 else [])
    threads = len(cpus) if cpus else max(1, min(16, (os.cpu_count() or 2) // 2))
    svc = CpuExpertService(threads=threads, spin_us=int(o.cpu_expert_spin_us), cpus=cpus)
    attach_cpu_experts(model, min(share, 0.95), service=svc)
    model.cpu_expert_service = svc
    log.info("cpu experts: %.0f %% of every layer's experts on the host, %d worker threads%s", 100 * min(share, 0.95), threads,
             f" pinned to {cpus}" if cpus else "")
    return svc


def configure_expert_tier(model, o, rank: int = 0) -> None:
    """``expert_cache`` below 1 keeps that fraction of every layer's routed experts in device memory and the rest in pinned
    host memory (read in place); ``expert_adapt_every`` decode steps apart the residency follows the routing heat
    (``expert_swaps`` per layer, or as many as ``expert_swap_mib`` pays for; a cold expert replaces a resident one when
    its heat exceeds 1.5 x the resident one's plus ``expert_swap_margin``). ``expert_heat_file``: counts of an earlier
    run choose the first resident set and are saved again at shutdown."""
    model.expert_adapt_every = 0
    frac = float(o.expert_cache)
    if not (0.0 < frac < 1.0) or not hasattr(model, "enable_expert_tier") or getattr(model, "e_local", 0) < 2:
        return
    bank = next((L.bank for L in model.layers if getattr(L, "bank", None) is not None and hasattr(L.bank, "gu_p")), None)
    if bank is None:
        raise ValueError("expert_cache < 1 needs routed experts in the NVFP4 bank form")
    hot = max(1, int(model.e_local * frac))
    per_expert = bank.nbytes() // max(1, bank.e_local)
    tiers = model.enable_expert_tier(hot, margin=1.5, margin_add=float(o.expert_swap_margin),
                                     history_pct=int(o.expert_history_pct), resident_bias=float(o.route_resident_bias))
    swaps = int(o.expert_swaps)
    if swaps < 0:
        swaps = max(1, (int(o.expert_swap_mib) << 20) // max(1, 2 * per_expert * max(1, len(tiers))))
    model.expert_adapt_every, model.expert_max_swaps = max(0, int(o.expert_adapt_every)), swaps
    path = (o.expert_heat_file + (f".r{rank}" if rank else "")) if o.expert_heat_file else ""
    if path and os.path.exists(path):
        import torch
        heat = torch.load(path, map_location="cpu", weights_only=True)
        if tuple(heat.shape) == tuple(model.heat.shape):
            model.heat.copy_(heat)
            model.rebalance_experts(max_swaps=hot)            # start with the hottest experts resident
    stage = "off"
    if int(o.expert_stage) != 0:                                # -1 (auto) and 1: on when the scratch fits
        st = model.enable_expert_staging()
        stage = "off (scratch does not fit)" if st is None else f"{st.n_cold} cold experts x 2 buffers"
    log.info("expert tier: prefill staging %s", stage)
    log.info("expert tier: %d of %d experts per layer resident (%d layers, %.1f MiB per expert), rebalance every %d steps, "
             "%d swaps per layer", hot, model.e_local, len(tiers), per_expert / 2**20, model.expert_adapt_every, swaps)


def dump_calibration(model, options, rank: int = 0) -> list[str]:
    """Writes what the capture options collected (Hessian files per site, the route dump); called at shutdown."""
    out = []
    hs = getattr(model, "hess", None)
    drafter = getattr(model, "_drafter_for_report", None)
    if drafter is not None and hasattr(drafter, "profile_report") and drafter.profile_report():
        log.info("drafter rounds: %s", drafter.profile_report())
    if hs is not None and options.hessian_dir:
        out += hs.dump(options.hessian_dir, rank)
    dh = getattr(model, "_drafter_hessians", None)
    if dh is not None:
        out += dh[0].dump(dh[1], rank)
    if getattr(options, "expert_heat_file", "") and getattr(model, "tiers", None) and getattr(model, "heat", None) is not None:
        import torch
        path = options.expert_heat_file + (f".r{rank}" if rank else "")
        torch.save(model.heat.detach().cpu(), path)
        out.append(path)
    rec = getattr(model, "route_recorder", None)
    if rec is not None and options.route_dump:
        path = options.route_dump if rank == 0 else f"{options.route_dump}.r{rank}"
        rec.save(path)
        out.append(path)
    return out


def build_server(cfg: LaunchConfig, device=None, comm=None, chan=None, agree=None):
    """Model directory -> (VoltaServer, Generator, Engine) on this rank (rank 0 of a world, or the only rank)."""
    from ..loader.chat_template import ChatTemplate
    from ..loader.tokenizer import Tokenizer
    from ..runtime.generator import Generator
    from ..runtime.prefix_cache import PrefixCache
    from .app import VoltaServer

    o = cfg.options
    model, hf, engine, pool_tokens = build_engine(cfg, device, comm, agree)
    if chan is not None:
        from ..runtime.tp_control import LeaderEngine
        engine = LeaderEngine(engine, chan)
    tok = Tokenizer.load(cfg.model_dir)
    try:
        template = ChatTemplate.load(cfg.model_dir)
    except (FileNotFoundError, KeyError):
        template = None
    cache = None
    if o.prefix_cache_mib > 0 and getattr(model, "prefix_resume", None) in ("kv", "kv+state"):
        # a snapshot holds KV pages only: families with state outside the pool (recurrent / conv state, window and
        # compressor rings, indexer keys) run without the cache instead of resuming from a stale state
        from ..runtime.prefix_cache import model_fingerprint
        kvc = engine.kv
        fp = model_fingerprint(cfg.model_dir, kv_format=o.kv_format, tp=cfg.tp_size, layers=kvc.n_layers, kv_heads=kvc.n_kv,
                               head_dim=kvc.head_dim, v_head_dim=kvc.v_head_dim, model_type=getattr(model.cfg, "model_type", ""))
        cache = PrefixCache(o.prefix_cache_mib << 20, o.prefix_cache_dir or None, fingerprint=fp,
                            disk_budget_bytes=max(0, o.prefix_cache_disk_gib) << 30)
    gen = Generator(engine, tok, o, prefix_cache=cache)
    if getattr(model.cfg, "mrope_sections", ()) or hf.get("vision_config") or o.vision_dir:
        front = load_vision_frontend(cfg.model_dir, hf, o, engine.device)
        if front is not None:
            gen.mm_frontend = front              # the server accepts image parts from here on
    if o.steer != "off":
        from ..runtime.steering import SteerConfig
        if getattr(model.cfg, "residual", "plain") != "plain":
            raise ValueError("steer: the residual edit is built for the plain-residual decoder families")
        gen.steer_cfg = SteerConfig(o, model.cfg.n_layers, tok)
        model.steer = gen.steer_cfg.tables(model.cfg.hidden, o.max_slots, engine.device)
        from ..runtime.steer_probe import ProbeSettings
        gen.probe_cfg = ProbeSettings.from_options(o, model.cfg.n_layers, gen.steer_cfg.first, gen.steer_cfg.last)
        if o.probe:
            from ..runtime.steer_probe import load_probe_files
            gen.probe_files = load_probe_files(o.probe, o.steer_dir)
    if o.speculator == "draft" and cfg.draft_model_dir and cfg.tp_size > 1 and not o.draft_tp:
        log.warning("draft_tp = false: the vocabulary-sharded head needs every rank in a draft step, so the drafter stays off")
    if o.speculator == "draft" and cfg.draft_model_dir and (cfg.tp_size == 1 or o.draft_tp):
        if chan is not None:                       # tensor parallel: the followers hold their shard (see _run_rank)
            from ..runtime.tp_control import LeaderDrafter
            raw = load_drafter(engine._e, cfg.draft_model_dir)
            engine._e.drafter = raw
            gen.drafter = LeaderDrafter(raw, engine)
        else:
            gen.drafter = load_drafter(engine, cfg.draft_model_dir)
        if hasattr(gen.drafter.cfg, "conf_threshold"):
            gen.drafter.cfg.conf_threshold = o.dspark_conf
        if o.sparse_head and hasattr(gen.drafter, "enable_sparse_head"):
            from ..runtime.sparse_head_policy import SparseHeadParams
            pol = gen.drafter.enable_sparse_head(params=SparseHeadParams(interval=max(1, o.sparse_head_interval)),
                                                 state_path=o.sparse_head_state or None)
            pol.force = bool(o.sparse_head_force)
        if o.spec_profile and hasattr(gen.drafter, "enable_profile"):
            gen.drafter.enable_profile()
            model._drafter_for_report = gen.drafter            # dump_calibration logs the per-round averages at shutdown
        if o.dflash_hessian_dir and hasattr(gen.drafter, "model") and hasattr(gen.drafter.model, "enable_hessians"):
            # calibration capture of the drafter's own projections (every block counts: its rows are few)
            gen.drafter.model.enable_hessians(None, min_rows=1)
            model._drafter_hessians = (gen.drafter.model.hess, o.dflash_hessian_dir)
        if o.tap_spool and hasattr(gen.drafter, "ring"):
            from ..runtime.spec_logs import TapSpool, TargetSpool
            gen.tap_spool = TapSpool(o.tap_spool, o.tap_spool_window)
            gen.target_spool = TargetSpool()
            gen.target_spool.enable()
        if o.spec_cand_log:
            from ..runtime.spec_logs import CandLog
            gen.cand_log = CandLog()
            gen.cand_log.open(o.spec_cand_log)
    defaults = {"temperature": cfg.default_temperature, "top_p": cfg.default_top_p, "top_k": cfg.default_top_k,
                "enable_thinking": cfg.default_enable_thinking}
    gc_path = os.path.join(cfg.model_dir, "generation_config.json")
    if os.path.exists(gc_path):
        with open(gc_path) as f:
            gc = json.load(f)
        for k in ("temperature", "top_p", "top_k"):
            if k in gc:
                defaults[k] = gc[k]
    name = cfg.model_name or os.path.basename(os.path.normpath(cfg.model_dir))
    srv = VoltaServer(gen, tok, template, model_name=name, model_type=hf.get("model_type", "dense"), host=cfg.host,
                      port=cfg.port, api_key=cfg.api_key, defaults=defaults, max_context=o.max_seq,
                      default_max_tokens=cfg.default_max_tokens, request_timeout_s=cfg.request_timeout_s,
                      info={"tp": o.tp, "kv_tokens": pool_tokens, "options": dict(o.values)})
    return srv, gen, engine


def _run_rank(cfg: LaunchConfig) -> int:
    import datetime
    import torch
    import torch.distributed as dist
    from ..parallel import make_comm
    rank, world = int(os.environ["RANK"]), int(os.environ["WORLD_SIZE"])
    local = int(os.environ.get("LOCAL_RANK", rank))
    cuda = torch.cuda.is_available()
    device = f"cuda:{local}" if cuda else "cpu"
    if cuda:
        torch.cuda.set_device(local)
    dist.init_process_group("nccl" if cuda else "gloo", timeout=datetime.timedelta(seconds=600))
    ctl = dist.new_group(backend="gloo", timeout=datetime.timedelta(seconds=3600))
    from ..runtime.tp_control import ControlChannel, follower_loop
    if cuda:
        comm = make_comm(cfg.options.comm, device, chunk_rows=max(4096, int(cfg.options.prefill_chunk)))
        if hasattr(comm, "use_ll"):
            comm.use_ll = cfg.options.ar_ll
    else:
        from ..parallel.host import HostComm
        comm = HostComm()
    chan = ControlChannel(ctl)

    def agree(n: int) -> int:
        t = torch.tensor([n], dtype=torch.int64)
        dist.all_reduce(t, op=dist.ReduceOp.MIN, group=ctl)
        return int(t.item())
    if rank == 0:
        srv, gen, engine = build_server(cfg, device, comm, chan, agree)
        return _serve_forever(cfg, srv, engine)
    _, _, engine, _ = build_engine(cfg, device, comm, agree)
    o = cfg.options
    if o.speculator == "draft" and cfg.draft_model_dir and o.draft_tp:
        engine.drafter = load_drafter(engine, cfg.draft_model_dir)      # this rank's shard of the block drafter
    follower_loop(engine, chan)
    return 0


def _serve_forever(cfg: LaunchConfig, srv, engine) -> int:
    srv.start()
    print(f"volta_server: listening on http://{cfg.host}:{srv.port}  model={srv.model_name}  tp={cfg.tp_size}", flush=True)
    stop = threading.Event()
    for sig in (signal.SIGINT, signal.SIGTERM):
        try:
            signal.signal(sig, lambda *_: stop.set())
        except ValueError:
            pass
    if cfg.tui:
        from .tui import run_tui
        run_tui(f"http://{cfg.host}:{srv.port}", stop)
    stop.wait()
    srv.stop()
    dump_calibration(engine.model, cfg.options, getattr(engine.model.comm, "rank", 0))
    if hasattr(engine, "shutdown"):
        engine.shutdown()
    return 0


def is_video_model_dir(model_dir: str) -> bool:
    """A directory whose ``model_index.json`` names the MiniMaxH3Pipeline class selects the video service: no language-model
    runtime, a job queue with one worker that owns the GPU (reference: docs/video.md:88-92)."""
    path = os.path.join(model_dir, "model_index.json")
    if not os.path.exists(path):
        return False
    with open(path) as f:
        return json.load(f).get("_class_name") == "MiniMaxH3Pipeline"


def build_video_service(model_dir: str, out_dir: str | None = None, device=None, max_rows: int = 0, lora_dirs=(),
                        captioner: bool = False):
    """The video pipeline of a MiniMax-H3 directory. Built: the synthetic form (``"synthetic_weights": <seed>`` in
    ``model_index.json``, optional ``"shape": "tiny"``): every component with random weights at the published or the tiny
    shape; the tensor mapping of the published checkpoints is not."""
    import torch
    from ..video import dit as D
    from ..video.audio import AudioConfig
    from ..video.pipeline import H3Pipeline
    from ..video.service import VideoService
    from ..video.text import H3TextTower
    from ..video.vae import VaeConfig
    with open(os.path.join(model_dir, "model_index.json")) as f:
        idx = json.load(f)
    if "synthetic_weights" not in idx:
        raise NotImplementedError("minimax_h3: loading checkpoint tensors is not built (model_index.json with "
                                  "\"synthetic_weights\": <seed> runs the pipeline with random weights)")
    seed = int(idx["synthetic_weights"])
    dev = device or ("cuda:0" if torch.cuda.is_available() else "cpu")
    if idx.get("shape", "full") == "tiny":
        pipe = H3Pipeline.tiny(dev, seed, captioner=captioner)
    else:
        vae, aud, cfg = VaeConfig(), AudioConfig(), D.H3Config()
        tok = lambda s: [1 + (b % 150000) for b in s.encode()][:512] or [1]
        text = H3TextTower.qwen3_vl_32b(dev, captioner=captioner).init_random(seed + 7)
        pipe = H3Pipeline(D.H3DiT(cfg, dev).init_random(seed), text, vae, aud, tok, dev, seed)
        if captioner:
            pipe.attach_captioner(lambda ids: bytes(32 + (i % 90) for i in ids).decode(), eos_ids=(151645,))
    if lora_dirs:
        from ..video.lora import AdapterCatalog
        pipe.catalog = AdapterCatalog().scan(list(lora_dirs))
        log.info("video: %d adapter files in %s", len(pipe.catalog.all()), ", ".join(lora_dirs))
    return VideoService(pipe, out_dir or os.path.join(model_dir, "out"), max_rows=max_rows)


def _serve_video(cfg) -> int:
    import time
    from ..video.service import serve
    vopt = getattr(cfg, "video", None) or {}
    svc = build_video_service(cfg.model_dir, vopt.get("out_dir"), max_rows=int(vopt.get("max_rows", 0)),
                              lora_dirs=tuple(vopt.get("lora_dirs", ()) or ()), captioner=bool(vopt.get("captioner", False)))
    stop = []
    srv = serve(svc, cfg.host, cfg.port, stop=lambda: bool(stop))
    log.info("video service on http://%s:%d (jobs under %s)", cfg.host, srv.port, svc.out_dir)
    try:
        while True:
            time.sleep(1.0)
    except KeyboardInterrupt:
        pass
    stop.append(1)
    srv.stop()
    svc.stop()
    return 0


def main(argv: list[str] | None = None) -> int:
    argv = sys.argv[1:] if argv is None else argv
    cfg, args = resolve_config(argv)
    if args.print_config_docs:
        print(config_docs())
        return 0
    if args.print_config:
        print(json.dumps(cfg.to_dict(), indent=1))
        return 0
    if not cfg.model_dir:
        print("volta_server: model_dir is required (flag --model-dir or key model_dir)", file=sys.stderr)
        return 2
    if is_video_model_dir(cfg.model_dir):
        return _serve_video(cfg)
    if cfg.tp_size > 1:
        if "RANK" not in os.environ:
            cmd = [sys.executable, "-m", "torch.distributed.run", "--nnodes=1", f"--nproc-per-node={cfg.tp_size}",
                   "--master-addr", "127.0.0.1", "--master-port", str(29500 + os.getpid() % 2000),
                   "-m", "volta_engine_b200.server.cli"] + argv
            os.execv(sys.executable, cmd)
        return _run_rank(cfg)
    srv, gen, engine = build_server(cfg)
    return _serve_forever(cfg, srv, engine)


if __name__ == "__main__":
    sys.exit(main())
