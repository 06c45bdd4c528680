"""Runtime options: one table -> defaults, ``ENGINE_*`` environment, ``--set key=value``, JSON ``options``
block, and generated documentation.

Mirrors the reference's single X-macro option table (inc/engine/runtime/options.def,
src/runtime/options.cpp, docs/CONFIG.md:54-203). Precedence: CLI ``--set`` > JSON launch file > environment
> default. Unknown keys are fatal.
"""
from __future__ import annotations

import os
from dataclasses import dataclass

# name, type, default, help
_TABLE = [
    ("tp", int, 1, "tensor-parallel ranks (1, 2, 4, 8)"),
    ("max_seq", int, 32768, "maximum tokens per sequence (paged; up to 262144)"),
    ("max_slots", int, 8, "concurrent sequences"),
    ("kv_pool", int, 0, "KV pool size in tokens (0 = size from free memory)"),
    ("kv_format", str, "bf16", "KV cache element format: bf16 | fp8 | k8v4 | nvfp4"),
    ("vram_reserve_mib", int, 2048, "device memory left unallocated"),
    ("prefill_chunk", int, 2048, "rows per prefill forward"),
    ("prefill_budget_ms", float, 50.0, "prefill time slice between decode steps when sequences are decoding"),
    ("prefix_cache_mib", int, 4096, "host memory for sequence snapshots (0 disables the prefix cache)"),
    ("prefix_cache_dir", str, "", "directory of the disk tier of the prefix cache"),
    ("prefix_interval", int, 16384, "automatic snapshot every N prompt tokens"),
    ("speculator", str, "none", "none | mtp | suffix | draft"),
    ("spec_depth", int, 3, "maximum draft tokens per round"),
    ("spec_ctrl", bool, True, "throughput controller chooses between speculative rounds and plain steps"),
    ("spec_suffix_min", int, 2, "shortest k-gram the suffix drafter matches"),
    ("gemm_mode", str, "w4a16", "prefill arithmetic for NVFP4 weights: w4a16 | w4a4"),
    ("comm", str, "symm", "tensor-parallel collectives: symm (own NVLink kernels) | nccl"),
    ("nvls", bool, True, "use NVSwitch multimem reductions when available"),
    ("no_graphs", bool, False, "disable CUDA-graph replay of decode steps"),
    ("loop_detect", bool, True, "finish requests whose output degenerates into a loop"),
    ("thinking_budget", int, 0, "soft cap of reasoning tokens (0 = unlimited)"),
    ("expert_parallel", bool, True, "shard MoE experts over ranks (else slice every expert)"),
    ("moe_heavy_rows", int, 64, "rows per expert above which the grouped GEMM path is used"),
    ("log_level", str, "info", "error | warn | info | debug"),
    ("dump_requests", str, "", "directory that receives one JSON file per request"),
    ("trace_layers", bool, False, "NVTX range per layer"),
    ("prefill_truncate", int, -1, "rows of a prompt's tail that the layers past a ratio-1 KV source run (-1 exact, 0 off; models that allow it)"),
    ("dspark_conf", float, 0.5, "confidence below which the DSpark block drafter cuts its drafts"),
    ("sparse_head", bool, False, "block drafter: draft through a learned subset of the head's columns when it pays"),
    ("sparse_head_state", str, "", "file that keeps the sparse head's token counts between runs"),
    ("spec_cand_log", str, "", "file that receives the block drafter's candidates per round (offline re-ranker training)"),
    ("hessian_dir", str, "", "calibration capture: x^T x of every projection input over the prefill rows, written here at shutdown"),
    ("hessian_layers", str, "", "lo-hi: capture these layers only (a slice that fits beside the weights)"),
    ("route_dump", str, "", "file that receives the MoE blocks' routed rows and routing weights at shutdown"),
]

_TYPES = {n: t for n, t, _, _ in _TABLE}


def _parse(name: str, raw):
    t = _TYPES[name]
    if t is bool:
        if isinstance(raw, bool):
            return raw
        return str(raw).strip().lower() in ("1", "true", "yes", "on")
    return t(raw)


@dataclass
class Options:
    values: dict

    def __getattr__(self, k):
        try:
            return self.__dict__["values"][k]
        except KeyError:
            raise AttributeError(k)

    @classmethod
    def resolve(cls, json_options: dict | None = None, cli_sets: list[str] | None = None, env=None) -> "Options":
        env = os.environ if env is None else env
        v = {n: d for n, _, d, _ in _TABLE}
        for n in v:
            raw = env.get("ENGINE_" + n.upper())
            if raw is not None:
                v[n] = _parse(n, raw)
        for k, raw in (json_options or {}).items():
            if k not in v:
                raise KeyError(f"unknown option '{k}'")
            v[k] = _parse(k, raw)
        for item in cli_sets or []:
            if "=" not in item:
                raise ValueError(f"--set expects key=value, got '{item}'")
            k, raw = item.split("=", 1)
            if k not in v:
                raise KeyError(f"unknown option '{k}'")
            v[k] = _parse(k, raw)
        if v["tp"] not in (1, 2, 4, 8):
            raise ValueError("tp must be 1, 2, 4 or 8")
        return cls(v)


def config_docs() -> str:
    """Markdown table of every option (the generated part of the configuration reference)."""
    lines = ["| option | type | default | env | meaning |", "|---|---|---|---|---|"]
    for n, t, d, h in _TABLE:
        lines.append(f"| `{n}` | {t.__name__} | `{d}` | `ENGINE_{n.upper()}` | {h} |")
    return "\n".join(lines) + "\n"
