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
    ("spec_tree", int, 0, "suffix speculator: > 1 verifies up to this many different continuations of the current suffix "
                          "as one token tree (tree attention mask, one forward; greedy requests on the dense GQA family)"),
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

# Keys of the reference's option table (inc/engine/runtime/options.def) that this engine takes under the same name, so a
# launch file written for the reference loads unchanged. Each entry says what the key does here: "-> name" = an alias of
# one of the options above (the value is converted), "live" = read by the engine under its own name, anything else = why
# the key has no effect on this engine (it is still parsed and type-checked; an unknown key stays fatal).
_NOOP_KERNEL = "no effect: selects between kernel variants of the reference's sm_70 / sm_80 build; here each op has one sm_100a kernel"
_NOOP_DEBUG = "no effect: debugging aid of a reference code path that has no counterpart here"
_COMPAT = [
    # name, type, default, disposition
    ("arena_gib", int, -1, "live"), ("scratch_mib", int, 256, "live"),
    ("prefix_cache_gib", int, 16, "-> prefix_cache_mib"), ("prefix_cache_disk_gib", int, 64, "live"),
    ("prefill_window", int, -1, "no effect: expert weights of a layer stay resident in HBM, so a prompt's chunks need not be "
                                 "regrouped layer by layer to amortise expert staging"),
    ("prefill_cooldown", int, 0, "live"), ("prefix_cache_reply", bool, True, "live"),
    ("nvfp4_experts", str, "", "live"), ("nvfp4_dense", str, "", "live"), ("nvfp4_dense_dir", str, "", "live"),
    ("nvfp4_dense_src", str, "", "live"), ("nvfp4_expert_layers", str, "", "live"),
    ("embed_host", bool, True, "no effect: the embedding table stays in HBM (180 GB per GPU); a host copy would add a PCIe "
                               "read to every step"),
    ("mtp_nvfp4", bool, False, "live"), ("mtp_head_dir", str, "", "live"), ("dflash_hessian_dir", str, "", "live"),
    ("sparse_head_interval", int, 2048, "live"), ("sparse_head_file", str, "", "-> sparse_head_state"),
    ("expert_cache", float, 1.0, "live"), ("expert_stage", int, -1, "live"), ("expert_adapt_every", int, 64, "live"),
    ("route_resident_bias", float, 0.0, "live"), ("expert_swap_margin", int, 2, "live"),
    ("expert_history_pct", int, 75, "live"), ("expert_swaps", int, -1, "live"), ("expert_swap_mib", int, 1024, "live"),
    ("expert_shard", int, -1, "-> expert_parallel"), ("expert_heat_file", str, "", "live"),
    ("cpu_experts", float, 0.0, "live"), ("cpu_expert_cpus", str, "", "live"), ("cpu_expert_node", int, -1, "live"),
    ("cpu_expert_spin_us", int, 2000, "live"),
    ("steer", str, "off", "live"), ("steer_layers", str, "", "live"), ("steer_file", str, "", "live"),
    ("steer_dir", str, "", "live"), ("probe", str, "", "live"), ("low_priority_models", str, "haiku", "live"),
    ("steer_scale", float, 1.0, "live"), ("steer_scope", str, "", "live"), ("steer_gate_threshold", str, "auto", "live"),
    ("steer_edit_strength", str, "auto", "live"), ("steer_hedge_strength", float, -1.0, "live"),
    ("steer_openings", str, "", "live"), ("steer_directions", int, 1, "live"), ("steer_keep_norm", bool, False, "live"),
    ("steer_push", float, 0.0, "live"), ("steer_band", str, "", "live"), ("steer_edit_layers", str, "", "live"),
    ("thinking_soft_close", int, 128, "live"), ("think_penalty", float, 0.0, "live"),
    ("think_penalty_words", str, "", "live"),
    ("exl3_gemv_max_m", int, 4, _NOOP_KERNEL), ("exl3_wmma_max_m", int, 64, _NOOP_KERNEL),
    ("glm_layers", int, 0, _NOOP_DEBUG), ("gemv_max_rows", int, 16, _NOOP_KERNEL), ("gemv_int8", bool, True, _NOOP_KERNEL),
    ("gguf_mma", bool, True, _NOOP_KERNEL), ("gguf_gemv_warp", int, -1, _NOOP_KERNEL),
    ("ar_ll", bool, True, "live"), ("dflash_attn_scalar", bool, False, _NOOP_KERNEL), ("spec_profile", bool, False, "live"),
    ("merge_expert_groups", bool, True, _NOOP_KERNEL), ("fp8_resident", bool, True, _NOOP_KERNEL),
    ("indexer_tc", bool, True, _NOOP_KERNEL),
    ("mtp_depth", int, 7, "live"), ("draft_tp", bool, True, "live"), ("dsa", bool, True, "live"),
    ("vision_cpu", int, 0, "no effect: the vision tower always runs on rank 0's GPU"), ("vision_cpus", str, "", "no effect: see vision_cpu"),
    ("vision_mmproj", str, "", "live"), ("vision_dir", str, "", "live"), ("max_image_tokens", int, 1024, "live"),
    ("expert_stats", bool, True, "live"), ("spec_block_cycle", str, "", _NOOP_DEBUG), ("spec_depth_rate", bool, False, "live"),
    ("spec_suffix", int, 0, "live"),
    ("moe_coop_mode", int, -1, _NOOP_KERNEL), ("moe_prefill_tile", bool, True, _NOOP_KERNEL), ("gguf_q8r", bool, True, _NOOP_KERNEL),
    ("gguf_moe_tile", bool, True, _NOOP_KERNEL), ("gguf_moe_tile884", bool, True, _NOOP_KERNEL),
    ("shared_slice", bool, True, _NOOP_KERNEL), ("moe_gemv", bool, False, _NOOP_KERNEL),
    ("nvfp4_hipblas", bool, False, "no effect: ROCm build switch"), ("ple_log", bool, False, "live"),
    ("expert_log", bool, False, "live"), ("glm_logit_rows", int, 0, _NOOP_DEBUG), ("expert_stream", bool, False, _NOOP_KERNEL),
    ("expert_synth", int, 0, _NOOP_DEBUG), ("dsa_diag", bool, False, _NOOP_DEBUG), ("sparse_head_force", bool, False, "live"),
    ("train_inputs", str, "", _NOOP_DEBUG), ("route_dump_from", int, 0, "live"), ("route_replay", str, "", _NOOP_DEBUG),
    ("gr_fuse", bool, True, _NOOP_KERNEL), ("mem_log", bool, False, "live"), ("side_streams", bool, True, "live"),
    ("kda_rows", bool, True, _NOOP_KERNEL), ("hc_rows", bool, True, _NOOP_KERNEL), ("hc_fuse", bool, True, _NOOP_KERNEL),
    ("normed_add_fuse", bool, True, _NOOP_KERNEL), ("dflash_graph", bool, True, "no effect: drafter rounds always replay as graphs"),
    ("mtp_chain", bool, True, "no effect: the draft chain always runs on the device"), ("mtp_graph", bool, True, "-> no_graphs"),
    ("qsa_off", bool, False, "live"), ("router_fp16", bool, False, _NOOP_KERNEL), ("spec_ctrl_log", bool, False, "live"),
    ("draft_per_slot", bool, True, "live"), ("spec_agg_dense", int, -1, _NOOP_DEBUG), ("tap_spool", str, "", "live"),
    ("tap_spool_window", int, 768, "live"), ("spec_joint_max", int, 2, "live"), ("spec_joint", int, -1, "live"),
    ("spec_interleave", bool, True, "live"), ("dflash_tap_shift", int, 0, _NOOP_DEBUG),
    ("dflash_embed_scale", bool, True, _NOOP_DEBUG), ("dflash_sliding_causal", bool, True, _NOOP_DEBUG),
    ("dump_draft_round", int, -1, _NOOP_DEBUG),
]
# keys both tables know under the same name but whose reference form is wider than ours: converted when parsed
_WIDE = {
    "loop_detect": lambda raw: (str(raw).strip().lower() in ("1", "true", "yes", "on", "stop", "report")) if not isinstance(raw, bool) else raw,
    "sparse_head": lambda raw: (int(raw) > 0 if str(raw).strip().lstrip("-").isdigit() else str(raw).strip().lower() in ("true", "yes", "on")) if not isinstance(raw, bool) else raw,
    "trace_layers": lambda raw: (str(raw).strip().lower() not in ("", "0", "false", "no", "off")) if not isinstance(raw, bool) else raw,
    "kv_format": lambda raw: {"": "bf16", "fp16": "bf16"}.get(str(raw), str(raw)),
    "tp": lambda raw: 1 if int(raw) < 0 else int(raw),
    "speculator": lambda raw: {"dflash": "draft", "dflash2": "draft", "dspark": "draft"}.get(str(raw), str(raw)),
    "spec_depth": lambda raw: max(0, int(float(raw))),
    "max_seq": lambda raw: int(raw) if int(raw) > 0 else 32768,
    "max_slots": lambda raw: int(raw) if int(raw) > 0 else 8,
    "vram_reserve_mib": lambda raw: int(raw) if int(raw) >= 0 else 2048,
    "moe_heavy_rows": lambda raw: int(raw) if int(raw) > 0 else 64,
}

_NOT_WIRED = {}
_COMPAT_HELP = {'expert_stage': 'with expert_cache < 1, prompt pieces above 16 rows: copy a layer\'s cold experts once into device scratch, a layer ahead of the compute, instead of reading them over PCIe for every route (two buffers of one layer\'s cold experts; off when they do not fit). -1 and 1: on; 0: off', 'nvfp4_dense_src': 'directory of another checkpoint of the model whose bf16 dense tensors (everything but the routed experts and the embedding) replace the model directory\u2019s and are quantised at load', 'vision_mmproj': 'a llama.cpp vision projector file (or a directory holding a *mmproj*.gguf) the tower takes its weights from instead of the model.visual.* tensors (config.json and preprocessor_config.json still come from vision_dir or model_dir)', 'probe': 'with steer: comma list of probe files in steer_dir (at most 4) scored on every request; the usage reports each file\u2019s score at the last prompt token', 'spec_interleave': 'no effect: several decoding slots take joint MTP rounds (spec_joint: every slot in one verify forward) or plain batched steps; one-slot-per-step interleaving is not offered', 'ple_log': 'no effect: the n-gram embedding lookup of this build runs on the device inside the forward; there is no host lookup to time', 'steer_gate_threshold': 'requests with steer_probe: the look-ahead score (0 = like the accepting openings, 1 = like the declining ones) above which the clamps are installed; auto = 0.5', 'steer_edit_strength': 'requests with steer_probe: the reference level of a clamp sits this many standard deviations (of the projections of the accepting openings) below their mean projection; auto = 1', 'steer_hedge_strength': 'requests with steer_probe: a second clamp on the plain -> hedged axis at this fraction of the gap above the plain mean; < 0 = off', 'steer_openings': 'requests with steer_probe: file that replaces the built-in forced openings (lines accept: / decline: / plain: / hedged: TEXT)', 'steer_directions': 'requests with steer_probe: directions clamped per edit layer (1 to 4: the mean difference of the openings, then the strongest remaining variations of the declining openings)', 'steer_keep_norm': 'requests with steer_probe: a row a clamp edited is rescaled to the norm it had before', 'steer_push': 'requests with steer_probe: add the declining direction to the edit layers, this many times the gap between the accepting and the declining openings, whether or not the gate fires; negative pushes towards accepting', 'steer_band': 'requests with steer_probe: layers the probe reads (first-last as steer_layers); empty = 1/3-2/3', 'steer_edit_layers': 'requests with steer_probe: layers the clamps edit inside the band; empty = the band', 'nvfp4_experts': 'directory of an NVFP4 checkpoint of the same model whose routed experts replace those of model_dir (MoE / MLA families)', 'nvfp4_expert_layers': 'layers ("3-10,12") whose experts come from nvfp4_experts; empty = all', 'mtp_head_dir': 'directory of a checkpoint the MTP head (the block past the last layer and its connectors) is taken from', 'mtp_nvfp4': 'take the MTP head from the nvfp4_experts checkpoint', 'nvfp4_dense_dir': 'directory of calibrated NVFP4 dense tensors used instead of the model directory\'s for the names it holds', 'nvfp4_dense': 'dense groups quantised to NVFP4 at load beyond the default (the MoE / MLA loaders quantise every dense projection already): head, or all', 'draft_tp': 'true: the block drafter runs tensor parallel on every rank (its calls are mirrored to the followers); false with tp > 1: the drafter stays off (the sharded head needs every rank)', 'vision_dir': 'directory that holds the vision tower (config.json with vision_config, preprocessor_config.json, model.visual.* tensors) when it is not model_dir', 'max_image_tokens': 'largest image the vision tower accepts, in language-model tokens (caps the resize); 0 = image input off', 'spec_depth_rate': 'block drafter: choose each round\'s draft depth for the most expected tokens per millisecond (per-position accuracy against a fitted fixed + per-row round time); replaces spec_depth while on', 'dflash_hessian_dir': 'directory that receives, at shutdown, the input Hessians of the block drafter\'s projections (the same per-site files as hessian_dir)', 'tap_spool': 'with a block drafter: file that receives, when a request finishes, its tokens, the drafter taps of its last tap_spool_window positions and the target\'s top-16 candidates at the positions speculation emitted (record layout in runtime/spec_logs.py)', 'tap_spool_window': 'positions of a finished request whose taps are written to tap_spool', 'draft_per_slot': 'true is how this engine always runs: every slot keeps its own drafter context and tap ring; false (one shared context) is not offered', 'route_resident_bias': 'with expert_cache < 1: added to the router\'s selection score of experts resident in device memory (the weights stay the raw scores); follows the residency after every rebalance', 'expert_history_pct': 'largest share (percent) of an expert swap decision taken from the long-run route counts (kept between runs with expert_heat_file) instead of the recent windows; grows with the amount of history', 'cpu_experts': 'share (0..1) of every layer\'s routed experts kept packed in host memory and computed by the host pool (native NVFP4 kernels) beside the GPU', 'cpu_expert_cpus': 'CPU list ("0-7,16") the host pool\'s workers are pinned to', 'cpu_expert_node': 'NUMA node whose CPUs the host pool takes when cpu_expert_cpus is empty', 'cpu_expert_spin_us': 'how long an idle host worker spins on the work counter before it sleeps', 'sparse_head_interval': 'generated tokens between rebuilds of the sparse drafter head', 'sparse_head_force': 'draft through the subset whenever one exists, whatever the miss rate (A/B)', 'route_dump_from': 'route_dump records only the layers from this index on (n_layers = the MTP block only)', 'dsa': 'false: the latent-attention layers drop their indexer and attend densely', 'qsa_off': 'true: the hybrid attention layers drop their block-sparse indexer and attend densely', 'expert_stats': 'false: no routing histogram is kept for the monitor (a model with an expert tier keeps it)', 'spec_profile': 'time the stages of every drafter round (ingest, backbone, head and walk) and log the averages at shutdown', 'thinking_soft_close': 'once a reasoning budget runs out the block closes after the next token that ends a sentence or a line, at most this many tokens later; 0 closes at the budget', 'expert_log': 'log the swaps of every expert rebalance', 'spec_ctrl_log': 'log the speculation controller\'s mode changes', 'arena_gib': 'size of the per-GPU arena in GiB; <= 0 sizes it from free memory minus vram_reserve_mib', 'scratch_mib': 'arena memory set aside for kernel workspaces before the model loads', 'prefix_cache_gib': 'prefix cache budget in GiB (alias of prefix_cache_mib)', 'prefix_cache_disk_gib': "size limit of the prefix cache's disk tier; the least recently used files go first", 'prefill_cooldown': 'decode steps that run between two prompt pieces while other requests decode', 'prefix_cache_reply': 'snapshot prompt + reply when a request ends', 'ar_ll': 'false: decode rows use the two-shot collective instead of the one-shot LL all-reduce (A/B)', 'mtp_depth': 'draft depth of the MTP speculator (alias of spec_depth when speculator=mtp)', 'spec_suffix': '> 0 turns the suffix drafter on when no speculator is named', 'mem_log': 'log device memory after start-up', 'side_streams': 'independent chains of a layer (shared expert beside the routed experts) run on a side stream', 'low_priority_models': 'comma list of model-name substrings whose requests queue behind the others', 'sparse_head_file': 'alias of sparse_head_state', 'expert_shard': '0 / 1: whole experts per rank / a slice of every expert per rank (alias of expert_parallel)', 'mtp_graph': 'false: alias of no_graphs'}
_COMPAT = [(n, t, d, ("parsed, not wired in this build: " + _NOT_WIRED[n]) if n in _NOT_WIRED else disp) for n, t, d, disp in _COMPAT]

_TYPES = {n: t for n, t, _, _ in _TABLE}
_TYPES.update({n: t for n, t, _, _ in _COMPAT})
_DISPOSITION = {n: d for n, _, _, d in _COMPAT}


def known_keys() -> set:
    """Every option name the launcher accepts."""
    return set(_TYPES)


def disposition(name: str) -> str:
    """What a reference option key does in this engine (see ``_COMPAT``); "native" for the engine's own options."""
    return _DISPOSITION.get(name, "native")


def _parse(name: str, raw):
    if name in _WIDE:
        return _WIDE[name](raw)
    t = _TYPES[name]
    if t is bool:
        if isinstance(raw, bool):
            return raw
        return str(raw).strip().lower() in ("1", "true", "yes", "on")
    if t is float and isinstance(raw, str) and raw.strip().lower() == "auto":
        return -1.0                     # "auto" of a numeric option (expert_cache): let the engine size it
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
        v.update({n: d for n, _, d, _ in _COMPAT})
        given = set()
        for n in list(v):
            raw = env.get("ENGINE_" + n.upper(), env.get("ENGINE_DEBUG_" + n.upper()))
            if raw is not None:
                v[n] = _parse(n, raw)
                given.add(n)
        for k, raw in (json_options or {}).items():
            if k not in v:
                raise KeyError(f"unknown option '{k}'")
            v[k] = _parse(k, raw)
            given.add(k)
        for item in cli_sets or []:
            if "=" not in item:
                raise ValueError(f"--set expects key=value, got '{item}'")
            k, raw = item.split("=", 1)
            if k not in v:
                raise KeyError(f"unknown option '{k}'")
            v[k] = _parse(k, raw)
            given.add(k)
        # aliases of the reference's names
        if "prefix_cache_gib" in given and "prefix_cache_mib" not in given:
            v["prefix_cache_mib"] = max(0, int(v["prefix_cache_gib"])) * 1024
        if "sparse_head_file" in given and "sparse_head_state" not in given:
            v["sparse_head_state"] = v["sparse_head_file"]
        if "expert_shard" in given and "expert_parallel" not in given and int(v["expert_shard"]) >= 0:
            v["expert_parallel"] = int(v["expert_shard"]) == 0
        if "mtp_graph" in given and "no_graphs" not in given and not v["mtp_graph"]:
            v["no_graphs"] = True
        if "mtp_depth" in given and "spec_depth" not in given and v["speculator"] == "mtp":
            v["spec_depth"] = int(v["mtp_depth"])
        if v["speculator"] == "none" and int(v["spec_suffix"]) > 0:
            v["speculator"] = "suffix"
        if v["tp"] not in (1, 2, 4, 8):
            raise ValueError("tp must be 1, 2, 4 or 8")
        o = cls(v)
        o.__dict__["given"] = given
        return o

    def ignored(self) -> list[tuple[str, str]]:
        """Keys the launch set explicitly that have no effect here, with the reason (the launcher logs them once)."""
        return [(k, _DISPOSITION[k]) for k in sorted(self.__dict__.get("given", ()))
                if _DISPOSITION.get(k, "").startswith(("no effect", "parsed, not wired"))]


def config_docs() -> str:
    """Markdown table of every option (the generated part of the configuration reference)."""
    lines = ["| option | type | default | env | meaning |", "|---|---|---|---|---|"]
    for n, t, d, h in _TABLE:
        lines.append(f"| `{n}` | {t.__name__} | `{d}` | `ENGINE_{n.upper()}` | {h} |")
    lines += ["", "Keys of the reference engine's option table accepted under the same name:", "",
              "| option | type | default | in this engine |", "|---|---|---|---|"]
    for n, t, d, disp in _COMPAT:
        lines.append(f"| `{n}` | {t.__name__} | `{d}` | {_COMPAT_HELP.get(n, disp)} |")
    return "\n".join(lines) + "\n"
