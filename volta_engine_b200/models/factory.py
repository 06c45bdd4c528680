"""Model directory -> running model. ``config.json``'s ``model_type`` alone decides the model family; weights come
from sharded safetensors (dense / NVFP4 / EXL3 / FP8-block) or from a GGUF file in the same directory.

Reference: src/models/model.cpp:82 (``create_model_pipeline`` switch on model_type), src/server/config.cpp (model
directory contract), src/loader/gguf_arch.h:21-66 (GGUF adapters).
"""
from __future__ import annotations

import json
from pathlib import Path

import torch

from ..loader.gguf_file import GGUFFile, _NORM_PLUS_ONE, _ROPE_PERMUTED, name_index, unpermute_rope_rows, _PLAIN
from ..loader.safetensors import SafeTensorsRepo, write_safetensors
from ..ops.linear import LinearBF16, fuse_linears
from ..ops.linear_gguf import LinearGGUF
from ..quant import gguf as gq
from .dense import DenseConfig, DenseLayer, DenseModel

DENSE_TYPES = {"llama", "mistral", "qwen2", "qwen3", "gemma2", "gemma3_text", "glm4", "dense"}
MOE_TYPES = {"qwen3_moe", "glm4_moe", "mixtral", "moe"}
MLA_TYPES = {"deepseek_v2", "deepseek_v3", "kimi_k2", "mla"}


def dense_config_from_hf(c: dict) -> DenseConfig:
    mt = c.get("model_type", "dense")
    hd = c.get("head_dim") or c["hidden_size"] // c["num_attention_heads"]
    gemma = mt.startswith("gemma")
    return DenseConfig(
        n_layers=c["num_hidden_layers"], hidden=c["hidden_size"], n_q=c["num_attention_heads"],
        n_kv=c.get("num_key_value_heads", c["num_attention_heads"]), head_dim=hd, ffn=c["intermediate_size"],
        vocab=c["vocab_size"], rope_theta=float(c.get("rope_theta", 10000.0)), rms_eps=float(c.get("rms_norm_eps", 1e-6)),
        norm_bias=1.0 if gemma else 0.0, rot_dim=int(hd * c.get("partial_rotary_factor", 1.0)) if c.get("partial_rotary_factor") else 0,
        qk_norm=mt in ("qwen3", "qwen3_moe", "gemma3_text"), act="gelu_tanh" if gemma else "silu",
        tie_embeddings=bool(c.get("tie_word_embeddings", False)),
        embed_scale=float(c["hidden_size"]) ** 0.5 if gemma else 1.0,
        sliding_window=int(c.get("sliding_window") or 0) if c.get("use_sliding_window", mt == "mistral" or gemma) else 0,
        attn_scale=float(c["query_pre_attn_scalar"]) ** -0.5 if c.get("query_pre_attn_scalar") else 0.0,
        logit_softcap=float(c.get("final_logit_softcapping") or 0.0), quant=c.get("volta_quant", "bf16"),
        window_pattern=int(c.get("sliding_window_pattern") or (2 if mt == "gemma2" else 0)) if gemma else 0,
        rope_theta_local=float(c.get("rope_local_base_freq") or 0.0), sandwich_norm=gemma, model_type=mt)


class TensorSource:
    """Checkpoint-name view over a safetensors repository or a GGUF file."""

    def __init__(self, model_dir, prefer: str | None = None):
        d = Path(model_dir)
        ggufs = [p for p in d.glob("*.gguf") if "mmproj" not in p.name.lower()]
        sts = list(d.glob("*.safetensors"))
        self.gguf = self.repo = None
        if ggufs and (prefer == "gguf" or not sts):
            self.gguf = GGUFFile(d)
            self.names = name_index(self.gguf)
            self.arch = self.gguf.arch
        elif sts:
            self.repo = SafeTensorsRepo(d)
        else:
            raise FileNotFoundError(f"{d}: neither *.safetensors nor *.gguf found")

    def has(self, name: str) -> bool:
        return name in self.names if self.gguf else self.repo.has(name)

    def tensor(self, name: str, device=None, dtype=None) -> torch.Tensor:
        if self.gguf:
            t = self.gguf.dequantize(self.names[name])
            if name.endswith("norm.weight") and self.arch in _NORM_PLUS_ONE:
                t = t - 1.0
        else:
            t = self.repo.load(name)
        if dtype is not None:
            t = t.to(dtype)
        return t.to(device) if device is not None else t

    def linear(self, base: str, split=None, rank=0, world=1, device=None, gemm_mode="w4a16", quantize=None,
               rope_heads: int = 0):
        """``rope_heads``: number of heads of a q/k projection (needed to undo the GGUF rope row permutation)."""
        if self.repo:
            return self.repo.load_linear(base, split, rank, world, device, gemm_mode, quantize)
        g = self.gguf
        info = g.tensors[self.names[base + ".weight"]]
        N, K = info.shape
        permuted = rope_heads and self.arch in _ROPE_PERMUTED
        if info.ggml_type in _PLAIN or permuted and split == "row":
            w = g.dequantize(info.name)
            if permuted:
                w = unpermute_rope_rows(w, rope_heads)
            n0, n1 = SafeTensorsRepo._range(N, "col" if split == "col" else None, rank, world, 1)
            k0, k1 = SafeTensorsRepo._range(K, "row" if split == "row" else None, rank, world, 1)
            w = w[n0:n1, k0:k1].to(torch.bfloat16).contiguous()
            return LinearBF16(w.to(device) if device is not None else w)
        raw = g.load(info.name)                                        # [N, row_bytes]
        if permuted:
            raw = unpermute_rope_rows(raw, rope_heads)
        n0, n1 = SafeTensorsRepo._range(N, "col" if split == "col" else None, rank, world, 1)
        blk = gq.BLOCK[info.ggml_type][0]
        k0, k1 = SafeTensorsRepo._range(K, "row" if split == "row" else None, rank, world, blk)
        bpb = gq.row_bytes(info.ggml_type, blk)
        raw = raw[n0:n1, k0 // blk * bpb:k1 // blk * bpb].contiguous()
        if device is not None:
            raw = raw.to(device)
        return LinearGGUF(raw, info.ggml_type, n1 - n0, k1 - k0)


class OverlaySource:
    """A tensor source assembled from several checkpoints: names that match a rule come from that rule's source, every
    other name from the primary one. Rules are (predicate(name) -> bool, TensorSource), first match wins. This is how
    the launch options that take parts of a model from other directories work (``nvfp4_experts``: routed experts from an
    NVFP4 checkpoint; ``mtp_head_dir``: the MTP head from another checkpoint; ``nvfp4_dense_dir``: calibrated dense
    tensors). Reference: docs/CONFIG.md:72-80 (the reference's loader options of the same names)."""

    def __init__(self, primary: TensorSource, rules: list):
        self.primary, self.rules = primary, list(rules)

    def source_for(self, name: str) -> TensorSource:
        for pred, src in self.rules:
            if pred(name) and (src.has(name) or src.has(name + ".weight") or src.has(name + ".weight_packed")
                               or any(src.has(name + s) for s in ("gate_proj.weight", "gate_proj.weight_packed", "0.gate_proj.weight",
                                                                  "0.gate_proj.weight_packed"))):
                return src
        return self.primary

    def has(self, name: str) -> bool:
        return self.source_for(name).has(name)

    def tensor(self, name: str, device=None, dtype=None):
        return self.source_for(name).tensor(name, device, dtype)

    def linear(self, base: str, *a, **k):
        return self.source_for(base).linear(base, *a, **k)

    def __getattr__(self, name):                   # gguf / repo / names / arch of the primary checkpoint
        return getattr(self.primary, name)


def parse_layer_set(text: str, n_layers: int) -> set:
    """"3-10,12" -> {3..10, 12}; empty -> every layer."""
    if not text:
        return set(range(n_layers + 8))
    out = set()
    for part in (p.strip() for p in text.split(",") if p.strip()):
        a, _, b = part.partition("-")
        out |= set(range(int(a), int(b or a) + 1))
    return out


def overlay_from_options(primary: TensorSource, hf: dict, nvfp4_experts: str = "", nvfp4_expert_layers: str = "",
                         mtp_head_dir: str = "", mtp_nvfp4: bool = False, nvfp4_dense_dir: str = "", nvfp4_dense_src: str = ""):
    """The tensor source the loader options describe (the primary source itself when none of them is set)."""
    import re as _re
    n_layers = int(hf.get("num_hidden_layers", 0))
    layer_of = _re.compile(r"model\.layers\.(\d+)\.")
    rules = []

    def layer(name):
        m = layer_of.match(name)
        return int(m.group(1)) if m else -1
    if mtp_head_dir:
        mtp_src = TensorSource(mtp_head_dir)
        rules.append((lambda n: layer(n) >= n_layers, mtp_src))
    if nvfp4_experts:
        ex_src = TensorSource(nvfp4_experts)
        layers = parse_layer_set(nvfp4_expert_layers, n_layers)
        rules.append((lambda n: ".mlp.experts." in n and layer(n) in layers and layer(n) < n_layers, ex_src))
        if mtp_nvfp4 and not mtp_head_dir:
            rules.append((lambda n: layer(n) >= n_layers, ex_src))
    if nvfp4_dense_dir:
        rules.append((lambda n: ".mlp.experts." not in n, TensorSource(nvfp4_dense_dir)))
    if nvfp4_dense_src:                            # bf16 dense tensors of another checkpoint, quantised at load like the model's own
        rules.append((lambda n: ".mlp.experts." not in n and "embed_tokens" not in n, TensorSource(nvfp4_dense_src)))
    return OverlaySource(primary, rules) if rules else primary


def load_dense_weights(model: DenseModel, src: TensorSource, gemm_mode="w4a16", quantize=None) -> DenseModel:
    """Fill a DenseModel from a checkpoint with the usual decoder names (``model.layers.N.self_attn.q_proj`` ...);
    this rank keeps its tensor-parallel shard (q/k/v/gate/up column-split, o/down row-split, vocabulary rows)."""
    cfg, dev = model.cfg, model.device
    r, tp = model.comm.rank, model.comm.size
    kw = dict(rank=r, world=tp, device=dev, gemm_mode=gemm_mode, quantize=quantize)
    bf = torch.bfloat16
    model.embed = src.tensor("model.embed_tokens.weight", dev, bf)
    model.layers = []
    for li in range(cfg.n_layers):
        p = f"model.layers.{li}."
        L = DenseLayer()
        q = src.linear(p + "self_attn.q_proj", "col", rope_heads=cfg.n_q, **kw)
        if cfg.n_kv >= tp:
            k = src.linear(p + "self_attn.k_proj", "col", rope_heads=cfg.n_kv, **kw)
            v = src.linear(p + "self_attn.v_proj", "col", **kw)
        else:                                       # fewer kv heads than ranks: ranks share heads
            kwr = dict(kw, rank=r // model.kv_rep, world=cfg.n_kv)
            k = src.linear(p + "self_attn.k_proj", "col", rope_heads=cfg.n_kv, **kwr)
            v = src.linear(p + "self_attn.v_proj", "col", **kwr)
        L.qkv = fuse_linears([q, k, v])
        L.o_proj = src.linear(p + "self_attn.o_proj", "row", **kw)
        L.gate_up = fuse_linears([src.linear(p + "mlp.gate_proj", "col", **kw), src.linear(p + "mlp.up_proj", "col", **kw)])
        if hasattr(L.gate_up, "interleave_gated"):
            L.gate_up.interleave_gated()
        L.down = src.linear(p + "mlp.down_proj", "row", **kw)
        L.attn_norm = src.tensor(p + "input_layernorm.weight", dev, bf)
        L.post_attn_norm = L.post_ffn_norm = None
        if cfg.sandwich_norm:      # pre / post norms around both blocks
            L.post_attn_norm = src.tensor(p + "post_attention_layernorm.weight", dev, bf)
            L.ffn_norm = src.tensor(p + "pre_feedforward_layernorm.weight", dev, bf)
            L.post_ffn_norm = src.tensor(p + "post_feedforward_layernorm.weight", dev, bf)
        else:
            L.ffn_norm = src.tensor(p + "post_attention_layernorm.weight", dev, bf)
        L.q_norm = L.k_norm = None
        if cfg.qk_norm:
            L.q_norm = src.tensor(p + "self_attn.q_norm.weight", dev, bf)
            L.k_norm = src.tensor(p + "self_attn.k_norm.weight", dev, bf)
        model.layers.append(L)
    model.final_norm = src.tensor("model.norm.weight", dev, bf)
    head_name = "model.embed_tokens.weight" if cfg.tie_embeddings or not src.has("lm_head.weight") else "lm_head.weight"
    full = src.tensor(head_name, None, bf)
    head = torch.zeros(model.vocab_local, cfg.hidden, dtype=bf)
    lo = r * model.vocab_local
    hi = min(cfg.vocab, lo + model.vocab_local)
    if hi > lo:
        head[: hi - lo] = full[lo:hi]
    model.lm_head = LinearBF16(head.to(dev))
    return model


def load_model(model_dir, device="cuda:0", comm=None, gemm_mode="w4a16", quantize=None, prefer=None, overlay: dict | None = None,
               nvfp4_dense: str = ""):
    """-> (model, hf_config dict). Raises for model types this build has no pipeline for. ``overlay``: keyword arguments of
    :func:`overlay_from_options` (parts of the model taken from other directories); ``nvfp4_dense``: comma list of dense
    groups quantised to NVFP4 at load beyond the default (``head``, or ``all``)."""
    d = Path(model_dir)
    hf = json.loads((d / "config.json").read_text())
    if "text_config" in hf and "num_hidden_layers" not in hf:
        hf = dict(hf["text_config"], **{k: v for k, v in hf.items() if k != "text_config"})
    mt = hf.get("model_type", "")
    if mt == "deepseek_v41":
        return load_dsv41(hf, d, device, comm), hf
    if mt in ("glm5_next", "glm5-next"):
        groups = {g.strip() for g in nvfp4_dense.split(",") if g.strip()}
        return load_glm5(hf, d, device, comm, gemm_mode, quantize, nvfp4_head=bool(groups & {"head", "all"})), hf
    src = TensorSource(d, prefer)
    if mt in ("qwen3_5", "qwen3_5_text", "qwen3_5_moe", "qwen3_next", "qwen4_exp"):
        from .hybrid_loader import load_hybrid
        groups = {g.strip() for g in nvfp4_dense.split(",") if g.strip()}
        if overlay:
            src = overlay_from_options(src, hf, **overlay)
        return load_hybrid(hf, src, device, comm, gemm_mode, quantize, nvfp4_head=bool(groups & {"head", "all"})), hf
    if mt in DENSE_TYPES:
        cfg = dense_config_from_hf(hf)
        cfg.gemm_mode = gemm_mode
        model = DenseModel(cfg, device, comm)
        return load_dense_weights(model, src, gemm_mode, quantize), hf
    if mt in MOE_TYPES or mt in MLA_TYPES:
        from .moe_loader import load_moe_family
        if overlay:
            src = overlay_from_options(src, hf, **overlay)
        groups = {g.strip() for g in nvfp4_dense.split(",") if g.strip()}
        return load_moe_family(hf, src, device, comm, gemm_mode, quantize, nvfp4_head=bool(groups & {"head", "all"})), hf
    raise NotImplementedError(f"model_type {mt!r} has no pipeline in this build")


def dsv4_config_from_hf(c: dict):
    """DeepSeek-V4.1 ``config.json`` (the official inference configuration's names) -> DSV4Config.
    Reference: src/models/deepseek_v41.cpp:439-489 (``read_config``: the same keys, the implemented layout checked)."""
    from .dsv4 import DSV4Config
    n = int(c.get("n_layers", c.get("num_hidden_layers", 40)))
    ratios = tuple(c.get("compress_ratios", ()))[:n] or (0,) * n
    return DSV4Config(
        n_layers=n, hidden=int(c.get("dim", c.get("hidden_size", 5120))), n_q=int(c.get("n_heads", 64)), n_kv=1,
        head_dim=int(c.get("head_dim", 512)), ffn=0, vocab=int(c.get("vocab_size", 129280)),
        n_experts=int(c.get("n_routed_experts", 384)), top_k=int(c.get("n_activated_experts", 6)),
        expert_ffn=int(c.get("moe_inter_dim", 2304)), shared_ffn=int(c.get("moe_inter_dim", 2304)) * int(c.get("n_shared_experts", 1)),
        router=c.get("score_func", "sqrtsoftplus"), router_scale=float(c.get("route_scale", 1.5)),
        act_limit=float(c.get("swiglu_limit", 10.0)), rms_eps=float(c.get("norm_eps", 1e-20)),
        rope_theta=float(c.get("rope_theta", 10000.0)), hc_sinkhorn=int(c.get("hc_sinkhorn_iters", 20)),
        hc_eps=float(c.get("hc_eps", 1e-6)), q_lora_rank=int(c.get("q_lora_rank", 1280)), o_groups=int(c.get("o_groups", 8)),
        o_lora_rank=int(c.get("o_lora_rank", 1024)), compress_ratios=ratios,
        kv_sources=tuple(c.get("kv_source_layers", ())), index_sources=tuple(c.get("index_source_layers", ())),
        candidate_source=int(c.get("candidate_source_layer", -1)), candidate_blocks=int(c.get("candidate_topk_blocks", 2048)),
        candidate_block=int(c.get("candidate_block_size", 8)), compress_rope_theta=float(c.get("compress_rope_theta", 160000.0)),
        rope_original_len=int(c.get("original_seq_len", 65536)), rope_factor=float(c.get("rope_factor", 16.0)),
        beta_fast=float(c.get("beta_fast", 32.0)), beta_slow=float(c.get("beta_slow", 1.0)),
        engram_layers=tuple(c.get("engram_layer_ids", ())), engram_dim=int(c.get("engram_n_heads", 8)) * int(c.get("engram_head_dim", 256)),
        engram_rows=int(c.get("engram_table_rows", 1 << 16)), engram_ngram=int(c.get("engram_max_ngram_size", 4)))


def glm5_config_from_hf(c: dict):
    """GLM-5-Next ``config.json`` -> Glm5NextConfig. Keys as the reference reads them (src/models/glm5_next.cpp:499-552;
    defaults are the published shape, inc/engine/models/glm5_next.h:33-52)."""
    from .glm5 import Glm5NextConfig
    base = Glm5NextConfig.glm5_next()
    n = int(c.get("num_hidden_layers", base.n_layers))
    n_mla = int(c.get("num_mla_layers", 0)) or sum(1 for li in range(n) if (li + 1) % base.full_interval == 0)
    base.n_layers, base.hidden = n, int(c.get("hidden_size", base.hidden))
    base.full_interval = max(1, n // max(1, n_mla))
    base.n_q = int(c.get("num_attention_heads", base.n_q))
    base.ffn = int(c.get("dense_intermediate_size", c.get("intermediate_size_dense", base.ffn)))
    base.expert_ffn = int(c.get("moe_intermediate_size", c.get("intermediate_size", base.expert_ffn)))
    base.shared_ffn = base.expert_ffn * int(c.get("n_shared_experts", 1))
    base.n_experts, base.top_k = int(c.get("n_routed_experts", c.get("num_experts", base.n_experts))), int(c.get("num_experts_per_tok", base.top_k))
    base.first_dense_layers = int(c.get("first_k_dense_replace", base.first_dense_layers))
    base.router_scale = float(c.get("routed_scaling_factor", base.router_scale))
    base.vocab = int(c.get("vocab_size", base.vocab))
    base.q_lora_rank = int(c.get("q_lora_rank", base.q_lora_rank))
    base.qk_nope, base.v_head_dim = int(c.get("qk_nope_head_dim", base.qk_nope)), int(c.get("v_head_dim", base.v_head_dim))
    base.gdn_k_heads = base.gdn_v_heads = int(c.get("kda_heads", c.get("linear_num_heads", base.gdn_k_heads)))
    base.gdn_dk = base.gdn_dv = int(c.get("kda_head_dim", c.get("linear_head_dim", base.gdn_dk)))
    base.kda_rank = int(c.get("kda_rank", base.kda_rank))
    base.rms_eps = float(c.get("rms_norm_eps", base.rms_eps))
    base.rope_theta = float(c.get("rope_theta", base.rope_theta))
    base.mtp_layers = int(c.get("num_nextn_predict_layers", base.mtp_layers))
    base.dsa = bool(c.get("dsa", c.get("index_topk", 1)))
    base.residual = "hc" if int(c.get("hc_mult", 4)) > 1 else "plain"
    return base


def load_glm5(hf: dict, model_dir: Path, device, comm, gemm_mode="w4a16", quantize=None, nvfp4_head: bool = False):
    """A GLM-5-Next directory: the published checkpoint's tensors (:mod:`.glm5_loader`), or, with ``"synthetic_weights":
    <seed>`` in ``config.json`` and no tensor files, the architecture (KDA mixers, latent attention with the indexer,
    experts, hyper-connection streams, MTP head) with random weights."""
    from .glm5 import Glm5NextModel
    if "synthetic_weights" not in hf:
        from .glm5_loader import load_glm5_checkpoint
        return load_glm5_checkpoint(hf, TensorSource(model_dir), device, comm, gemm_mode, quantize, nvfp4_head)
    cfg = glm5_config_from_hf(hf)
    cfg.expert_quant = hf.get("expert_quant", "nvfp4_random")
    model = Glm5NextModel(cfg, device, comm).init_random(seed=int(hf["synthetic_weights"]))
    if cfg.residual != "plain":
        model.init_stream_weights()
    return model


def load_dsv41(hf: dict, model_dir: Path, device, comm):
    """A DeepSeek-V4.1 directory. Only the synthetic form is built: ``config.json`` with ``"synthetic_weights": <seed>``
    and no tensor files gives the architecture with random weights (benchmarks, tests); the tensor-name mapping of the
    published FP8 / FP4 checkpoint is not."""
    from .dsv4 import DSV4Model
    cfg = dsv4_config_from_hf(hf)
    if "synthetic_weights" not in hf:
        raise NotImplementedError("deepseek_v41: loading checkpoint tensors is not built (config.json with "
                                  "\"synthetic_weights\": <seed> runs the architecture with random weights)")
    return DSV4Model(cfg, device, comm).init_random(seed=int(hf["synthetic_weights"]))


def save_dense_checkpoint(model_dir, cfg: DenseConfig, seed: int = 0, std: float = 0.02, fmt: str = "bf16",
                          shards: int = 2, model_type: str = "qwen3"):
    """Write a random-weight model directory (config.json + sharded safetensors) in format ``fmt``:
    bf16 | nvfp4 (compressed-tensors names) | nvfp4_modelopt | exl3. For tests and synthetic benchmarks."""
    from ..quant import exl3 as ex, nvfp4 as qn
    d = Path(model_dir)
    d.mkdir(parents=True, exist_ok=True)
    g = torch.Generator().manual_seed(seed)
    hf = {"model_type": model_type, "num_hidden_layers": cfg.n_layers, "hidden_size": cfg.hidden,
          "num_attention_heads": cfg.n_q, "num_key_value_heads": cfg.n_kv, "head_dim": cfg.head_dim,
          "intermediate_size": cfg.ffn, "vocab_size": cfg.vocab, "rope_theta": cfg.rope_theta,
          "rms_norm_eps": cfg.rms_eps, "tie_word_embeddings": cfg.tie_embeddings}
    (d / "config.json").write_text(json.dumps(hf, indent=1))
    tensors, u16 = {}, []

    def put_linear(base, n, k):
        w = torch.randn(n, k, generator=g) * std
        if fmt == "bf16":
            tensors[base + ".weight"] = w.to(torch.bfloat16)
        elif fmt in ("nvfp4", "nvfp4_modelopt"):
            p, s, gs = qn.quantize_nvfp4(w, search=False)
            if fmt == "nvfp4":
                tensors[base + ".weight_packed"] = p
                tensors[base + ".weight_scale"] = s.view(torch.float8_e4m3fn)
                tensors[base + ".weight_global_scale"] = torch.tensor([1.0 / gs])
            else:
                tensors[base + ".weight"] = p
                tensors[base + ".weight_scale"] = s.view(torch.float8_e4m3fn)
                tensors[base + ".weight_scale_2"] = torch.tensor([gs])
        elif fmt == "exl3":
            codes, suh, svh = ex.synth_linear(k, n, 4, std, g)
            tensors[base + ".trellis"], tensors[base + ".suh"], tensors[base + ".svh"] = codes, suh, svh
            tensors[base + ".mul1"] = torch.zeros(1, dtype=torch.int32)
            u16.append(base + ".trellis")
        else:
            raise ValueError(fmt)

    H, hd = cfg.hidden, cfg.head_dim
    tensors["model.embed_tokens.weight"] = (torch.randn(cfg.vocab, H, generator=g) * std).to(torch.bfloat16)
    for li in range(cfg.n_layers):
        p = f"model.layers.{li}."
        put_linear(p + "self_attn.q_proj", cfg.n_q * hd, H)
        put_linear(p + "self_attn.k_proj", cfg.n_kv * hd, H)
        put_linear(p + "self_attn.v_proj", cfg.n_kv * hd, H)
        put_linear(p + "self_attn.o_proj", H, cfg.n_q * hd)
        put_linear(p + "mlp.gate_proj", cfg.ffn, H)
        put_linear(p + "mlp.up_proj", cfg.ffn, H)
        put_linear(p + "mlp.down_proj", H, cfg.ffn)
        tensors[p + "input_layernorm.weight"] = torch.ones(H, dtype=torch.bfloat16)
        tensors[p + "post_attention_layernorm.weight"] = torch.ones(H, dtype=torch.bfloat16)
        if model_type == "qwen3":
            tensors[p + "self_attn.q_norm.weight"] = torch.ones(hd, dtype=torch.bfloat16)
            tensors[p + "self_attn.k_norm.weight"] = torch.ones(hd, dtype=torch.bfloat16)
    tensors["model.norm.weight"] = torch.ones(H, dtype=torch.bfloat16)
    if not cfg.tie_embeddings:
        tensors["lm_head.weight"] = (torch.randn(cfg.vocab, H, generator=g) * std).to(torch.bfloat16)
    names = sorted(tensors)
    per = (len(names) + shards - 1) // shards
    for si in range(shards):
        part = {n: tensors[n] for n in names[si * per:(si + 1) * per]}
        if part:
            write_safetensors(d / f"model-{si + 1:05d}-of-{shards:05d}.safetensors", part, unsigned16=tuple(u16))
    return hf
