"""Checkpoint -> MoE / MLA-MoE model: router, stacked NVFP4 expert bank (expert parallel: whole experts per rank),
shared expert, leading dense layers, GQA or latent attention, optional MTP block.

Expert weights arrive either already NVFP4 (per-expert ``...experts.E.gate_proj.weight_packed`` and friends) or as
dense / FP8-block tensors that are quantised at load; gate and up are stacked into one [2I, H] operand, which for
NVFP4 sources needs a common tensor scale (re-quantised when the checkpoint's two scales differ).
Reference: src/models/model.cpp:82 (factory), inc/engine/loader/safetensors.h:208-223 (NVFP4 expert loading),
src/models/*moe*.cpp (weight names per family).
"""
from __future__ import annotations

import torch

from ..ops.linear import LinearBF16, LinearNVFP4, fuse_linears
from ..quant import nvfp4 as qn
from .factory import TensorSource, dense_config_from_hf
from .mla import LAT, ROPE, MLAConfig, MLAModel
from .moe import ExpertBank, MoEConfig, MoEModel


def moe_config_from_hf(c: dict):
    d = dense_config_from_hf(c)
    mt = c.get("model_type", "moe")
    base = {k: getattr(d, k) for k in d.__dataclass_fields__}
    base.update(
        n_experts=c.get("num_experts") or c.get("n_routed_experts") or c.get("num_local_experts"),
        top_k=c.get("num_experts_per_tok", 2), expert_ffn=c.get("moe_intermediate_size", c["intermediate_size"]),
        shared_ffn=(c.get("shared_expert_intermediate_size") or
                    c.get("n_shared_experts", 0) * c.get("moe_intermediate_size", 0) or 0),
        router="sigmoid" if c.get("scoring_func") == "sigmoid" else "softmax",
        router_scale=float(c.get("routed_scaling_factor", 1.0)), n_group=c.get("n_group") or 1,
        topk_group=c.get("topk_group") or 1, first_dense_layers=c.get("first_k_dense_replace", 0), model_type=mt)
    if "kv_lora_rank" in c:
        base.update(q_lora_rank=c["q_lora_rank"], kv_lora_rank=c["kv_lora_rank"], qk_nope=c["qk_nope_head_dim"],
                    qk_rope=c["qk_rope_head_dim"], v_head_dim=c["v_head_dim"], n_kv=1,
                    head_dim=c["kv_lora_rank"] + c["qk_rope_head_dim"], mtp_layers=c.get("num_nextn_predict_layers", 0))
        return MLAConfig(**base)
    return MoEConfig(**base)


def _nvfp4_of(src: TensorSource, base: str):
    """-> (packed, scales, gscale) of linear ``base``, quantising dense sources."""
    lin = src.linear(base, quantize="nvfp4")
    if isinstance(lin, LinearNVFP4):
        return lin.packed, lin.scales, lin.gscale
    w = lin.weight.float() if isinstance(lin, LinearBF16) else lin.dequant().float()
    return qn.quantize_nvfp4(w, search=True)


def _load_bank_gguf(src: TensorSource, prefix: str, cfg, e0: int, e_local: int, dev):
    """GGUF files stack the experts of a layer in three tensors ([experts, rows, cols]: ``ffn_gate_exps``, ``ffn_up_exps``,
    ``ffn_down_exps``). When gate and up share a block type the blocks are kept as they are (``GGUFExpertBank``: fused
    dequant mat-vec, slab dequantise + grouped GEMM); ``None`` when the file has no stacked experts or mixes types that
    cannot be stacked (the caller then goes through the per-expert path).
    Reference: src/loader/gguf_arch.h:21-66 (expert tensors of the GGUF adapters), src/kernels/cuda/gguf/gguf_moe.cu."""
    g = src.gguf
    if g is None:
        return None
    names = {k: src.names.get(f"{prefix}experts.{k}_proj.weight") for k in ("gate", "up", "down")}
    if not all(names.values()):
        return None
    from ..loader.gguf_file import _PLAIN
    from ..ops.linear_gguf import FUSED_TYPES
    from ..ops.moe_gguf import GGUFExpertBank
    info = {k: g.tensors[n] for k, n in names.items()}
    gt, dt = info["gate"].ggml_type, info["down"].ggml_type
    if gt != info["up"].ggml_type or gt in _PLAIN or dt in _PLAIN or gt not in FUSED_TYPES or dt not in FUSED_TYPES:
        return None
    E, I, H = cfg.n_experts, cfg.expert_ffn, cfg.hidden
    gate = g.load(names["gate"]).reshape(E, I, -1)[e0:e0 + e_local]
    up = g.load(names["up"]).reshape(E, I, -1)[e0:e0 + e_local]
    down = g.load(names["down"]).reshape(E, H, -1)[e0:e0 + e_local]
    return GGUFExpertBank(torch.cat([gate, up], 1).to(dev), gt, down.contiguous().to(dev), dt, e0, I, H)


def _load_bank(src: TensorSource, prefix: str, cfg, e0: int, e_local: int, dev) -> ExpertBank:
    if hasattr(src, "source_for"):                 # an overlay: this layer's experts may live in another checkpoint
        src = src.source_for(prefix + "experts.")
    bank = _load_bank_gguf(src, prefix, cfg, e0, e_local, dev)
    if bank is not None:
        return bank
    gp, gs, gg, dp, ds, dg = [], [], [], [], [], []
    for e in range(e0, e0 + e_local):
        p = f"{prefix}experts.{e}."
        g_p, g_s, g_g = _nvfp4_of(src, p + "gate_proj")
        u_p, u_s, u_g = _nvfp4_of(src, p + "up_proj")
        if g_g != u_g:                    # one tensor scale per stacked operand
            w = torch.cat([qn.dequantize_nvfp4(g_p, g_s, g_g), qn.dequantize_nvfp4(u_p, u_s, u_g)], 0)
            f_p, f_s, f_g = qn.quantize_nvfp4(w, search=True)
        else:
            f_p, f_s, f_g = torch.cat([g_p, u_p], 0), torch.cat([g_s, u_s], 0), g_g
        gp.append(f_p), gs.append(f_s), gg.append(f_g)
        d_p, d_s, d_g = _nvfp4_of(src, p + "down_proj")
        dp.append(d_p), ds.append(d_s), dg.append(d_g)
    st = lambda xs: torch.stack(xs).to(dev)
    return ExpertBank(st(gp), st(gs), torch.tensor(gg, dtype=torch.float32, device=dev), st(dp), st(ds),
                      torch.tensor(dg, dtype=torch.float32, device=dev), e0, cfg.expert_ffn, cfg.hidden)


def _load_ffn(model, src, L, p, li, kw):
    cfg, dev = model.cfg, model.device
    r, tp = model.comm.rank, model.comm.size
    L.gate_up = L.down = None
    L.dense_ffn = li < cfg.first_dense_layers or not src.has(p + "mlp.gate.weight")
    if L.dense_ffn:
        L.gate_up = fuse_linears([src.linear(p + "mlp.gate_proj", "col", **kw), src.linear(p + "mlp.up_proj", "col", **kw)])
        L.down = src.linear(p + "mlp.down_proj", "row", **kw)
        return
    rw = src.tensor(p + "mlp.gate.weight", dev, torch.bfloat16)
    L.shared_gated = src.has(p + "mlp.shared_expert_gate.weight")
    if L.shared_gated:                      # the gate's logit rides as one more router row
        rw = torch.cat([rw, src.tensor(p + "mlp.shared_expert_gate.weight", dev, torch.bfloat16).reshape(1, -1)], 0)
    L.router = LinearBF16(rw.contiguous())
    L.router_bias = None
    if src.has(p + "mlp.gate.e_score_correction_bias"):
        L.router_bias = src.tensor(p + "mlp.gate.e_score_correction_bias", dev, torch.float32)
    L.bank = _load_bank(src, p + "mlp.", cfg, model.e0, model.e_local, dev)
    L.shared_gu = L.shared_dn = None
    if cfg.shared_ffn:
        sp = p + ("mlp.shared_expert." if src.has(p + "mlp.shared_expert.gate_proj.weight") or
                  src.repo and src.repo.linear_kind(p + "mlp.shared_expert.gate_proj") else "mlp.shared_experts.")
        S = cfg.shared_ffn
        sliced = S % tp == 0 and (S // tp) % 16 == 0 and tp > 1
        model._shared_sliced = sliced
        skw = kw if sliced else dict(kw, rank=0, world=1)
        L.shared_gu = fuse_linears([src.linear(sp + "gate_proj", "col", **skw), src.linear(sp + "up_proj", "col", **skw)])
        L.shared_dn = src.linear(sp + "down_proj", "row", **skw)


def _load_gqa(model, src, L, p, kw):
    cfg = model.cfg
    r, tp = model.comm.rank, model.comm.size
    q = src.linear(p + "self_attn.q_proj", "col", **kw)
    kwr = kw if cfg.n_kv >= tp else dict(kw, rank=r // model.kv_rep, world=cfg.n_kv)
    L.qkv = fuse_linears([q, src.linear(p + "self_attn.k_proj", "col", **kwr), src.linear(p + "self_attn.v_proj", "col", **kwr)])
    L.o_proj = src.linear(p + "self_attn.o_proj", "row", **kw)
    L.q_norm = L.k_norm = None
    if cfg.qk_norm:
        L.q_norm = src.tensor(p + "self_attn.q_norm.weight", model.device, torch.bfloat16)
        L.k_norm = src.tensor(p + "self_attn.k_norm.weight", model.device, torch.bfloat16)


def _load_mla(model, src, L, p, kw):
    cfg, dev = model.cfg, model.device
    r, hl = model.comm.rank, model.heads
    bf = torch.bfloat16
    # q_a and kv_a share the input: one stacked operand, rows padded to the kernel's granularity
    qa = src.repo.load_dense_weight(p + "self_attn.q_a_proj") if src.repo else src.tensor(p + "self_attn.q_a_proj.weight")
    kva = (src.repo.load_dense_weight(p + "self_attn.kv_a_proj_with_mqa") if src.repo
           else src.tensor(p + "self_attn.kv_a_proj_with_mqa.weight"))
    wa = torch.zeros(model.a_rows, cfg.hidden)
    wa[: cfg.q_lora_rank] = qa.float()
    wa[cfg.q_lora_rank: cfg.q_lora_rank + LAT + ROPE] = kva.float()
    L.qkv_a = model._make_linear(wa.to(dev), True)
    L.q_a_norm = src.tensor(p + "self_attn.q_a_layernorm.weight", dev, bf)
    L.kv_a_norm = src.tensor(p + "self_attn.kv_a_layernorm.weight", dev, bf)
    L.q_b = src.linear(p + "self_attn.q_b_proj", "col", **kw)
    wkvb = (src.repo.load_dense_weight(p + "self_attn.kv_b_proj") if src.repo
            else src.tensor(p + "self_attn.kv_b_proj.weight")).float()
    mine = wkvb.reshape(cfg.n_q, cfg.qk_nope + cfg.v_head_dim, LAT)[r * hl:(r + 1) * hl].to(dev)
    L.w_uk = mine[:, : cfg.qk_nope].contiguous().to(bf)
    L.w_uv = mine[:, cfg.qk_nope:].contiguous().to(bf)
    L.w_ukv = LinearBF16(mine.reshape(hl * (cfg.qk_nope + cfg.v_head_dim), LAT).to(bf))
    L.o_proj = src.linear(p + "self_attn.o_proj", "row", **kw)
    L.qkv = None
    L.q_norm = L.k_norm = None


def load_head(model, src, embed_name: str, nvfp4_head: bool = False, gemm_mode: str | None = None) -> None:
    """This rank's vocabulary shard of the output head (``lm_head.weight``, or the embedding when they are tied), padded
    with zero rows to the shard size; NVFP4 when asked for and the shapes allow it (a quarter of the bytes a decode step
    streams for it)."""
    cfg, dev, bf = model.cfg, model.device, torch.bfloat16
    head_name = "lm_head.weight" if src.has("lm_head.weight") and not cfg.tie_embeddings else embed_name
    full = src.tensor(head_name, None, bf)
    head = torch.zeros(model.vocab_local, cfg.hidden, dtype=bf)
    lo = model.comm.rank * model.vocab_local
    hi = min(cfg.vocab, lo + model.vocab_local)
    if hi > lo:
        head[: hi - lo] = full[lo:hi]
    if nvfp4_head and cfg.hidden % 128 == 0 and model.vocab_local % 128 == 0:
        model.lm_head = LinearNVFP4.from_dense(head.float().to(dev), gemm_mode or cfg.gemm_mode, search=True).prepare()
    else:
        model.lm_head = LinearBF16(head.to(dev))


def load_moe_family(hf: dict, src: TensorSource, device, comm, gemm_mode="w4a16", quantize=None, nvfp4_head: bool = False):
    cfg = moe_config_from_hf(hf)
    cfg.gemm_mode = gemm_mode
    mla = isinstance(cfg, MLAConfig)
    model = (MLAModel if mla else MoEModel)(cfg, device, comm)
    dev, bf = model.device, torch.bfloat16
    kw = dict(rank=model.comm.rank, world=model.comm.size, device=dev, gemm_mode=gemm_mode, quantize=quantize or "nvfp4")
    model.embed = src.tensor("model.embed_tokens.weight", dev, bf)
    model.heat = torch.zeros(cfg.n_layers, cfg.n_experts, dtype=torch.float32, device=dev)
    model.layers = []

    def load_layer(li):
        p = f"model.layers.{li}."
        L = model.layer_cls()
        (_load_mla if mla else _load_gqa)(model, src, L, p, kw)
        L.attn_norm = src.tensor(p + "input_layernorm.weight", dev, bf)
        L.ffn_norm = src.tensor(p + "post_attention_layernorm.weight", dev, bf)
        _load_ffn(model, src, L, p, li, kw)
        return L

    for li in range(cfg.n_layers):
        model.layers.append(load_layer(li))
    model.final_norm = src.tensor("model.norm.weight", dev, bf)
    load_head(model, src, "model.embed_tokens.weight", nvfp4_head, gemm_mode)
    if mla and cfg.mtp_layers and src.has(f"model.layers.{cfg.n_layers}.eh_proj.weight"):
        p = f"model.layers.{cfg.n_layers}."
        block = load_layer(cfg.n_layers)
        fc = src.tensor(p + "eh_proj.weight", dev).float()
        model.mtp = {"layer": block, "fc": model._make_linear(fc, True), "norm_e": src.tensor(p + "enorm.weight", dev, bf),
                     "norm_h": src.tensor(p + "hnorm.weight", dev, bf),
                     "norm_out": src.tensor(p + "shared_head.norm.weight", dev, bf), "cache_layer": cfg.n_layers}
    return model
