"""Hybrid Gated-DeltaNet / gated-attention checkpoints (``model_type`` qwen3_5, qwen3_5_moe, qwen3_next, and the
Flash-Next assembly qwen4_exp) -> :class:`.hybrid.HybridModel`.

Names (under ``model.language_model.``; a plain ``model.`` prefix is accepted too), per layer ``layers.<i>.``:

  * linear layers (those that hold ``linear_attn.A_log``): ``linear_attn.in_proj_qkv`` (rows [q | k | v]: key heads x dk,
    key heads x dk, value heads x dv), ``in_proj_z`` (value heads x dv), ``in_proj_b.weight`` / ``in_proj_a.weight`` (one row
    per value head), ``conv1d.weight`` [q | k | v channels, (1,) taps], ``A_log`` / ``dt_bias`` [value heads],
    ``norm.weight`` [dv], ``out_proj``. The six projections are stacked into the fused input projection the kernels read
    ([q | k | v | z | b | a]); a rank keeps a contiguous slice of the heads of every section;
  * full-attention layers: ``self_attn.q_proj`` carries the output gate (per head 2 x head_dim rows: query, then gate),
    ``k_proj``, ``v_proj``, ``o_proj``, ``q_norm.weight``, ``k_norm.weight``;
  * feed-forward: ``mlp.gate_proj`` / ``up_proj`` / ``down_proj``, or a router ``mlp.gate.weight`` with ``mlp.experts.<e>.*``,
    ``mlp.shared_expert.*`` and ``mlp.shared_expert_gate.weight`` (:func:`.moe_loader._load_ffn`);
  * the MTP head: ``mtp.fc`` ([H, 2 H] over [norm(embedding) | norm(hidden)]), ``mtp.pre_fc_norm_embedding.weight``,
    ``mtp.pre_fc_norm_hidden.weight``, ``mtp.layers.0.*`` (a full-attention block), ``mtp.norm.weight``.

  * qwen4_exp adds, per sublayer, the gated residual-stream mixers ``attn_hyper_connection`` / ``mlp_hyper_connection``
    (``hc_norm.weight`` [streams, H], ``input_mix_weight_down.weight`` [rank, streams x H], ``input_mix_weight_up.weight``
    [streams x H, rank], ``block_inject_weight.weight`` [streams, streams x H]), the final ``hyper_connection_mixer`` (no
    inject), and on the full-attention layers the block-sparse indexer ``self_attn.indexer.index_qk_proj`` /
    ``q_layernorm.weight`` / ``k_layernorm.weight``. Its n-gram embedding tensors (``layers.<i>.ple.*``) have no counterpart
    in this model and a checkpoint that carries them is refused.

RMSNorm weights are stored as w - 1 (``norm_bias`` 1), the gated norm of the linear layers as w.
Reference: src/models/qwen3_5.cpp:330-440 (layer tensors and their tensor-parallel slices), :440-520 (MTP head),
inc/engine/models/qwen3_5.h:30-52 (shape and norm bias); src/models/qwen4_exp.cpp:451-478 (mixers), :576-584 (indexer),
:82-99 (configuration keys).
"""
from __future__ import annotations

import json
from pathlib import Path

import torch

from .glm5_loader import _dense, _maybe
from .moe_loader import _load_ffn, load_head

HYBRID_TYPES = {"qwen3_5", "qwen3_5_text", "qwen3_5_moe", "qwen3_next", "qwen4_exp"}


def hybrid_config_from_hf(c: dict):
    from .hybrid import HybridConfig
    hd = int(c.get("head_dim") or c["hidden_size"] // c["num_attention_heads"])
    n = int(c["num_hidden_layers"])
    E = int(c.get("num_experts", c.get("n_routed_experts", 0)) or 0)
    moe_ffn = int(c.get("moe_intermediate_size", 0) or 0)
    cfg = HybridConfig(
        n_layers=n, hidden=int(c["hidden_size"]), n_q=int(c["num_attention_heads"]),
        n_kv=int(c.get("num_key_value_heads", c["num_attention_heads"])), head_dim=hd, ffn=int(c.get("intermediate_size", 0) or 0),
        vocab=int(c["vocab_size"]), rope_theta=float(c.get("rope_theta", 1e7)), rms_eps=float(c.get("rms_norm_eps", 1e-6)),
        norm_bias=1.0, rot_dim=int(hd * float(c.get("partial_rotary_factor", 0.25))), qk_norm=True,
        tie_embeddings=bool(c.get("tie_word_embeddings", False)),
        n_experts=E or 1, top_k=int(c.get("num_experts_per_tok", 1) or 1), expert_ffn=moe_ffn or 128,
        shared_ffn=int(c.get("shared_expert_intermediate_size", 0) or 0) if E else 0, shared_gate=bool(E),
        router="softmax", first_dense_layers=0 if E else n,
        full_interval=int(c.get("full_attention_interval", 4)), gdn_k_heads=int(c.get("linear_num_key_heads", 16)),
        gdn_v_heads=int(c.get("linear_num_value_heads", 32)), gdn_dk=int(c.get("linear_key_head_dim", 128)),
        gdn_dv=int(c.get("linear_value_head_dim", 128)), gdn_conv=int(c.get("linear_conv_kernel_dim", 4)), attn_gate=True,
        mtp_layers=int(c.get("mtp_num_hidden_layers", c.get("num_nextn_predict_layers", 0)) or 0), quant=c.get("volta_quant", "nvfp4"),
        model_type=c.get("model_type", "qwen3_5"))
    if c.get("model_type") == "qwen4_exp" or int(c.get("hc_count", 0) or 0) > 1:
        cfg.residual, cfg.hc_mult, cfg.hc_rank = "gated", int(c.get("hc_count", 4)), int(c.get("hc_rank", cfg.hc_rank))
    return cfg


def _load_mixer(src, prefix: str, dev, inject: bool):
    from ..ops.streams import GatedResidualWeights
    bf = torch.bfloat16
    return GatedResidualWeights(norm=src.tensor(prefix + ".hc_norm.weight", dev, bf),
                                down=src.tensor(prefix + ".input_mix_weight_down.weight", dev, bf).contiguous(),
                                up=src.tensor(prefix + ".input_mix_weight_up.weight", dev, bf).contiguous(),
                                inject=src.tensor(prefix + ".block_inject_weight.weight", dev, bf).contiguous() if inject else None)


def _load_gdn(model, src, L, p: str) -> None:
    cfg, dev, d, df = model.cfg, model.device, model.dims, model.dims_full
    r, H = model.comm.rank, cfg.hidden
    a = p + "linear_attn."
    qkv = _dense(src, a + "in_proj_qkv")
    assert tuple(qkv.shape) == (df.conv_dim, H), f"{a}in_proj_qkv: shape {tuple(qkv.shape)}"
    z = _dense(src, a + "in_proj_z")
    b, aa = _maybe(src, a + "in_proj_b.weight").float(), _maybe(src, a + "in_proj_a.weight").float()
    conv = _maybe(src, a + "conv1d.weight").float().reshape(df.conv_dim, -1)
    assert conv.shape[1] == d.conv_k, f"{a}conv1d.weight: {conv.shape[1]} taps, the kernels take {d.conv_k}"
    full = torch.cat([qkv, z, b, aa], 0)                                # [q | k | v | z | b | a] of all heads
    sizes_full = [df.n_k * d.dk, df.n_k * d.dk, df.n_v * d.dv, df.n_v * d.dv, df.n_v, df.n_v]
    sizes_mine = [d.n_k * d.dk, d.n_k * d.dk, d.n_v * d.dv, d.n_v * d.dv, d.n_v, d.n_v]
    rows, at = [], 0
    for nf, nm in zip(sizes_full, sizes_mine):
        rows.append(torch.arange(at + r * nm, at + (r + 1) * nm))
        at += nf
    rows = torch.cat(rows)
    w_in = torch.zeros(d.proj_out, H)
    w_in[:rows.numel()] = full[rows]
    v0, v1 = r * d.n_v, (r + 1) * d.n_v
    w_out = _dense(src, a + "out_proj")
    L.gdn = {"in_proj": model._make_linear(w_in.to(dev), True),
             "conv_w": conv[rows[: d.conv_dim]].contiguous().to(dev),
             "A_log": _maybe(src, a + "A_log").float().flatten()[v0:v1].contiguous().to(dev),
             "dt_bias": _maybe(src, a + "dt_bias").float().flatten()[v0:v1].contiguous().to(dev),
             "norm_w": _maybe(src, a + "norm.weight").float().to(dev),
             "out_proj": model._make_linear(w_out[:, v0 * d.dv:v1 * d.dv].contiguous().to(dev), True)}
    L.qkv = L.o_proj = L.q_norm = L.k_norm = None


def _load_gated_attention(model, src, L, p: str) -> None:
    cfg, dev, bf = model.cfg, model.device, torch.bfloat16
    r, tp, hd, H = model.comm.rank, model.comm.size, cfg.head_dim, cfg.hidden
    a = p + "self_attn."
    wq = _dense(src, a + "q_proj")
    gated = wq.shape[0] == 2 * cfg.n_q * hd
    assert gated or wq.shape[0] == cfg.n_q * hd, f"{a}q_proj: {wq.shape[0]} rows for {cfg.n_q} heads of {hd}"
    if gated:                                                            # per head: head_dim query rows, then head_dim gate rows
        wq = wq.reshape(cfg.n_q, 2, hd, H)
        wq, wg = wq[:, 0].reshape(cfg.n_q * hd, H), wq[:, 1].reshape(cfg.n_q * hd, H)
    q0, q1 = r * model.nq * hd, (r + 1) * model.nq * hd
    kr = r if cfg.n_kv >= tp else r // model.kv_rep                      # fewer KV heads than ranks: a head serves kv_rep ranks
    k0, k1 = kr * model.nkv * hd, (kr + 1) * model.nkv * hd
    wk, wv = _dense(src, a + "k_proj"), _dense(src, a + "v_proj")
    L.qkv = model._make_linear(torch.cat([wq[q0:q1], wk[k0:k1], wv[k0:k1]], 0).contiguous().to(dev), True)
    L.gate_proj = model._make_linear(wg[q0:q1].contiguous().to(dev), True) if gated and cfg.attn_gate else None
    wo = _dense(src, a + "o_proj")
    L.o_proj = model._make_linear(wo[:, q0:q1].contiguous().to(dev), True)
    L.q_norm = src.tensor(a + "q_norm.weight", dev, bf) if src.has(a + "q_norm.weight") else None
    L.k_norm = src.tensor(a + "k_norm.weight", dev, bf) if src.has(a + "k_norm.weight") else None


def load_hybrid(hf: dict, src, device, comm, gemm_mode: str = "w4a16", quantize=None, nvfp4_head: bool = False):
    from .hybrid import HybridModel
    cfg = hybrid_config_from_hf(hf)
    cfg.gemm_mode = gemm_mode
    cfg._n_main = cfg.n_layers
    if cfg.first_dense_layers >= cfg.n_layers:                          # no routed experts: the placeholder count divides by the ranks
        cfg.n_experts = max(1, comm.size if comm is not None else 1)
    P = "model.language_model." if src.has("model.language_model.embed_tokens.weight") else "model."
    kinds = [src.has(f"{P}layers.{li}.linear_attn.A_log") for li in range(cfg.n_layers)]
    if kinds != [not cfg.is_full(li) for li in range(cfg.n_layers)]:
        raise ValueError(f"{cfg.model_type}: the checkpoint's linear-attention layers {[i for i, k in enumerate(kinds) if k]} do "
                         f"not follow the configured interval of {cfg.full_interval}")
    if cfg.mtp_layers and not (src.has("mtp.fc.weight") or src.has("mtp.fc.weight_packed") or src.has("mtp.fc.trellis")):
        cfg.mtp_layers = 0                                               # the checkpoint was exported without its MTP head
    cfg.qk_norm = src.has(f"{P}layers.{cfg.full_interval - 1}.self_attn.q_norm.weight")
    if any(src.has(f"{P}layers.{li}.ple.{n}") for li in range(cfg.n_layers) for n in ("key_proj.weight", "conv1d.weight", "norm_key.weight")):
        raise NotImplementedError(f"{cfg.model_type}: the checkpoint carries n-gram embedding tensors (layers.<i>.ple.*), which "
                                  "this model does not implement")
    cfg.qsa = src.has(f"{P}layers.{cfg.full_interval - 1}.self_attn.indexer.index_qk_proj.weight")
    gated_streams = cfg.residual == "gated"
    if gated_streams:
        cfg.hc_rank = int(src.tensor(f"{P}layers.0.attn_hyper_connection.input_mix_weight_down.weight").shape[0])
    model = HybridModel(cfg, device, comm)
    dev, bf = model.device, torch.bfloat16
    kw = dict(rank=model.comm.rank, world=model.comm.size, device=dev, gemm_mode=gemm_mode, quantize=quantize or "nvfp4")
    model.embed = src.tensor(P + "embed_tokens.weight", dev, bf)
    model.heat = torch.zeros(cfg.n_layers + cfg.mtp_layers, cfg.n_experts, dtype=torch.float32, device=dev)
    model.layers = []
    n_attn = 0

    def load_layer(p: str, li: int, linear: bool):
        nonlocal n_attn
        L = model.layer_cls()
        L.gdn = L.gate_proj = L.qsa = None
        L.kv_index = -1
        if linear:
            _load_gdn(model, src, L, p)
        else:
            _load_gated_attention(model, src, L, p)
            L.kv_index = n_attn
            n_attn += 1
            if cfg.qsa and src.has(p + "self_attn.indexer.index_qk_proj.weight"):
                from ..ops import dsa as D
                from ..ops.linear import LinearBF16
                L.qsa = D.QSAWeights(proj=LinearBF16(src.tensor(p + "self_attn.indexer.index_qk_proj.weight", dev, bf)),
                                     q_norm=src.tensor(p + "self_attn.indexer.q_layernorm.weight", dev, bf),
                                     k_norm=src.tensor(p + "self_attn.indexer.k_layernorm.weight", dev, bf),
                                     rot=min(64, D.DIM), theta=cfg.rope_theta, eps=cfg.rms_eps)
        if gated_streams and src.has(p + "attn_hyper_connection.hc_norm.weight"):
            L.attn_hc = _load_mixer(src, p + "attn_hyper_connection", dev, True)
            L.mlp_hc = _load_mixer(src, p + "mlp_hyper_connection", dev, True)
        L.attn_norm = src.tensor(p + "input_layernorm.weight", dev, bf)
        L.ffn_norm = src.tensor(p + "post_attention_layernorm.weight", dev, bf)
        _load_ffn(model, src, L, p, li, kw)
        return L

    for li in range(cfg.n_layers):
        model.layers.append(load_layer(f"{P}layers.{li}.", li, kinds[li]))
    model.final_norm = src.tensor(P + "norm.weight", dev, bf)
    load_head(model, src, P + "embed_tokens.weight", nvfp4_head)
    if gated_streams:
        model.final_hc = _load_mixer(src, P.rstrip(".") + ".hyper_connection_mixer", dev, False)
    if cfg.mtp_layers:
        block = load_layer("mtp.layers.0.", cfg.n_layers, False)
        model.mtp = {"layer": block, "fc": model._make_linear(_dense(src, "mtp.fc").to(dev), True),
                     "norm_e": src.tensor("mtp.pre_fc_norm_embedding.weight", dev, bf),
                     "norm_h": src.tensor("mtp.pre_fc_norm_hidden.weight", dev, bf),
                     "norm_out": src.tensor("mtp.norm.weight", dev, bf), "cache_layer": cfg.n_layers}
    return model


def save_hybrid_checkpoint(model_dir, cfg, seed: int = 0, std: float = 0.05, prefix: str = "model.language_model.") -> dict:
    """Write a random-weight hybrid directory (``config.json`` + one bf16 safetensors file) under the checkpoint's tensor
    names, for tests and synthetic runs. Returns the tensors written."""
    from ..loader.safetensors import write_safetensors
    d = Path(model_dir)
    d.mkdir(parents=True, exist_ok=True)
    g = torch.Generator().manual_seed(seed)
    bf = torch.bfloat16
    H, hd, nk, nv, dk, dv = cfg.hidden, cfg.head_dim, cfg.gdn_k_heads, cfg.gdn_v_heads, cfg.gdn_dk, cfg.gdn_dv
    moe = cfg.first_dense_layers < cfg.n_layers
    hf = {"model_type": "qwen3_5_moe" if moe else "qwen3_5", "num_hidden_layers": cfg.n_layers, "hidden_size": H,
          "num_attention_heads": cfg.n_q, "num_key_value_heads": cfg.n_kv, "head_dim": hd, "intermediate_size": cfg.ffn,
          "vocab_size": cfg.vocab, "rope_theta": cfg.rope_theta, "partial_rotary_factor": cfg.rot_dim / hd, "rms_norm_eps": cfg.rms_eps,
          "full_attention_interval": cfg.full_interval, "linear_num_key_heads": nk, "linear_num_value_heads": nv,
          "linear_key_head_dim": dk, "linear_value_head_dim": dv, "linear_conv_kernel_dim": cfg.gdn_conv,
          "mtp_num_hidden_layers": cfg.mtp_layers, "volta_quant": cfg.quant}
    if moe:
        hf.update({"num_experts": cfg.n_experts, "num_experts_per_tok": cfg.top_k, "moe_intermediate_size": cfg.expert_ffn,
                   "shared_expert_intermediate_size": cfg.shared_ffn})
    (d / "config.json").write_text(json.dumps(hf, indent=1))
    rnd = lambda *s, k=1.0: (torch.randn(*s, generator=g) * std * k).to(bf)
    zeros = lambda n: torch.zeros(n).to(bf)                              # RMSNorm weights are stored as w - 1
    t = {prefix + "embed_tokens.weight": rnd(cfg.vocab, H), "lm_head.weight": rnd(cfg.vocab, H), prefix + "norm.weight": zeros(H)}

    def layer(p: str, li: int, linear: bool):
        t[p + "input_layernorm.weight"], t[p + "post_attention_layernorm.weight"] = zeros(H), zeros(H)
        if linear:
            a = p + "linear_attn."
            t[a + "in_proj_qkv.weight"], t[a + "in_proj_z.weight"] = rnd(2 * nk * dk + nv * dv, H), rnd(nv * dv, H)
            t[a + "in_proj_b.weight"], t[a + "in_proj_a.weight"] = rnd(nv, H), rnd(nv, H)
            t[a + "conv1d.weight"] = (torch.randn(2 * nk * dk + nv * dv, 1, cfg.gdn_conv, generator=g) * 0.5).to(bf)
            t[a + "A_log"], t[a + "dt_bias"] = torch.log(torch.linspace(1.0, 8.0, nv)), torch.linspace(-1.0, 1.0, nv)
            t[a + "norm.weight"], t[a + "out_proj.weight"] = torch.ones(dv).to(bf), rnd(H, nv * dv)
        else:
            a = p + "self_attn."
            t[a + "q_proj.weight"] = rnd(cfg.n_q * hd * (2 if cfg.attn_gate else 1), H)
            t[a + "k_proj.weight"], t[a + "v_proj.weight"] = rnd(cfg.n_kv * hd, H), rnd(cfg.n_kv * hd, H)
            t[a + "o_proj.weight"] = rnd(H, cfg.n_q * hd)
            t[a + "q_norm.weight"], t[a + "k_norm.weight"] = zeros(hd), zeros(hd)
        m = p + "mlp."
        if li < cfg.first_dense_layers:
            t[m + "gate_proj.weight"], t[m + "up_proj.weight"], t[m + "down_proj.weight"] = rnd(cfg.ffn, H), rnd(cfg.ffn, H), rnd(H, cfg.ffn)
        else:
            I, S = cfg.expert_ffn, cfg.shared_ffn
            t[m + "gate.weight"] = rnd(cfg.n_experts, H)
            for e in range(cfg.n_experts):
                t[m + f"experts.{e}.gate_proj.weight"], t[m + f"experts.{e}.up_proj.weight"] = rnd(I, H), rnd(I, H)
                t[m + f"experts.{e}.down_proj.weight"] = rnd(H, I)
            if S:
                t[m + "shared_expert.gate_proj.weight"], t[m + "shared_expert.up_proj.weight"] = rnd(S, H), rnd(S, H)
                t[m + "shared_expert.down_proj.weight"], t[m + "shared_expert_gate.weight"] = rnd(H, S), rnd(1, H)

    def mixer(pfx: str, inject: bool):
        hc, rk = cfg.hc_mult, cfg.hc_rank
        t[pfx + ".hc_norm.weight"] = rnd(hc, H)
        t[pfx + ".input_mix_weight_down.weight"], t[pfx + ".input_mix_weight_up.weight"] = rnd(rk, hc * H), rnd(hc * H, rk, k=4)
        if inject:
            t[pfx + ".block_inject_weight.weight"] = rnd(hc, hc * H)

    for li in range(cfg.n_layers):
        p = f"{prefix}layers.{li}."
        layer(p, li, not cfg.is_full(li))
        if cfg.residual == "gated":
            mixer(p + "attn_hyper_connection", True)
            mixer(p + "mlp_hyper_connection", True)
        if cfg.qsa and cfg.is_full(li):
            from ..ops import dsa as D
            t[p + "self_attn.indexer.index_qk_proj.weight"] = rnd(D.QSA_HEADS * D.DIM + D.DIM, H, k=8)
            t[p + "self_attn.indexer.q_layernorm.weight"], t[p + "self_attn.indexer.k_layernorm.weight"] = zeros(D.DIM), zeros(D.DIM)
    if cfg.residual == "gated":
        mixer(prefix.rstrip(".") + ".hyper_connection_mixer", False)
        hf.update({"model_type": "qwen4_exp", "hc_count": cfg.hc_mult, "hc_rank": cfg.hc_rank})
        (d / "config.json").write_text(json.dumps(hf, indent=1))
    if cfg.mtp_layers:
        layer("mtp.layers.0.", cfg.n_layers, False)
        t["mtp.fc.weight"] = rnd(H, 2 * H)
        for n in ("mtp.pre_fc_norm_embedding.weight", "mtp.pre_fc_norm_hidden.weight", "mtp.norm.weight"):
            t[n] = zeros(H)
    write_safetensors(d / "model.safetensors", t)
    return t
