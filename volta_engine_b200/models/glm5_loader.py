"""GLM-5-Next checkpoint directories: the published tensor names -> :class:`.glm5.Glm5NextModel`.

Names (under ``model.language_model.``; a plain ``model.`` prefix is accepted too), per layer ``layers.<i>.``:

  * both layer kinds: ``input_layernorm.weight``, ``post_attention_layernorm.weight``, the six hyper-connection tensors
    ``hc_attn_fn`` [24, 4 H] / ``hc_attn_base`` [24] / ``hc_attn_scale`` [3] and ``hc_ffn_*``;
  * Kimi-delta-attention layers (those that hold ``self_attn.A_log``): ``self_attn.q_proj`` / ``k_proj`` / ``v_proj``
    [heads x 128, H], ``conv1d.weight`` [3 x heads x 128, (1,) 4] in q | k | v order, ``A_log`` [heads], ``dt_bias``
    [heads x 128], ``b_proj.weight`` [heads, H], the low-rank pairs ``f_a_proj`` / ``f_b_proj`` (decay) and ``g_a_proj`` /
    ``g_b_proj`` (output gate), ``o_norm.weight`` [128], ``o_proj``. A rank keeps a contiguous slice of the heads of every
    section; q, k, v and b are stacked into the fused input projection the KDA kernels read;
  * latent-attention layers: the ``q_a`` / ``q_b`` / ``kv_a_proj_with_mqa`` / ``kv_b`` / ``o_proj`` set of the DeepSeek
    family (:func:`.moe_loader._load_mla`) plus the indexer under ``self_attn.indexer.``: ``wq_b``, ``wk.weight``,
    ``weights_proj.weight``, ``index_kpool_compress_gate`` (stacked [k | head weights | pool gate]), ``k_norm.weight`` /
    ``.bias``, ``index_kpool_compress_ape``;
  * feed-forward: ``mlp.gate_proj`` / ``up_proj`` / ``down_proj`` on the leading dense layers, else ``mlp.gate.weight``,
    ``mlp.gate.e_score_correction_bias``, ``mlp.experts.<e>.*`` and ``mlp.shared_experts.*`` (:func:`.moe_loader._load_ffn`);
  * the MTP head is layer ``num_hidden_layers`` (a latent-attention block) with ``eh_proj``, ``enorm``, ``hnorm``,
    ``shared_head.norm``.

Dense projections given as bf16 are quantised to NVFP4 at load (``quantize``); tensors that are NVFP4 in the checkpoint
are taken as they are. Trellis-coded (EXL3) fused ``qkv_proj`` tensors of the KDA layers are not read here.
Reference: src/models/glm5_next.cpp:766-1000 (layer tensors), :1060-1100 (MTP head), :886-916 (indexer).
"""
from __future__ import annotations

import json
from pathlib import Path

import torch

from ..ops.linear import LinearBF16
from .moe_loader import _load_ffn, _load_mla, load_head


def _dense(src, base: str) -> torch.Tensor:
    """The dense fp32 weight of linear ``base`` (bf16 tensors as stored; quantised ones dequantised)."""
    repo = getattr(src, "repo", None)
    if repo is not None and not src.has(base + ".weight"):
        return repo.load_dense_weight(base).float()
    return src.tensor(base + ".weight").float()


def _load_kda(model, src, L, p: str, kw) -> None:
    cfg, dev, d, df = model.cfg, model.device, model.dims, model.dims_full
    from ..ops.gdn import KDAWeights
    r, H, bf = model.comm.rank, cfg.hidden, torch.bfloat16
    assert d.n_k == d.n_v, "KDA has as many key heads as value heads"
    w_in = torch.zeros(d.proj_out, H)
    conv = _maybe(src, p + "self_attn.conv1d.weight").float().reshape(df.conv_dim, -1)
    assert conv.shape[1] == d.conv_k, f"{p}self_attn.conv1d.weight: {conv.shape[1]} taps, the kernels take {d.conv_k}"
    conv_mine, at, at_full = [], 0, 0
    for name, n_full, n_mine, width in (("q_proj", df.n_k, d.n_k, d.dk), ("k_proj", df.n_k, d.n_k, d.dk), ("v_proj", df.n_v, d.n_v, d.dv)):
        w = _dense(src, p + "self_attn." + name)
        assert tuple(w.shape) == (n_full * width, H), f"{p}self_attn.{name}: shape {tuple(w.shape)}"
        lo = r * n_mine * width
        w_in[at:at + n_mine * width] = w[lo:lo + n_mine * width]
        conv_mine.append(conv[at_full + lo:at_full + lo + n_mine * width])
        at += n_mine * width
        at_full += n_full * width
    b = src.tensor(p + "self_attn.b_proj.weight").float()
    b_at = d.conv_dim + d.n_v * d.dv                                  # [q | k | v | (unused z) | b | (unused a)]
    w_in[b_at:b_at + d.n_v] = b[r * d.n_v:(r + 1) * d.n_v]
    v0, v1 = r * d.n_v, (r + 1) * d.n_v
    w_out = _dense(src, p + "self_attn.o_proj")
    f_b = src.tensor(p + "self_attn.f_b_proj.weight").to(bf)
    g_b = src.tensor(p + "self_attn.g_b_proj.weight").to(bf)
    dt = src.tensor(p + "self_attn.dt_bias").float().flatten()
    if dt.numel() == df.n_v:                                          # one bias per head: the same for its channels
        dt = dt.repeat_interleave(d.dk)
    norm_w = src.tensor(p + "self_attn.o_norm.weight").float().to(dev)
    g = {"in_proj": model._make_linear(w_in.to(dev), True),
         "conv_w": torch.cat(conv_mine, 0).contiguous().to(dev),
         "A_log": torch.zeros(d.n_v, device=dev), "dt_bias": torch.zeros(d.n_v, device=dev),      # (gated-delta fields, unused by KDA)
         "norm_w": norm_w,
         "out_proj": model._make_linear(w_out[:, v0 * d.dv:v1 * d.dv].contiguous().to(dev), True)}
    g["kda"] = KDAWeights(f_a=LinearBF16(src.tensor(p + "self_attn.f_a_proj.weight", dev, bf)),
                          f_b=LinearBF16(f_b[v0 * d.dk:v1 * d.dk].contiguous().to(dev)),
                          g_a=LinearBF16(src.tensor(p + "self_attn.g_a_proj.weight", dev, bf)),
                          g_b=LinearBF16(g_b[v0 * d.dv:v1 * d.dv].contiguous().to(dev)),
                          A_log=src.tensor(p + "self_attn.A_log").float().flatten()[v0:v1].contiguous().to(dev),
                          dt_bias=dt[v0 * d.dk:v1 * d.dk].contiguous().to(dev), norm_w=norm_w)
    L.gdn = g
    L.qkv = L.o_proj = None
    L.q_norm = L.k_norm = None


def _maybe(src, name: str) -> torch.Tensor:
    if not src.has(name):
        raise KeyError(f"glm5_next checkpoint: tensor {name} is missing")
    return src.tensor(name)


def _load_indexer(model, src, L, p: str) -> None:
    """The sparse-attention indexer of a latent-attention layer (replicated on every rank: the lists must agree)."""
    from ..ops import dsa as D
    dev, bf = model.device, torch.bfloat16
    pre = p + "self_attn.indexer."
    parts = [_maybe(src, pre + "wk.weight"), _maybe(src, pre + "weights_proj.weight"), _maybe(src, pre + "index_kpool_compress_gate")]
    for t, rows in zip(parts, (D.DIM, D.HEADS, D.DIM)):
        assert tuple(t.shape) == (rows, model.cfg.hidden), f"{pre}: indexer projection shape {tuple(t.shape)}"
    wq = _dense(src, pre + "wq_b")
    assert tuple(wq.shape) == (D.HEADS * D.DIM, model.cfg.q_lora_rank), f"{pre}wq_b: shape {tuple(wq.shape)}"
    L.dsa = D.DSAWeights(proj=LinearBF16(torch.cat([t.to(bf) for t in parts], 0).contiguous().to(dev)),
                         q_proj=LinearBF16(wq.to(bf).to(dev)),
                         ln_w=src.tensor(pre + "k_norm.weight", dev, bf), ln_b=src.tensor(pre + "k_norm.bias", dev, bf),
                         ape=src.tensor(pre + "index_kpool_compress_ape", dev, bf).reshape(D.POOL, D.DIM).contiguous())


def _load_hc(src, p: str, which: str, dev):
    f = lambda n: src.tensor(f"{p}hc_{which}_{n}", dev, torch.float32).contiguous()
    return (f("fn"), f("base").flatten(), f("scale").flatten())


def load_glm5_checkpoint(hf: dict, src, device, comm, gemm_mode: str = "w4a16", quantize=None, nvfp4_head: bool = False):
    from .factory import glm5_config_from_hf
    from .glm5 import Glm5NextModel
    cfg = glm5_config_from_hf(hf)
    cfg.gemm_mode = gemm_mode
    cfg._n_main = cfg.n_layers
    P = "model.language_model." if src.has("model.language_model.embed_tokens.weight") else "model."
    # the checkpoint says which layers are linear; the configuration's interval has to agree with it
    kinds = [src.has(f"{P}layers.{li}.self_attn.A_log") for li in range(cfg.n_layers)]
    want = [not cfg.is_full(li) for li in range(cfg.n_layers)]
    if kinds != want:
        raise ValueError(f"glm5_next: the checkpoint's linear-attention layers {[i for i, k in enumerate(kinds) if k]} do not "
                         f"follow the configured interval of {cfg.full_interval}")
    cfg.dsa = bool(cfg.dsa and any(src.has(f"{P}layers.{li}.self_attn.indexer.wk.weight") for li in range(cfg.n_layers)))
    cfg.residual = "hc" if src.has(f"{P}layers.0.hc_attn_fn") else "plain"
    model = Glm5NextModel(cfg, device, comm)
    dev, bf = model.device, torch.bfloat16
    kw = dict(rank=model.comm.rank, world=model.comm.size, device=dev, gemm_mode=gemm_mode, quantize=quantize or "nvfp4")
    model.embed = src.tensor(P + "embed_tokens.weight", dev, bf)
    model.heat = torch.zeros(cfg.n_layers + int(cfg.mtp_layers or 0), cfg.n_experts, dtype=torch.float32, device=dev)
    model.layers = []
    n_attn = 0

    def load_layer(li: int, linear: bool):
        nonlocal n_attn
        p = f"{P}layers.{li}."
        L = model.layer_cls()
        L.gdn = L.gate_proj = L.qsa = L.dsa = None
        L.kv_index = -1
        if linear:
            _load_kda(model, src, L, p, kw)
        else:
            _load_mla(model, src, L, p, kw)
            L.kv_index = n_attn
            n_attn += 1
            if cfg.dsa and src.has(p + "self_attn.indexer.wk.weight"):
                _load_indexer(model, src, L, p)
        L.attn_norm = src.tensor(p + "input_layernorm.weight", dev, bf)
        L.ffn_norm = src.tensor(p + "post_attention_layernorm.weight", dev, bf)
        _load_ffn(model, src, L, p, li, kw)
        if cfg.residual == "hc" and src.has(p + "hc_attn_fn"):
            L.attn_hc, L.mlp_hc = _load_hc(src, p, "attn", dev), _load_hc(src, p, "ffn", dev)
        return L

    for li in range(cfg.n_layers):
        model.layers.append(load_layer(li, kinds[li]))
    model.final_norm = src.tensor(P + "norm.weight", dev, bf)
    load_head(model, src, P + "embed_tokens.weight", nvfp4_head)
    model.final_hc = None                               # the head reads the mean of the streams
    p = f"{P}layers.{cfg.n_layers}."
    if cfg.mtp_layers and src.has(p + "eh_proj.weight"):
        block = load_layer(cfg.n_layers, False)
        model.mtp = {"layer": block, "fc": model._make_linear(src.tensor(p + "eh_proj.weight", dev).float(), True),
                     "norm_e": src.tensor(p + "enorm.weight", dev, bf), "norm_h": src.tensor(p + "hnorm.weight", dev, bf),
                     "norm_out": src.tensor(p + "shared_head.norm.weight", dev, bf), "cache_layer": cfg.n_layers}
    else:
        cfg.mtp_layers = 0
    return model


def save_glm5_checkpoint(model_dir, cfg, seed: int = 0, std: float = 0.05, prefix: str = "model.language_model.") -> dict:
    """Write a random-weight GLM-5-Next directory (``config.json`` + one bf16 safetensors file) under the published
    tensor names, for tests and synthetic runs. Returns the tensors written."""
    from ..loader.safetensors import write_safetensors
    from ..ops import dsa as D
    d = Path(model_dir)
    d.mkdir(parents=True, exist_ok=True)
    g = torch.Generator().manual_seed(seed)
    bf = torch.bfloat16
    H, nh, dk, kr = cfg.hidden, cfg.gdn_k_heads, cfg.gdn_dk, cfg.kda_rank
    n_mla = sum(1 for li in range(cfg.n_layers) if cfg.is_full(li))
    hf = {"model_type": "glm5_next", "num_hidden_layers": cfg.n_layers, "num_mla_layers": n_mla, "hidden_size": H,
          "num_attention_heads": cfg.n_q, "dense_intermediate_size": cfg.ffn, "moe_intermediate_size": cfg.expert_ffn,
          "n_shared_experts": 1 if cfg.shared_ffn else 0, "n_routed_experts": cfg.n_experts, "num_experts_per_tok": cfg.top_k,
          "first_k_dense_replace": cfg.first_dense_layers, "routed_scaling_factor": cfg.router_scale, "vocab_size": cfg.vocab,
          "q_lora_rank": cfg.q_lora_rank, "qk_nope_head_dim": cfg.qk_nope, "v_head_dim": cfg.v_head_dim, "kda_heads": nh,
          "kda_head_dim": dk, "kda_rank": kr, "rms_norm_eps": cfg.rms_eps, "rope_theta": cfg.rope_theta,
          "num_nextn_predict_layers": cfg.mtp_layers, "dsa": bool(cfg.dsa), "hc_mult": 4 if cfg.residual == "hc" else 1}
    (d / "config.json").write_text(json.dumps(hf, indent=1))
    rnd = lambda *s, k=1.0: (torch.randn(*s, generator=g) * std * k).to(bf)
    ones = lambda n: (torch.ones(n) * (1.0 - cfg.norm_bias)).to(bf)
    t = {prefix + "embed_tokens.weight": rnd(cfg.vocab, H), "lm_head.weight": rnd(cfg.vocab, H), prefix + "norm.weight": ones(H)}

    def layer(li: int, linear: bool):
        p = f"{prefix}layers.{li}."
        t[p + "input_layernorm.weight"], t[p + "post_attention_layernorm.weight"] = ones(H), ones(H)
        a = p + "self_attn."
        if linear:
            for n in ("q_proj", "k_proj", "v_proj"):
                t[a + n + ".weight"] = rnd(nh * dk, H)
            t[a + "conv1d.weight"] = (torch.randn(3 * nh * dk, 1, cfg.gdn_conv, generator=g) * 0.5).to(bf)
            t[a + "A_log"] = torch.log(torch.linspace(0.5, 2.0, nh))
            t[a + "dt_bias"] = torch.linspace(-1.0, 1.0, nh * dk)
            t[a + "b_proj.weight"] = rnd(nh, H)
            t[a + "f_a_proj.weight"], t[a + "f_b_proj.weight"] = rnd(kr, H), rnd(nh * dk, kr, k=4)
            t[a + "g_a_proj.weight"], t[a + "g_b_proj.weight"] = rnd(kr, H), rnd(nh * dk, kr, k=4)
            t[a + "o_norm.weight"] = torch.ones(dk).to(bf)
            t[a + "o_proj.weight"] = rnd(H, nh * dk)
        else:
            qd = cfg.qk_nope + cfg.qk_rope
            t[a + "q_a_proj.weight"], t[a + "q_a_layernorm.weight"] = rnd(cfg.q_lora_rank, H), torch.ones(cfg.q_lora_rank).to(bf)
            t[a + "kv_a_proj_with_mqa.weight"], t[a + "kv_a_layernorm.weight"] = rnd(cfg.kv_lora_rank + cfg.qk_rope, H), torch.ones(cfg.kv_lora_rank).to(bf)
            t[a + "q_b_proj.weight"] = rnd(cfg.n_q * qd, cfg.q_lora_rank)
            t[a + "kv_b_proj.weight"] = rnd(cfg.n_q * (cfg.qk_nope + cfg.v_head_dim), cfg.kv_lora_rank)
            t[a + "o_proj.weight"] = rnd(H, cfg.n_q * cfg.v_head_dim)
            if cfg.dsa:
                i = a + "indexer."
                t[i + "wq_b.weight"] = rnd(D.HEADS * D.DIM, cfg.q_lora_rank, k=8)
                t[i + "wk.weight"], t[i + "weights_proj.weight"] = rnd(D.DIM, H, k=8), rnd(D.HEADS, H, k=8)
                t[i + "index_kpool_compress_gate"] = rnd(D.DIM, H, k=8)
                t[i + "k_norm.weight"], t[i + "k_norm.bias"] = torch.ones(D.DIM).to(bf), torch.zeros(D.DIM).to(bf)
                t[i + "index_kpool_compress_ape"] = rnd(D.POOL, D.DIM, k=20)
        m = p + "mlp."
        if li < cfg.first_dense_layers:
            t[m + "gate_proj.weight"], t[m + "up_proj.weight"], t[m + "down_proj.weight"] = rnd(cfg.ffn, H), rnd(cfg.ffn, H), rnd(H, cfg.ffn)
        else:
            I = cfg.expert_ffn
            t[m + "gate.weight"], t[m + "gate.e_score_correction_bias"] = rnd(cfg.n_experts, H), torch.zeros(cfg.n_experts)
            for e in range(cfg.n_experts):
                t[m + f"experts.{e}.gate_proj.weight"], t[m + f"experts.{e}.up_proj.weight"] = rnd(I, H), rnd(I, H)
                t[m + f"experts.{e}.down_proj.weight"] = rnd(H, I)
            if cfg.shared_ffn:
                S = cfg.shared_ffn
                t[m + "shared_experts.gate_proj.weight"], t[m + "shared_experts.up_proj.weight"] = rnd(S, H), rnd(S, H)
                t[m + "shared_experts.down_proj.weight"] = rnd(H, S)
        if cfg.residual == "hc":
            for w in ("attn", "ffn"):
                t[p + f"hc_{w}_fn"] = torch.randn(24, 4 * H, generator=g) * 0.02
                t[p + f"hc_{w}_base"] = torch.randn(24, generator=g) * 0.5
                t[p + f"hc_{w}_scale"] = torch.tensor([0.5, 0.5, 0.5])
        return p

    for li in range(cfg.n_layers):
        layer(li, not cfg.is_full(li))
    if cfg.mtp_layers:
        p = layer(cfg.n_layers, False)
        t[p + "eh_proj.weight"] = rnd(H, 2 * H)
        t[p + "enorm.weight"], t[p + "hnorm.weight"], t[p + "shared_head.norm.weight"] = ones(H), ones(H), ones(H)
    write_safetensors(d / "model.safetensors", t)
    return t
