"""The GLM-5-Next-style assembly (KDA mixers + latent attention with the indexer + experts + hyper-connection streams +
MTP head): chunked prefill and decode agree with a whole prefill on the CPU statement, the CUDA path agrees with the CPU
statement, the MTP rounds on the device reproduce plain greedy decoding, and the launch configuration maps."""
import json

import pytest
import torch

from volta_engine_b200.models.glm5 import Glm5NextConfig, Glm5NextModel
from volta_engine_b200.runtime.engine import Engine


def _model(dev, **kw):
    cfg = Glm5NextConfig.tiny_glm5(**kw)
    m = Glm5NextModel(cfg, dev).init_random(seed=3)
    if cfg.residual != "plain":
        m.init_stream_weights()
    return cfg, m


@pytest.mark.parametrize("kw", [{}, {"residual": "hc"}, {"dsa": True}, {"mtp_layers": 1}])
def test_glm5_prefill_equals_decode_on_cpu(kw):
    cfg, m = _model("cpu", **kw)
    assert ["kda" if L.gdn is not None else "mla" for L in m.layers] == ["kda", "mla", "kda", "mla"]
    assert m.kv_layers == 2 + cfg.mtp_layers
    assert m.prefix_resume == (None if cfg.dsa else "kv+state")
    prompt = list(range(5, 45))
    out, _ = Engine(m, m.make_cache(16, 2, 512), use_graphs=False, prefill_chunk=16).generate(prompt, 5)
    m.gdn_states = None
    nxt = Engine(m, m.make_cache(16, 2, 512), use_graphs=False, prefill_chunk=1000).prefill(0, prompt + out[:3])
    assert nxt == out[3]


def test_glm5_config_from_launch_directory(tmp_path):
    from volta_engine_b200.models.factory import glm5_config_from_hf, load_model
    c = glm5_config_from_hf({})
    assert (c.n_layers, c.hidden, c.n_experts, c.top_k, c.expert_ffn, c.ffn, c.vocab) == (45, 4096, 288, 8, 2048, 12288, 154880)
    assert sum(1 for li in range(c.n_layers) if c.is_full(li)) == 11 and c.linear_mixer == "kda" and c.residual == "hc"
    hf = {"model_type": "glm5_next", "num_hidden_layers": 4, "num_mla_layers": 2, "hidden_size": 256, "num_attention_heads": 4,
          "dense_intermediate_size": 512, "moe_intermediate_size": 128, "n_routed_experts": 8, "num_experts_per_tok": 2,
          "first_k_dense_replace": 1, "vocab_size": 1024, "q_lora_rank": 128, "kda_heads": 2, "kda_head_dim": 64, "kda_rank": 32,
          "num_nextn_predict_layers": 0, "dsa": False, "synthetic_weights": 5, "expert_quant": "nvfp4"}
    (tmp_path / "config.json").write_text(json.dumps(hf))
    m, _ = load_model(tmp_path, device="cpu")
    assert isinstance(m, Glm5NextModel) and len(m.layers) == 4 and m.kv_layers == 2
    out, _ = Engine(m, m.make_cache(16, 1, 256), use_graphs=False, prefill_chunk=16).generate(list(range(3, 30)), 3)
    assert len(out) == 3
    (tmp_path / "config.json").write_text(json.dumps({k: v for k, v in hf.items() if k != "synthetic_weights"}))
    with pytest.raises(FileNotFoundError):                     # no synthetic seed: the directory has to hold the tensors
        load_model(tmp_path, device="cpu")


def test_glm5_checkpoint_directory_loads_under_the_published_names(tmp_path):
    """A directory written under the checkpoint's tensor names (KDA q / k / v / conv / gates, latent attention with the
    indexer, experts + shared expert, hyper-connection tensors, MTP head as layer n) loads, generates, and a rank of a
    two-rank layout holds its heads' slice of every KDA section."""
    from volta_engine_b200.models.factory import load_model
    from volta_engine_b200.models.glm5_loader import load_glm5_checkpoint, save_glm5_checkpoint
    from volta_engine_b200.models.factory import TensorSource
    from volta_engine_b200.parallel.comm import LocalComm
    cfg = Glm5NextConfig.tiny_glm5(residual="hc", dsa=True, mtp_layers=1, qk_nope=192, v_head_dim=256, gdn_k_heads=4, gdn_v_heads=4,
                                   expert_ffn=256, shared_ffn=256)
    t = save_glm5_checkpoint(tmp_path, cfg, seed=2)
    P = "model.language_model."
    m, hf = load_model(tmp_path, device="cpu")
    assert isinstance(m, Glm5NextModel) and ["kda" if L.gdn is not None else "mla" for L in m.layers] == ["kda", "mla", "kda", "mla"]
    c = m.cfg
    assert (c.qk_nope, c.v_head_dim, c.gdn_k_heads, c.residual, c.dsa, c.mtp_layers) == (192, 256, 4, "hc", True, 1)
    assert m.mtp is not None and m.mtp["layer"].kv_index == 2 and m.mtp["layer"].dsa is not None and m.kv_layers == 3
    assert m.layers[0].dense_ffn and not m.layers[1].dense_ffn and m.layers[1].router_bias is not None
    L0, d = m.layers[0], m.dims
    w = L0.gdn["in_proj"].dequant() if hasattr(L0.gdn["in_proj"], "dequant") else L0.gdn["in_proj"].weight.float()
    q, k, v = (t[P + f"layers.0.self_attn.{n}_proj.weight"].float() for n in "qkv")
    from util import cos
    n = d.n_k * d.dk
    assert cos(w[:n], q) > 0.99 and cos(w[n:2 * n], k) > 0.99 and cos(w[2 * n:3 * n], v) > 0.99
    b_at = d.conv_dim + d.n_v * d.dv
    assert float(w[3 * n:b_at].abs().max()) == 0.0 and cos(w[b_at:b_at + d.n_v], t[P + "layers.0.self_attn.b_proj.weight"].float()) > 0.98
    assert torch.equal(L0.gdn["conv_w"], t[P + "layers.0.self_attn.conv1d.weight"].float().reshape(-1, 4))
    assert torch.equal(L0.gdn["kda"].A_log, t[P + "layers.0.self_attn.A_log"]) and L0.gdn["kda"].dt_bias.numel() == d.n_v * d.dk
    L1 = m.layers[1]
    assert torch.equal(L1.dsa.proj.weight[:128].cpu(), t[P + "layers.1.self_attn.indexer.wk.weight"])
    assert torch.equal(L1.attn_hc[0], t[P + "layers.1.hc_attn_fn"]) and L1.mlp_hc[1].shape == (24,)
    assert L1.w_uk.shape == (4, 192, 512) and L1.w_uv.shape == (4, 256, 512)
    out, _ = Engine(m, m.make_cache(16, 1, 256), use_graphs=False, prefill_chunk=16).generate(list(range(3, 40)), 4)
    assert len(out) == 4
    # chunked prefill + decode against one whole prefill of the same tokens
    m.gdn_states = None
    nxt = Engine(m, m.make_cache(16, 1, 256), use_graphs=False, prefill_chunk=1000).prefill(0, list(range(3, 40)) + out[:2])
    assert nxt == out[2]

    class Rank1(LocalComm):
        rank, size = 1, 2
    m1 = load_glm5_checkpoint(hf, TensorSource(tmp_path), "cpu", Rank1())
    d1 = m1.dims
    assert d1.n_k == 2 and m1.heads == 2
    w1 = m1.layers[0].gdn["in_proj"].dequant() if hasattr(m1.layers[0].gdn["in_proj"], "dequant") else m1.layers[0].gdn["in_proj"].weight.float()
    h = d1.n_k * d1.dk
    assert cos(w1[:h], q[h:2 * h]) > 0.99 and cos(w1[h:2 * h], k[h:2 * h]) > 0.99
    conv = t[P + "layers.0.self_attn.conv1d.weight"].float().reshape(-1, 4)
    assert torch.equal(m1.layers[0].gdn["conv_w"], torch.cat([conv[h:2 * h], conv[n + h:n + 2 * h], conv[2 * n + h:2 * n + 2 * h]], 0))
    assert torch.equal(m1.layers[0].gdn["kda"].A_log, t[P + "layers.0.self_attn.A_log"][2:4])
    assert m1.layers[0].gdn["out_proj"].in_features == h if hasattr(m1.layers[0].gdn["out_proj"], "in_features") else True


@pytest.mark.gpu
def test_gpu_glm5_matches_cpu_statement_and_whole_prefill():
    dev = torch.device("cuda:0")
    cfg, m = _model(dev, residual="hc", dsa=True)
    prompt = torch.randint(0, cfg.vocab, (150,), generator=torch.Generator().manual_seed(0)).tolist()
    eng = Engine(m, m.make_cache(16, 2, 512), use_graphs=True, prefill_chunk=64)
    t1 = eng.prefill(0, prompt)
    h1 = m.last_hidden[-1].float().cpu()
    out, _ = eng.generate(prompt, 8, slot=1)
    assert len(out) == 8 and out[0] == t1
    m.gdn_states = None
    m.dsa_states = {}
    Engine(m, m.make_cache(16, 2, 512), use_graphs=False, prefill_chunk=1000).prefill(0, prompt)
    h2 = m.last_hidden[-1].float().cpu()
    assert torch.nn.functional.cosine_similarity(h1, h2, dim=0) > 0.995
    from volta_engine_b200.models.util import to_device
    mc = to_device(m, "cpu")
    mc.gdn_states = None
    mc.dsa_states = {}
    Engine(mc, mc.make_cache(16, 2, 512), use_graphs=False, prefill_chunk=1000).prefill(0, prompt)
    assert torch.nn.functional.cosine_similarity(mc.last_hidden[-1].float(), h2, dim=0) > 0.98


@pytest.mark.gpu
def test_gpu_glm5_checkpoint_with_the_published_head_shapes_matches_the_cpu_statement(tmp_path):
    """A checkpoint directory with 192 + 64 query dims and 256 value dims per latent-attention head (the published head
    shape) loaded on the device: chunked prefill + decode agree with the CPU statement of the same tensors."""
    from volta_engine_b200.models.factory import load_model
    from volta_engine_b200.models.glm5_loader import save_glm5_checkpoint
    from volta_engine_b200.models.util import to_device
    cfg = Glm5NextConfig.tiny_glm5(residual="hc", dsa=True, mtp_layers=1, qk_nope=192, v_head_dim=256, gdn_k_heads=4, gdn_v_heads=4,
                                   expert_ffn=256, shared_ffn=256)
    save_glm5_checkpoint(tmp_path, cfg, seed=2)
    m, _ = load_model(tmp_path, device="cuda:0")
    prompt = torch.randint(0, cfg.vocab, (150,), generator=torch.Generator().manual_seed(0)).tolist()
    eng = Engine(m, m.make_cache(16, 2, 512), use_graphs=True, prefill_chunk=64)
    out, _ = eng.generate(prompt, 6, slot=1)
    h1 = m.last_hidden[-1].float().cpu()
    assert len(out) == 6
    mc = to_device(m, "cpu")
    mc.gdn_states = None
    mc.dsa_states = {}
    Engine(mc, mc.make_cache(16, 2, 512), use_graphs=False, prefill_chunk=1000).prefill(0, prompt + out[:5])
    assert torch.nn.functional.cosine_similarity(mc.last_hidden[-1].float(), h1, dim=0) > 0.98


@pytest.mark.gpu
def test_gpu_glm5_mtp_rounds_match_plain_greedy():
    """MTP rounds (draft chain through the head's latent-attention block, journalled verify block, rollback of the KDA
    state) emit what plain greedy decoding emits. A verify block of four rows and a single decode row take different
    kernels, so where the plain model's two best logits are closer than 0.02 the two may legitimately part ways: the
    sequences must agree up to the first such near tie."""
    from volta_engine_b200.runtime.mtp_runner import MtpRunner
    dev = torch.device("cuda:0")
    cfg, m = _model(dev, mtp_layers=1)
    prompt = torch.randint(0, cfg.vocab, (77,), generator=torch.Generator().manual_seed(4)).tolist()

    def fresh():
        m.gdn_states = None
        return Engine(m, m.make_cache(16, 2, 512), prefill_chunk=64)
    e = fresh()
    plain, gaps, pos = [e.prefill(0, prompt)], [], len(prompt)
    for _ in range(20):
        c = e.step_candidates([plain[-1]], [pos], [0])[0]
        v = sorted(c.logits, reverse=True)
        plain.append(c.ids[max(range(len(c.ids)), key=lambda i: c.logits[i])])
        gaps.append(v[0] - v[1])
        pos += 1
    eng = fresh()
    run = MtpRunner(eng, depth=3)
    assert run._device_round_ok()
    eng.kv.reserve(0, len(prompt) + 40)
    out, pos = [run.prefill_rows(0, prompt, 0, len(prompt), True)], len(prompt)
    while len(out) < 20:
        new = run.round(0, out[-1], pos)
        out += new
        pos += len(new)
    div = next((i for i in range(20) if out[i] != plain[i]), None)
    assert div is None or (div > 0 and gaps[div - 1] < 0.02), (div, out, plain, gaps)
    assert div is None or div >= 4
    assert run.stats["rounds"] > 0 and run._sts[(1, 3)]["graph"] is not None
