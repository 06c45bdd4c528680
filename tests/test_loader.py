"""Checkpoint containers and the model factory: safetensors (sharded, sliced, quantised dialects), GGUF files,
and a model directory round trip through ``load_model``."""
import json
import re

import pytest
import torch

from volta_engine_b200.loader.gguf_file import GGUFFile, hf_name, unpermute_rope_rows, write_gguf
from volta_engine_b200.loader.safetensors import SafeTensorsRepo, write_safetensors
from volta_engine_b200.models.dense import DenseConfig
from volta_engine_b200.models.factory import load_model, save_dense_checkpoint
from volta_engine_b200.quant import gguf as gq, nvfp4 as qn
from volta_engine_b200.runtime.engine import Engine
from volta_engine_b200.runtime.kv_cache import PagedKVCache


def test_safetensors_roundtrip_slices_and_padding(tmp_path):
    g = torch.Generator().manual_seed(0)
    a = torch.randn(8, 12, generator=g).to(torch.bfloat16)
    b = torch.randint(-30000, 30000, (4, 2, 32), generator=g, dtype=torch.int32).to(torch.int16)
    emb = torch.randn(1000, 16, generator=g).to(torch.float16)
    write_safetensors(tmp_path / "model-00001-of-00002.safetensors", {"a": a, "b.trellis": b}, unsigned16=("b.trellis",))
    write_safetensors(tmp_path / "model-00002-of-00002.safetensors", {"emb": emb}, metadata={"format": "pt"})
    repo = SafeTensorsRepo(tmp_path)
    assert set(repo.names()) == {"a", "b.trellis", "emb"}
    assert torch.equal(repo.load("a"), a) and torch.equal(repo.load("b.trellis"), b)
    assert torch.equal(repo.load_slice("a", 1, 2, 3), a[:, 8:12])
    assert torch.equal(repo.load_slice("a", 0, 1, 2), a[4:8])
    with pytest.raises(ValueError):
        repo.load_slice("a", 1, 0, 5)
    sh = repo.load_rows_padded("emb", 3, 4, 256)
    assert sh.shape == (256, 16) and torch.equal(sh[:232], emb[768:]) and float(sh[232:].abs().sum()) == 0.0


def test_nvfp4_dialects_and_tp_slices_agree(tmp_path):
    g = torch.Generator().manual_seed(1)
    w = torch.randn(64, 128, generator=g) * 0.05
    p, s, gs = qn.quantize_nvfp4(w)
    write_safetensors(tmp_path / "m.safetensors", {
        "x.weight_packed": p, "x.weight_scale": s.view(torch.float8_e4m3fn), "x.weight_global_scale": torch.tensor([1 / gs]),
        "y.weight": p, "y.weight_scale": s.view(torch.float8_e4m3fn), "y.weight_scale_2": torch.tensor([gs]),
        "z.weight": w.to(torch.bfloat16)})
    repo = SafeTensorsRepo(tmp_path)
    assert [repo.linear_kind(n) for n in "xyz"] == ["nvfp4_ct", "nvfp4_mo", "dense"]
    ref = qn.dequantize_nvfp4(p, s, gs)
    lx, ly = repo.load_linear("x"), repo.load_linear("y")
    assert torch.allclose(qn.dequantize_nvfp4(lx.packed, lx.scales, lx.gscale), ref, rtol=1e-6)
    assert torch.allclose(qn.dequantize_nvfp4(ly.packed, ly.scales, ly.gscale), ref, rtol=1e-6)
    x = torch.randn(3, 128, generator=g)
    full = lx.forward(x)
    cols = torch.cat([repo.load_linear("x", "col", r, 2).forward(x) for r in range(2)], -1)
    rows = sum(repo.load_linear("x", "row", r, 2).forward(x[:, r * 64:(r + 1) * 64]) for r in range(2))
    assert torch.allclose(cols, full, atol=1e-5) and torch.allclose(rows, full, atol=1e-4)
    zq = repo.load_linear("z", quantize="nvfp4")
    assert zq.packed.shape == (64, 64)


def test_exl3_linear_loads_and_slices_keep_hadamard_spans(tmp_path):
    from volta_engine_b200.quant import exl3 as ex
    g = torch.Generator().manual_seed(2)
    codes, suh, svh = ex.synth_linear(256, 256, 3, 0.05, g)
    write_safetensors(tmp_path / "m.safetensors", {"l.trellis": codes, "l.suh": suh, "l.svh": svh,
                                                  "l.mcg": torch.zeros(1, dtype=torch.int32)}, unsigned16=("l.trellis",))
    repo = SafeTensorsRepo(tmp_path)
    lin = repo.load_linear("l")
    assert (lin.bits, lin.cb) == (3, ex.CB_MCG)
    x = torch.randn(2, 256, generator=g)
    full = lin.forward(x, out_f32=True)
    cols = torch.cat([repo.load_linear("l", "col", r, 2).forward(x, out_f32=True) for r in range(2)], -1)
    rows = sum(repo.load_linear("l", "row", r, 2).forward(x[:, r * 128:(r + 1) * 128], out_f32=True) for r in range(2))
    assert torch.allclose(cols, full, atol=1e-4) and torch.allclose(rows, full, atol=1e-3)
    with pytest.raises(ValueError):
        repo.load_linear("l", "col", 0, 4)          # 64-wide slices would cut a 128-wide rotation


def test_gguf_file_roundtrip_and_name_map(tmp_path):
    g = torch.Generator().manual_seed(3)
    w = torch.randn(32, 64, generator=g)
    q8 = gq.quantize(w, gq.GGML_Q8_0)
    norm = torch.ones(64)
    write_gguf(tmp_path / "m.gguf", {"general.architecture": "qwen3", "qwen3.block_count": 1, "tokenizer.ggml.tokens": ["a", "b"],
                                     "general.alignment": 32, "x.scale": 0.5},
               {"blk.0.attn_q.weight": (q8, gq.GGML_Q8_0, (32, 64)), "output_norm.weight": (norm, 0, (64,)),
                "token_embd.weight": (w.to(torch.float16), 1, (32, 64))})
    f = GGUFFile(tmp_path / "m.gguf")
    assert f.arch == "qwen3" and f.metadata["qwen3.block_count"] == 1 and f.metadata["tokenizer.ggml.tokens"] == ["a", "b"]
    assert abs(f.metadata["x.scale"] - 0.5) < 1e-7
    assert f.tensors["blk.0.attn_q.weight"].shape == (32, 64)
    assert torch.equal(f.load("blk.0.attn_q.weight"), q8.reshape(32, -1))
    assert torch.allclose(f.dequantize("blk.0.attn_q.weight"), gq.dequantize(q8, gq.GGML_Q8_0, 64).reshape(32, 64))
    assert torch.equal(f.load("token_embd.weight"), w.to(torch.float16))
    assert hf_name("blk.7.ffn_down.weight") == "model.layers.7.mlp.down_proj.weight"
    assert hf_name("output.weight") == "lm_head.weight" and hf_name("rope_freqs.weight") is None
    # the converter permutation interleaves the two rotary halves of every head; the inverse restores them
    hd, nh = 8, 2
    orig = torch.arange(nh * hd * 3.0).reshape(nh * hd, 3)
    perm = orig.reshape(nh, 2, hd // 2, 3).transpose(1, 2).reshape(nh * hd, 3)
    assert torch.equal(unpermute_rope_rows(perm, nh), orig)


@pytest.mark.parametrize("fmt", ["bf16", "nvfp4", "nvfp4_modelopt", "exl3"])
def test_model_directory_roundtrip(tmp_path, fmt):
    cfg = DenseConfig(n_layers=2, hidden=256, n_q=4, n_kv=2, head_dim=64, ffn=512, vocab=512, qk_norm=True)
    save_dense_checkpoint(tmp_path, cfg, seed=4, fmt=fmt, std=0.05)
    model, hf = load_model(tmp_path, "cpu")
    assert hf["model_type"] == "qwen3" and model.cfg.qk_norm and len(model.layers) == 2
    kv = PagedKVCache(cfg.n_layers, model.nkv, cfg.head_dim, 8, 2, 256, "cpu")
    out, st = Engine(model, kv, use_graphs=False, prefill_chunk=32).generate(list(range(40)), 4)
    assert len(out) == 4 and all(0 <= t < cfg.vocab for t in out)
    # loading the same directory twice is deterministic
    model2, _ = load_model(tmp_path, "cpu")
    kv2 = PagedKVCache(cfg.n_layers, model2.nkv, cfg.head_dim, 8, 2, 256, "cpu")
    out2, _ = Engine(model2, kv2, use_graphs=False, prefill_chunk=64).generate(list(range(40)), 4)
    assert out2 == out


def test_unknown_model_type_is_refused(tmp_path):
    (tmp_path / "config.json").write_text(json.dumps({"model_type": "not_a_model"}))
    write_safetensors(tmp_path / "m.safetensors", {"a": torch.zeros(1)})
    with pytest.raises(NotImplementedError):
        load_model(tmp_path, "cpu")


def _moe_dir(tmp_path, mla: bool):
    g = torch.Generator().manual_seed(7)
    H, E, I, V, hd = 256, 4, 128, 512, 64
    hf = {"model_type": "deepseek_v3" if mla else "qwen3_moe", "num_hidden_layers": 2, "hidden_size": H,
          "num_attention_heads": 4, "num_key_value_heads": 2, "head_dim": hd, "intermediate_size": 256,
          "moe_intermediate_size": I, "vocab_size": V, "num_experts_per_tok": 2, "rms_norm_eps": 1e-6,
          "first_k_dense_replace": 1 if mla else 0}
    hf.update({"n_routed_experts": E, "n_shared_experts": 1, "scoring_func": "sigmoid", "routed_scaling_factor": 2.5,
               "q_lora_rank": 128, "kv_lora_rank": 512, "qk_nope_head_dim": 64, "qk_rope_head_dim": 64, "v_head_dim": 64,
               "n_group": 2, "topk_group": 1} if mla else {"num_experts": E})
    (tmp_path / "config.json").write_text(json.dumps(hf))
    t = {}
    rnd = lambda *s: (torch.randn(*s, generator=g) * 0.05).to(torch.bfloat16)
    t["model.embed_tokens.weight"], t["lm_head.weight"], t["model.norm.weight"] = rnd(V, H), rnd(V, H), torch.ones(H).bfloat16()
    for li in range(2):
        p = f"model.layers.{li}."
        t[p + "input_layernorm.weight"] = t[p + "post_attention_layernorm.weight"] = torch.ones(H).bfloat16()
        if mla:
            t[p + "self_attn.q_a_proj.weight"], t[p + "self_attn.q_a_layernorm.weight"] = rnd(128, H), torch.ones(128).bfloat16()
            t[p + "self_attn.kv_a_proj_with_mqa.weight"], t[p + "self_attn.kv_a_layernorm.weight"] = rnd(576, H), torch.ones(512).bfloat16()
            t[p + "self_attn.q_b_proj.weight"], t[p + "self_attn.kv_b_proj.weight"] = rnd(4 * 128, 128), rnd(4 * 128, 512)
            t[p + "self_attn.o_proj.weight"] = rnd(H, 4 * 64)
        else:
            for n, rows in (("q", 4 * hd), ("k", 2 * hd), ("v", 2 * hd)):
                t[p + f"self_attn.{n}_proj.weight"] = rnd(rows, H)
            t[p + "self_attn.o_proj.weight"] = rnd(H, 4 * hd)
            t[p + "self_attn.q_norm.weight"] = t[p + "self_attn.k_norm.weight"] = torch.ones(hd).bfloat16()
        if mla and li == 0:
            t[p + "mlp.gate_proj.weight"], t[p + "mlp.up_proj.weight"], t[p + "mlp.down_proj.weight"] = rnd(256, H), rnd(256, H), rnd(H, 256)
            continue
        t[p + "mlp.gate.weight"] = rnd(E, H)
        if mla:
            t[p + "mlp.gate.e_score_correction_bias"] = torch.zeros(E)
            for n, shp in (("gate", (I, H)), ("up", (I, H)), ("down", (H, I))):
                t[p + f"mlp.shared_experts.{n}_proj.weight"] = rnd(*shp)
        for e in range(E):
            for n, shp in (("gate", (I, H)), ("up", (I, H)), ("down", (H, I))):
                t[p + f"mlp.experts.{e}.{n}_proj.weight"] = rnd(*shp)
    write_safetensors(tmp_path / "model.safetensors", t)
    return hf


@pytest.mark.parametrize("mla", [False, True])
def test_moe_family_directories_load_and_generate(tmp_path, mla):
    _moe_dir(tmp_path, mla)
    model, hf = load_model(tmp_path, "cpu")
    cfg = model.cfg
    assert cfg.n_experts == 4 and cfg.top_k == 2 and (cfg.router == "sigmoid") == mla
    assert model.layers[0].dense_ffn == mla and not model.layers[1].dense_ffn
    kv = PagedKVCache(cfg.n_layers, model.nkv, cfg.head_dim, 8, 2, 256, "cpu",
                      **({"v_head_dim": 0} if mla else {}))
    out, _ = Engine(model, kv, use_graphs=False, prefill_chunk=16).generate(list(range(20)), 3)
    assert len(out) == 3


def test_gguf_model_directory_loads_and_matches_the_safetensors_twin(tmp_path):
    """The same random weights stored as bf16 safetensors and as a GGUF file (Q8_0 linears, F32 norms, llama.cpp tensor
    names) give the same first token; the GGUF linears stay block-quantised in memory."""
    cfg = DenseConfig(n_layers=2, hidden=256, n_q=4, n_kv=2, head_dim=64, ffn=512, vocab=512, qk_norm=True)
    st_dir, gg_dir = tmp_path / "st", tmp_path / "gg"
    save_dense_checkpoint(st_dir, cfg, seed=9, fmt="bf16", std=0.05)
    repo = SafeTensorsRepo(st_dir)
    gg_dir.mkdir()
    (gg_dir / "config.json").write_text((st_dir / "config.json").read_text())
    inv = {"input_layernorm": "attn_norm", "post_attention_layernorm": "ffn_norm", "self_attn.q_proj": "attn_q",
           "self_attn.k_proj": "attn_k", "self_attn.v_proj": "attn_v", "self_attn.o_proj": "attn_output",
           "self_attn.q_norm": "attn_q_norm", "self_attn.k_norm": "attn_k_norm", "mlp.gate_proj": "ffn_gate",
           "mlp.up_proj": "ffn_up", "mlp.down_proj": "ffn_down"}
    tensors = {}
    for name in repo.names():
        t = repo.load(name).float()
        if name.startswith("model.layers."):
            _, _, li, rest = name.split(".", 3)
            inner, kind = rest.rsplit(".", 1)
            gname = f"blk.{li}.{inv[inner]}.{kind}"
        else:
            gname = {"model.embed_tokens.weight": "token_embd.weight", "model.norm.weight": "output_norm.weight",
                     "lm_head.weight": "output.weight"}[name]
        if t.dim() == 2 and "embd" not in gname and gname != "output.weight":
            tensors[gname] = (gq.quantize(t, gq.GGML_Q8_0), gq.GGML_Q8_0, tuple(t.shape))
        else:
            tensors[gname] = (t.contiguous(), 0, tuple(t.shape))
    write_gguf(gg_dir / "model.gguf", {"general.architecture": "qwen3", "qwen3.block_count": 2}, tensors)
    mg, _ = load_model(gg_dir, "cpu")
    ms, _ = load_model(st_dir, "cpu")
    assert type(mg.layers[0].qkv).__name__ in ("LinearGroup", "LinearGGUF")
    outs = []
    for m in (mg, ms):
        kv = PagedKVCache(cfg.n_layers, m.nkv, cfg.head_dim, 8, 2, 256, "cpu")
        outs.append(Engine(m, kv, use_graphs=False, prefill_chunk=32).generate(list(range(30)), 3)[0])
    assert outs[0][0] == outs[1][0]


def test_ngram_table_hashing_and_the_three_row_formats(tmp_path):
    import numpy as np
    from volta_engine_b200.loader.ngram_table import ROW_DIM, NgramTable, encode_trellis_row
    from volta_engine_b200.quant import exl3 as qx
    rng = np.random.default_rng(0)
    ngram, hpn = 3, 2
    sizes = np.array([11, 13, 17, 19], dtype=np.int64)
    offs = np.concatenate([[0], np.cumsum(sizes)[:-1]]).astype(np.int64)
    mult = np.array([0x9E3779B97F4A7C15 - (1 << 64), 1000003, -7046029254386353131], dtype=np.int64)
    total = int(sizes.sum())
    # trellis form: random rings decode to codebook values; scale and per-head bias on top
    K = 6
    cb = qx.decode_windows(torch.arange(65536), qx.CB_MUL1).numpy()
    rows = np.zeros((total, 1 + ROW_DIM * K // 16), dtype=np.uint16)
    plain = np.zeros((total, ROW_DIM), dtype=np.float32)
    for r in range(total):
        words, vals = encode_trellis_row(np.zeros(ROW_DIM), K, cb, rng)
        rows[r, 0] = np.float16(0.5 + 0.01 * r).view(np.uint16)
        rows[r, 1:] = words
        plain[r] = vals * np.float32(np.float16(0.5 + 0.01 * r))
    bias = (torch.randn(4, ROW_DIM) * 0.1).to(torch.float16)
    write_safetensors(tmp_path / "ngram.safetensors", {
        "t.head_offsets": torch.from_numpy(offs), "t.head_vocab_sizes": torch.from_numpy(sizes),
        "t.layer_multipliers": torch.from_numpy(mult), "t.head_bias": bias,
        "t.shard_0.trellis": torch.from_numpy(rows[:30].view(np.int16)), "t.shard_1.trellis": torch.from_numpy(rows[30:].view(np.int16)),
    }, metadata={"K": str(K)})
    t = NgramTable.open_trellis(tmp_path / "ngram.safetensors")
    assert (t.ngram_size, t.heads_per_ngram, t.num_heads, t.rows_per_shard) == (3, 2, 4, 30)
    # hashing: wrapping int64 products, xor over the n-gram, non-negative remainder
    toks = [151643, 77, 123456789]
    M = (1 << 64)
    p = [(toks[i] * int(mult[i])) % M for i in range(3)]
    s64 = lambda v: v - M if v >= (1 << 63) else v
    mixed2, mixed3 = s64(p[0] ^ p[1]), s64(p[0] ^ p[1] ^ p[2])
    want = [mixed2 % 11 + 0, mixed2 % 13 + 11, mixed3 % 17 + 24, mixed3 % 19 + 41]
    ids = t.row_ids(toks)
    assert ids.tolist() == want
    for h in range(4):
        got = t.decode_row(ids[h], h)
        assert np.allclose(got, plain[ids[h]] + bias[h].float().numpy(), atol=1e-6)
    assert t.lookup(toks).shape == (4 * ROW_DIM,)
    seq = t.lookup_sequence([5, 6, 2, 7, 8], eos_id=2)
    assert seq.shape == (5, 4 * ROW_DIM)
    assert torch.equal(seq[3], torch.from_numpy(t.lookup([7, 2, 2])))       # history stops at the eos before position 3
    # fp8 form
    codes = torch.randint(0, 120, (total, ROW_DIM), dtype=torch.uint8)
    write_safetensors(tmp_path / "fp8.safetensors", {
        "m.ngram_heads_offsets": torch.from_numpy(offs), "m.ngram_heads_vocab_sizes": torch.from_numpy(sizes),
        "m.layer_multipliers": torch.from_numpy(mult), "m.ngram_embedding.weight_scale": torch.tensor([0.25], dtype=torch.bfloat16),
        "m.ngram_embedding.shard_0.weight": codes.view(torch.float8_e4m3fn)})
    f = NgramTable.open_fp8(SafeTensorsRepo(tmp_path / "fp8.safetensors"), "m")
    assert f.row_ids(toks).tolist() == want
    assert np.allclose(f.decode_row(7, 0), qn.e4m3_decode(codes[7]).float().numpy() * 0.25)
    # gguf form (IQ4_NL rows)
    dense = torch.randn(total, ROW_DIM) * 0.05
    raw = gq.quantize(dense, gq.GGML_IQ4_NL)
    write_gguf(tmp_path / "t.gguf", {"general.architecture": "qwen4exp", "qwen4exp.ple.head_offsets": offs.tolist(),
                                     "qwen4exp.ple.head_vocab_sizes": sizes.tolist(), "qwen4exp.ple.layer_multipliers": mult.tolist(),
                                     "qwen4exp.ple.ngram_size": 3, "qwen4exp.ple.heads_per_ngram": 2},
               {"per_layer_token_embd.weight": (raw, gq.GGML_IQ4_NL, (total, ROW_DIM))})
    gt = NgramTable.open_gguf(GGUFFile(tmp_path / "t.gguf"), "per_layer_token_embd.weight")
    assert gt.row_ids(toks).tolist() == want
    assert np.allclose(gt.decode_row(9, 0), gq.dequantize(raw[9:10], gq.GGML_IQ4_NL, ROW_DIM)[0].numpy())


@pytest.mark.parametrize("mla", [False, True])
def test_moe_gguf_file_with_stacked_experts_keeps_the_blocks_and_matches_its_safetensors_twin(tmp_path, mla):
    """The MoE / MLA test model as a GGUF file in llama.cpp's layout (experts of a layer stacked in ffn_*_exps, Q8_0 blocks;
    dense tensors F32): the routed experts stay GGUF blocks in memory (GGUFExpertBank) and the model gives the
    safetensors twin's first token."""
    from volta_engine_b200.ops.moe_gguf import GGUFExpertBank
    st_dir, gg_dir = tmp_path / "st", tmp_path / "gg"
    st_dir.mkdir()
    gg_dir.mkdir()
    hf = _moe_dir(st_dir, mla)
    (gg_dir / "config.json").write_text((st_dir / "config.json").read_text())
    repo = SafeTensorsRepo(st_dir)
    inv = {"input_layernorm": "attn_norm", "post_attention_layernorm": "ffn_norm", "self_attn.q_proj": "attn_q",
           "self_attn.k_proj": "attn_k", "self_attn.v_proj": "attn_v", "self_attn.o_proj": "attn_output",
           "self_attn.q_norm": "attn_q_norm", "self_attn.k_norm": "attn_k_norm", "mlp.gate_proj": "ffn_gate",
           "mlp.up_proj": "ffn_up", "mlp.down_proj": "ffn_down", "mlp.gate": "ffn_gate_inp",
           "mlp.gate.e_score_correction_bias": "exp_probs_b", "self_attn.q_a_proj": "attn_q_a", "self_attn.q_b_proj": "attn_q_b",
           "self_attn.q_a_layernorm": "attn_q_a_norm", "self_attn.kv_a_proj_with_mqa": "attn_kv_a_mqa",
           "self_attn.kv_b_proj": "attn_kv_b", "self_attn.kv_a_layernorm": "attn_kv_a_norm",
           "mlp.shared_experts.gate_proj": "ffn_gate_shexp", "mlp.shared_experts.up_proj": "ffn_up_shexp",
           "mlp.shared_experts.down_proj": "ffn_down_shexp"}
    tensors, stacks = {}, {}
    for name in repo.names():
        t = repo.load(name).float()
        if name.startswith("model.layers."):
            _, _, li, rest = name.split(".", 3)
            m = re.match(r"mlp\.experts\.(\d+)\.(gate|up|down)_proj\.weight$", rest)
            if m:
                stacks.setdefault((li, m.group(2)), {})[int(m.group(1))] = t
                continue
            if rest == "mlp.gate.e_score_correction_bias":
                tensors[f"blk.{li}.exp_probs_b.bias"] = (t.contiguous(), 0, tuple(t.shape))
                continue
            inner, kind = rest.rsplit(".", 1)
            tensors[f"blk.{li}.{inv[inner]}.{kind}"] = (t.contiguous(), 0, tuple(t.shape))
        else:
            gname = {"model.embed_tokens.weight": "token_embd.weight", "model.norm.weight": "output_norm.weight",
                     "lm_head.weight": "output.weight"}[name]
            tensors[gname] = (t.contiguous(), 0, tuple(t.shape))
    for (li, which), per in stacks.items():
        full = torch.stack([per[e] for e in range(len(per))])                       # [E, rows, cols]
        raw = gq.quantize(full.reshape(-1, full.shape[-1]), gq.GGML_Q8_0)
        tensors[f"blk.{li}.ffn_{which}_exps.weight"] = (raw, gq.GGML_Q8_0, tuple(full.shape))
    arch = "deepseek2" if mla else "qwen3moe"
    write_gguf(gg_dir / "model.gguf", {"general.architecture": arch, f"{arch}.block_count": 2}, tensors)
    mg, _ = load_model(gg_dir, "cpu")
    ms, _ = load_model(st_dir, "cpu")
    moe_layer = mg.layers[1]
    assert isinstance(moe_layer.bank, GGUFExpertBank) and moe_layer.bank.gu_type == gq.GGML_Q8_0
    assert moe_layer.bank.gu_raw.shape[:2] == (4, 2 * mg.cfg.expert_ffn)
    from volta_engine_b200.runtime.batch import BatchRows
    rows = []
    for m in (mg, ms):
        kv = PagedKVCache(m.cfg.n_layers, m.nkv, m.cfg.head_dim, 8, 2, 256, "cpu", **({"v_head_dim": 0} if mla else {}))
        kv.reserve(0, 32)
        b = BatchRows.make(list(range(20)), list(range(20)), [0] * 20, "cpu", "last", max(1, m.nq // m.nkv), prefill=True)
        rows.append(m.forward(b, kv).float().flatten())
    # the twin holds every linear as NVFP4 (4-bit) and this file F32 / Q8_0: the logits agree to that quantisation noise
    c = float(torch.dot(rows[0], rows[1]) / (rows[0].norm() * rows[1].norm()))
    assert c > 0.93, c
    # and the bank holds exactly the file's blocks: expert 2 of layer 1 decodes to the Q8_0 rounding of the source tensors
    src = {w: stacks[("1", w)][2] for w in ("gate", "up", "down")}
    want_gu = gq.dequantize(gq.quantize(torch.cat([src["gate"], src["up"]], 0), gq.GGML_Q8_0), gq.GGML_Q8_0, src["gate"].shape[1])
    assert torch.equal(moe_layer.bank.dequant("gu", 2), want_gu)
    want_dn = gq.dequantize(gq.quantize(src["down"], gq.GGML_Q8_0), gq.GGML_Q8_0, src["down"].shape[1])
    assert torch.equal(moe_layer.bank.dequant("dn", 2), want_dn)


def test_loader_options_take_experts_and_dense_tensors_from_other_directories(tmp_path):
    """nvfp4_experts / nvfp4_expert_layers / nvfp4_dense_dir: an overlay of checkpoints. The experts of layer 1 come from a
    second directory (other weights), a dense tensor from a third; the model then differs from the plain load exactly
    there. nvfp4_dense = head quantises the head."""
    from volta_engine_b200.loader.safetensors import SafeTensorsRepo
    from volta_engine_b200.models.factory import OverlaySource, TensorSource, parse_layer_set
    from volta_engine_b200.ops.linear import LinearBF16
    base, other, dense = tmp_path / "base", tmp_path / "experts", tmp_path / "dense"
    for d in (base, other, dense):
        d.mkdir()
    _moe_dir(base, mla=False)
    repo = SafeTensorsRepo(base)
    g = torch.Generator().manual_seed(99)
    swapped = {n: (torch.randn(repo.load(n).shape, generator=g) * 0.05).to(torch.bfloat16) for n in repo.names() if ".mlp.experts." in n}
    write_safetensors(other / "model.safetensors", swapped)
    o_new = (torch.randn(256, 256, generator=g) * 0.05).to(torch.bfloat16)
    write_safetensors(dense / "model.safetensors", {"model.layers.0.self_attn.o_proj.weight": o_new})
    plain, _ = load_model(base, "cpu")
    mixed, _ = load_model(base, "cpu", overlay={"nvfp4_experts": str(other), "nvfp4_expert_layers": "1", "nvfp4_dense_dir": str(dense)},
                          nvfp4_dense="head")
    assert torch.equal(plain.layers[0].bank.gu_p, mixed.layers[0].bank.gu_p)              # layer 0 experts untouched
    assert not torch.equal(plain.layers[1].bank.gu_p, mixed.layers[1].bank.gu_p)          # layer 1 experts from the other directory
    assert not torch.equal(plain.layers[0].o_proj.packed, mixed.layers[0].o_proj.packed)  # the calibrated dense tensor
    assert torch.equal(plain.layers[1].o_proj.packed, mixed.layers[1].o_proj.packed)
    assert isinstance(plain.lm_head, LinearBF16) and not isinstance(mixed.lm_head, LinearBF16)
    assert mixed.lm_head.nbytes() < plain.lm_head.weight.numel() * 2 / 3
    assert parse_layer_set("3-5,9", 12) == {3, 4, 5, 9} and 7 in parse_layer_set("", 12)
    kv = PagedKVCache(mixed.cfg.n_layers, mixed.nkv, mixed.cfg.head_dim, 8, 2, 256, "cpu")
    out, _ = Engine(mixed, kv, use_graphs=False, prefill_chunk=16).generate(list(range(20)), 3)
    assert len(out) == 3
    via_src, _ = load_model(base, "cpu", overlay={"nvfp4_dense_src": str(dense)})
    assert torch.equal(via_src.layers[0].o_proj.packed, mixed.layers[0].o_proj.packed)    # the same tensor by the other option
    src = OverlaySource(TensorSource(base), [])
    assert src.has("model.norm.weight") and src.repo is not None
