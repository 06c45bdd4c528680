"""Host-side tools: terminal dashboard frames and the HTTP load generator's self-test against its mock server."""
import io
import threading

from volta_engine_b200.server import tui
from volta_engine_b200.tools import bench_serve

STATS = {
    "server": {"model": "m27", "model_type": "dense", "uptime_s": 3723, "slots": 2, "max_context": 32768, "tp": 4,
               "queued": 1, "speculation": True, "speculator": "mtp", "kv_format": "bf16"},
    "totals": {"requests": 12, "completed": 11, "tokens_out": 3456, "tokens_prefilled": 99999, "cached_tokens": 2048},
    "averages": {"ttft_ms": 812.4, "prefill_tok_s": 12839.0, "decode_tok_s": 136.4},
    "latency": {"gap_ms": [7.3, 7.9, 9.1, 15.0, 41.0], "gap_samples": 3400, "ttft_ms": [500, 900, 1500]},
    "speculation": {"rounds": 100, "accept_rate": 0.71, "tokens_per_round": 2.4},
    "history": {"t": list(range(30)), "decode": [i % 7 for i in range(30)], "prefill": [0] * 30, "active": [1] * 30},
    "prefix_cache": {"lookups": 12, "hits": 5, "hit_tokens": 2048, "inserts": 9, "evictions": 1, "entries": 8,
                     "bytes": 1 << 30, "budget_bytes": 4 << 30, "disk": {"hits": 0, "entries": 0, "bytes": 0}},
    "slots": [{"slot": 0, "active": True, "phase": "decode", "req_id": 12, "pos": 16500, "prompt_tokens": 16384,
               "cached_tokens": 0, "generated": 116, "max_tokens": 128, "age_s": 3.2, "decode_tok_s": 135.9},
              {"slot": 1, "active": False, "phase": "idle"}],
    "gpus": [{"index": 0, "name": "NVIDIA B200", "power_w": 612.0, "power_limit_w": 1000.0, "temp_c": 54, "util_gpu": 97,
              "sm_mhz": 1830, "mem_used": 40 << 30, "mem_total": 179 << 30, "throttle": ["sw_power_cap"]}],
    "host": {"cpu_pct": 12.0, "load1": 1.5, "mem_used": 8 << 30, "mem_total": 64 << 30, "rss": 3 << 30},
    "recent": [{"req_id": 11, "prompt_tokens": 16384, "cached_tokens": 2048, "generated": 128, "queue_ms": 1.0,
                "ttft_ms": 1290.0, "total_ms": 2230.0, "decode_tok_s": 136.0, "reason": "length"}],
}


def test_tui_frame_contents_and_width():
    frame = tui.render_frame(STATS, width=120)
    lines = frame.splitlines()
    assert all(len(ln) <= 120 for ln in lines)
    assert "m27 [dense]" in lines[0] and "tp=4" in lines[0] and "up 01:02:03" in lines[0]
    assert "decode 136.4 tok/s" in frame and "accept 71.0%" in frame
    assert "p50 7.3" in frame and "max 41.0" in frame
    assert "prefix cache" in frame and "1.0 GiB / 4.0 GiB" in frame
    assert "sw_power_cap" in frame and "NVIDIA B200" in frame
    assert any(ln.split()[:2] == ["0", "decode"] for ln in lines)
    assert any(ln.split()[:2] == ["1", "idle"] for ln in lines)
    assert tui.spark([0, 1, 2, 4, 8], 5)[-1] == "█" and len(tui.spark(range(100), 10)) == 10
    assert tui.render_frame({}, 60).startswith("volta_top")      # an empty document still renders


def test_tui_loop_survives_an_unreachable_server():
    out = io.StringIO()
    n = tui.run_tui("http://127.0.0.1:9", stop=threading.Event(), interval=0.01, out=out, frames=2)
    assert n == 2 and "volta_top: http://127.0.0.1:9" in out.getvalue()


def test_bench_serve_selftest():
    rep = bench_serve.selftest()
    assert rep["selftest"] == "pass", rep
    assert rep["failed"] == 0 and rep["req_per_s"] > 0 and rep["tok_per_s"] > 0
    assert bench_serve.percentile([1, 2, 3, 4, 5], 0.5) == 3 and bench_serve.percentile([], 0.9) == 0.0


def test_quantize_tool_round_trip(tmp_path):
    import torch
    from volta_engine_b200.models.dense import DenseConfig
    from volta_engine_b200.models.factory import load_model, save_dense_checkpoint
    from volta_engine_b200.runtime.engine import Engine
    from volta_engine_b200.runtime.kv_cache import PagedKVCache
    from volta_engine_b200.tools.quantize import plan, quantize_dir
    from volta_engine_b200.loader.safetensors import SafeTensorsRepo
    cfg = DenseConfig(n_layers=1, hidden=128, n_q=2, n_kv=1, head_dim=64, ffn=256, vocab=300, qk_norm=True)
    src = tmp_path / "src"
    save_dense_checkpoint(src, cfg, seed=3, fmt="bf16", std=0.05)
    pl = plan(SafeTensorsRepo(src), "nvfp4", min_dim=64)
    acts = pl["actions"]
    assert acts["model.layers.0.mlp.down_proj.weight"] == "quantize" and acts["model.embed_tokens.weight"] == "copy"
    assert acts["model.layers.0.input_layernorm.weight"] == "copy" and acts["lm_head.weight"] == "copy"
    ref_model, _ = load_model(src, "cpu")
    kv = PagedKVCache(1, 1, 64, 8, 1, 256, "cpu")
    ref, _ = Engine(ref_model, kv, use_graphs=False, prefill_chunk=32).generate(list(range(24)), 3)
    for fmt in ("nvfp4", "nvfp4_modelopt"):
        dst = tmp_path / fmt
        rep = quantize_dir(src, dst, fmt, min_dim=64, log=lambda *_: None)
        assert rep["quantized"] == 7 and (dst / "config.json").exists() and (dst / "quantization_config.json").exists()
        m, _ = load_model(dst, "cpu")
        assert type(m.layers[0].down).__name__ == "LinearNVFP4"
        kv2 = PagedKVCache(1, 1, 64, 8, 1, 256, "cpu")
        out, _ = Engine(m, kv2, use_graphs=False, prefill_chunk=32).generate(list(range(24)), 3)
        assert len(out) == 3
    # the dequantised weights stay close to the source
    w0 = ref_model.layers[0].down.weight.float()
    wq = m.layers[0].down
    from volta_engine_b200.quant import nvfp4 as qn
    rel = (qn.dequantize_nvfp4(wq.packed, wq.scales, wq.gscale) - w0).norm() / w0.norm()
    assert rel < 0.12


def test_tune_expert_lowers_the_held_out_error_and_matches_exl3_semantics():
    import torch
    from volta_engine_b200.quant import exl3 as ex
    from volta_engine_b200.tools import tune as T
    from volta_engine_b200.train import grad as G
    g = torch.Generator().manual_seed(0)
    H, I, rows = 128, 256, 400
    orig = {"gate": torch.randn(H, I, generator=g) * 0.08, "up": torch.randn(H, I, generator=g) * 0.08,
            "down": torch.randn(I, H, generator=g) * 0.08}
    # a "quantised" expert: the original weights with multiplicative channel noise that scale tuning can undo
    quant = {}
    for n, W in orig.items():
        su = 1.0 + 0.2 * torch.randn(W.shape[0], generator=g)
        sv = 1.0 + 0.2 * torch.randn(W.shape[1], generator=g)
        quant[n] = G.ScaledLinear((W / su[:, None] / sv[None, :]).contiguous(), torch.ones(W.shape[0]), torch.ones(W.shape[1]))
    X = torch.randn(rows, H, generator=g)
    w = torch.rand(rows, generator=g)
    res = T.tune_expert(orig, quant, X, w, steps=60, lr=0.02)
    assert res.err_after < 0.5 * res.err_before and res.best_step > 0
    assert res.train_curve[-1] < res.train_curve[0]
    assert set(res.scales) == {"gate", "up", "down"}
    # the trainable view of an EXL3 tensor computes the same linear map as the kernel-side definition
    codes = ex.random_codes(128, 128, 3, torch.Generator().manual_seed(1))
    suh, svh = torch.rand(128) + 0.5, torch.rand(128) + 0.5
    lin = T.exl3_scaled_linear(codes, 3, suh, svh)
    x = torch.randn(5, 128, generator=g)
    y, _ = G.scaled_linear_forward(lin, x)
    assert torch.allclose(y, ex.linear_reference(x, codes, 3, suh, svh), atol=1e-3, rtol=1e-3)


def test_sessions_tool_builds_message_bodies(tmp_path):
    import json
    from volta_engine_b200.tools import sessions as S
    lines = [
        json.dumps({"type": "system", "message": {"role": "system", "content": "be brief"}}),
        json.dumps({"type": "user", "message": {"role": "user", "content": "hello"}}),
        json.dumps({"type": "user", "message": {"role": "user", "content": [{"type": "text", "text": "again"}]}}),
        json.dumps({"type": "assistant", "isSidechain": True, "message": {"role": "assistant", "content": "side"}}),
        json.dumps({"type": "assistant", "message": {"role": "assistant", "content": [
            {"type": "thinking", "thinking": "hm"}, {"type": "tool_use", "id": "t1", "name": "ls", "input": {"p": "."}}]}}),
        json.dumps({"type": "user", "message": {"role": "user", "content": [{"type": "tool_result", "tool_use_id": "t1", "content": "a b"}]}}),
        "not json",
        json.dumps({"type": "assistant", "message": {"role": "assistant", "content": "x" * 50}}),
        json.dumps({"type": "user", "message": {"role": "user", "content": "tail that is cut"}}),
    ]
    body = S.session_to_body(lines, max_chars=40)
    roles = [m["role"] for m in body["messages"]]
    assert roles == ["user", "assistant", "user", "assistant"] and body["system"] == "be brief"
    assert [b["type"] for b in body["messages"][0]["content"]] == ["text", "text"]           # consecutive user entries joined
    assert body["messages"][1]["content"][1]["name"] == "ls" and body["messages"][2]["content"][0]["type"] == "tool_result"
    p = tmp_path / "s.jsonl"
    p.write_text("\n".join(lines))
    assert S.main(["--out", str(tmp_path / "o"), "--max-chars", "40", str(p)]) == 0
    assert json.loads((tmp_path / "o" / "req_0.json").read_text())["messages"][0]["role"] == "user"
    reqs = S.prompts_to_requests(["a", {"prompt": "b"}], "m", 10)
    assert reqs[1]["messages"][0]["content"] == "b" and reqs[0]["max_tokens"] == 10
    ex = S.exchange_to_body("q", {"choices": [{"message": {"reasoning_content": "r", "content": "c"}}]})
    assert [b["type"] for b in ex["messages"][1]["content"]] == ["thinking", "text"]


def test_e2e_tuning_recovers_perturbed_scales_and_matches_the_engine_forward():
    import torch
    from volta_engine_b200.models.dense import DenseConfig, DenseModel
    from volta_engine_b200.runtime.batch import BatchRows
    from volta_engine_b200.runtime.kv_cache import PagedKVCache
    from volta_engine_b200.tools import e2e as E
    cfg = DenseConfig.tiny(vocab=128)
    cfg.quant = "bf16"
    m = DenseModel(cfg, "cpu").init_random(seed=0)
    teacher = E.build_from_engine_model(m).eval()
    # the training form computes what the engine computes
    ids = torch.randint(1, 120, (24,), generator=torch.Generator().manual_seed(1))
    kv = PagedKVCache(cfg.n_layers, m.nkv, cfg.head_dim, 4, 1, 128, "cpu")
    kv.reserve(0, 64)
    eng = m.forward(BatchRows.make(ids.tolist(), list(range(24)), [0] * 24, "cpu", "all", m.nq // m.nkv, prefill=True), kv)
    with torch.no_grad():
        tl = teacher(ids)
    a, b = eng[:, : cfg.vocab].float().flatten(), tl.flatten()
    assert float(torch.dot(a, b) / (a.norm() * b.norm())) > 0.999
    # student = teacher with perturbed channel scales: tuning brings the held-out KL down
    student = E.build_from_engine_model(m)
    g = torch.Generator().manual_seed(2)
    with torch.no_grad():
        for L in student.layers:
            for lin in (L.qkv, L.o, L.gu, L.dn):
                lin.su.mul_(1.0 + 0.15 * torch.randn(lin.su.shape, generator=g))
                lin.sv.mul_(1.0 + 0.15 * torch.randn(lin.sv.shape, generator=g))
    seqs = [torch.randint(1, 120, (32,), generator=g) for _ in range(5)]
    with torch.no_grad():
        teachers = [teacher(s) for s in seqs]
    o = E.E2EOptions(steps=40, batch=2, lr=0.02, warmup=2, eval_every=20)
    hist = E.tune(student, seqs, teachers, o, held_out=1, log=lambda s: None)
    assert hist["eval"][-1][1] < 0.5 * hist["eval"][0][1]
    assert abs(E.lr_at(0, o) - 0.01) < 1e-9 and abs(E.lr_at(o.steps, o) - 0.002) < 1e-6        # warm-up, then cosine to lr_min
    # two stages: the same numbers with the layers split over two (cpu) devices
    two = E.build_from_engine_model(m, ("cpu", "cpu")).eval()
    assert two.stage == [0, 1] or two.stage[0] == 0
    with torch.no_grad():
        assert torch.allclose(two(ids), tl, atol=1e-5)


def test_hessian_capture_files_ldl_feedback_and_resumable_hessian_aware_quantize(tmp_path):
    import torch
    from volta_engine_b200.models.dense import DenseConfig
    from volta_engine_b200.models.factory import load_model, save_dense_checkpoint
    from volta_engine_b200.runtime.engine import Engine
    from volta_engine_b200.runtime.kv_cache import PagedKVCache
    from volta_engine_b200.ops import hessian as hz
    from volta_engine_b200.quant import ldlq, nvfp4 as qn
    from volta_engine_b200.tools.quantize import quantize_dir
    from volta_engine_b200.loader.safetensors import SafeTensorsRepo
    # capture file round trip; a short or foreign file is refused
    H = torch.randn(32, 32)
    hz.write_hessian(tmp_path / "a.f32", H, 77)
    got = hz.read_hessian(tmp_path / "a.f32")
    assert got[1] == 77 and torch.equal(got[0], H)
    (tmp_path / "bad.f32").write_bytes(b"\0" * 40)
    assert hz.read_hessian(tmp_path / "bad.f32") is None and hz.read_hessian(tmp_path / "none.f32") is None
    assert hz.site_of_tensor("model.layers.7.self_attn.o_proj.weight") == (7, 2)
    assert hz.site_of_tensor("model.layers.3.mlp.up_proj.weight") == (3, 1) and hz.site_of_tensor("lm_head.weight") == (0, 4)
    assert hz.parse_layer_range("2-5", 8) == (2, 6) and hz.parse_layer_range("", 8) == (0, 8)
    # block LDL: exact factorisation, unit diagonal blocks
    g = torch.Generator().manual_seed(0)
    K, N = 256, 128
    X = torch.randn(2048, K, generator=g) @ (torch.randn(K, K, generator=g) * 0.3 + torch.eye(K))
    X[:, :8] *= 6.0
    Hs = X.t() @ X
    Hd = ldlq.damp(Hs)
    L, D = ldlq.block_ldl(Hd, 16)
    assert float((L @ torch.block_diag(*D) @ L.t() - Hd).abs().max() / Hd.abs().max()) < 1e-12
    assert torch.allclose(L[16:32, 16:32], torch.eye(16, dtype=torch.float64)) and float(L[0:16, 16:].abs().max()) == 0.0
    # the feedback lowers the Hessian-metric error below round-to-nearest (which has the lower plain squared error)
    w = torch.randn(N, K, generator=g) * 0.02
    p, s, gs = ldlq.quantize_nvfp4_hessian(w, Hs)
    wq = qn.dequantize_nvfp4(p, s, gs)
    p0, s0, g0 = qn.quantize_nvfp4(w, search=True)
    w0 = qn.dequantize_nvfp4(p0, s0, g0)
    e_ldl, e_rtn = ldlq.proxy_error(w.t(), wq.t(), Hs), ldlq.proxy_error(w.t(), w0.t(), Hs)
    assert e_ldl < 0.85 * e_rtn and ((w0 - w) ** 2).mean() < ((wq - w) ** 2).mean()
    # a model's capture: prefill rows are counted, decode rows are not; the sums are those of the taps
    cfg = DenseConfig(n_layers=2, hidden=128, n_q=2, n_kv=1, head_dim=64, ffn=256, vocab=300)
    src = tmp_path / "src"
    save_dense_checkpoint(src, cfg, seed=3, fmt="bf16", std=0.05)
    model, _ = load_model(src, "cpu")
    hs = model.enable_hessians(layer_range=(0, 2))
    kv = PagedKVCache(2, 1, 64, 8, 1, 256, "cpu")
    Engine(model, kv, use_graphs=False, prefill_chunk=64).generate(list(range(40)), 3)
    cap = tmp_path / "cap"
    files = hs.dump(cap)
    assert "L00_s0_r0.f32" in files and "L01_s3_r0.f32" in files and "L00_s4_r0.f32" in files
    h0, rows = hz.read_hessian(cap / "L00_s0_r0.f32")
    assert rows == 40 and h0.shape == (128, 128) and float(h0.diagonal().min()) > 0
    h3, _ = hz.read_hessian(cap / "L01_s3_r0.f32")
    assert h3.shape == (256, 256)
    # Hessian-aware quantise: proxy errors reported, .partial resumes, the result loads and runs
    dst = tmp_path / "q"
    logs = []
    r1 = quantize_dir(src, dst, "nvfp4", min_dim=64, log=logs.append, hess_dir=cap, only=["layers.0."], assemble=False)
    assert r1["quantized"] == 7 and not r1["shards"] and len(r1["proxy_errors"]) == 7
    assert all(0 < v < 0.05 for v in r1["proxy_errors"].values())
    assert (dst / ".partial" / "model.layers.0.mlp.down_proj.weight.safetensors").exists()
    r2 = quantize_dir(src, dst, "nvfp4", min_dim=64, log=logs.append, hess_dir=cap)
    assert r2["resumed"] == 7 and r2["quantized"] == 14 and len(r2["proxy_errors"]) == 7
    m, _ = load_model(dst, "cpu")
    out, _ = Engine(m, PagedKVCache(2, 1, 64, 8, 1, 256, "cpu"), use_graphs=False, prefill_chunk=64).generate(list(range(24)), 3)
    assert len(out) == 3
    # the Hessian-aware result beats the plain one in the capture's metric
    plain = tmp_path / "plain"
    quantize_dir(src, plain, "nvfp4", min_dim=64, log=lambda *_: None)
    from volta_engine_b200.tools.hess_compare import load_quantized
    base = "model.layers.1.mlp.down_proj"
    W = SafeTensorsRepo(src).load(base + ".weight").float().t()
    assert ldlq.proxy_error(W, load_quantized(dst, base), h3) < ldlq.proxy_error(W, load_quantized(plain, base), h3)


def test_hess_compare_subcommands(tmp_path, capsys):
    import torch
    from volta_engine_b200.ops import hessian as hz
    from volta_engine_b200.loader.safetensors import write_safetensors
    from volta_engine_b200.runtime.route_dump import RouteRecorder
    from volta_engine_b200.tools import hess_compare as hc
    from volta_engine_b200.tools.quantize import quantize_dir
    g = torch.Generator().manual_seed(1)
    K = 128
    Xa = torch.randn(512, K, generator=g)
    Xa[:, :4] *= 5
    Xb = torch.randn(768, K, generator=g)
    Xb[:, 64:68] *= 5
    da, db, dm = tmp_path / "a", tmp_path / "b", tmp_path / "m"
    da.mkdir(); db.mkdir()
    for d, X in ((da, Xa), (db, Xb)):
        hz.write_hessian(d / "L00_s0_r0.f32", X.t() @ X, X.shape[0])
        hz.write_hessian(d / "L00_s1_r0.f32", X.t() @ X * 2, X.shape[0])
    hz.write_hessian(da / "L01_s0_r0.f32", Xa.t() @ Xa, 512)
    st = hc.stats(da, db, out=lambda *_: None)
    assert st["missing"] == 1 and set(st["sites"]) == {"s0", "s1"} and st["sites"]["s0"]["mean"] > 0.3
    same = hc.stats(da, da, out=lambda *_: None)
    assert same["sites"]["s0"]["worst"] == 0 and same["files"][0]["trace"] == 1.0
    assert hz.merge_dirs(dm, [da, db]) == ["L00_s0_r0.f32", "L00_s1_r0.f32"]
    hm, rows = hz.read_hessian(dm / "L00_s0_r0.f32")
    assert rows == 1280 and torch.allclose(hm, Xa.t() @ Xa + Xb.t() @ Xb, rtol=1e-5, atol=1e-3)
    # cross: each Hessian's own quantisation is the best under itself
    src = tmp_path / "src"
    src.mkdir()
    E, H, I = 3, 128, 128
    tensors = {"model.layers.0.self_attn.q_proj.weight": (torch.randn(128, K, generator=g) * 0.03).bfloat16()}
    pre = "model.layers.0.mlp.experts.{expert}.{proj}_proj"
    for e in range(E):
        for p, shape in (("gate", (I, H)), ("up", (I, H)), ("down", (H, I))):
            tensors[pre.format(expert=e, proj=p) + ".weight"] = (torch.randn(*shape, generator=g) * 0.05).bfloat16()
    write_safetensors(src / "model.safetensors", tensors)
    res = hc.cross(src, "model.layers.0.self_attn.q_proj", da / "L00_s0_r0.f32", db / "L00_s0_r0.f32", out=lambda *_: None)
    assert res["A"]["under_A"] < res["B"]["under_A"] and res["B"]["under_B"] < res["A"]["under_B"] and res["ratio"] > 1.0
    # score under a capture: the Hessian-aware checkpoint beats the plain one; a .partial directory is readable
    qa, qp = tmp_path / "qa", tmp_path / "qp"
    quantize_dir(src, qa, "nvfp4", min_dim=64, log=lambda *_: None, hess_dir=da, assemble=False)
    quantize_dir(src, qp, "nvfp4", min_dim=64, log=lambda *_: None)
    tab = hc.score(src, ["model.layers.0.self_attn.q_proj"], [qa, qp], hess_dir=da, out=lambda *_: None)
    row = tab["model.layers.0.self_attn.q_proj"]
    assert 0 < row[0] < row[1]
    # route dump: recorder, busiest experts, expert scores under the activation Hessian, block output error
    rec = RouteRecorder(max_rows=64)
    x = torch.randn(200, H, generator=g).bfloat16()
    ids = torch.stack([torch.randint(0, 2, (200,), generator=g), torch.full((200,), 2)], 1)
    ids[:150, 0] = 0
    w = torch.rand(200, 2, generator=g)
    rec.record(0, x[:8], ids[:8], w[:8])                      # a decode-sized batch is ignored
    rec.record(0, x, ids, w)
    dump = rec.result()
    assert set(dump[0]) == {0, 1, 2} and dump[0][2][0].shape == (64, H) and dump[0][1][0].shape[0] < 64
    r, c = (ids == 1).nonzero(as_tuple=True)
    assert torch.equal(dump[0][1][0], x[r]) and torch.allclose(dump[0][1][1], w[r, c])
    rec.save(tmp_path / "route.pt")
    rt = hc.routes(str(tmp_path / "route.pt"), [0], top=2, prefix="model.layers.{layer}.mlp.experts.{expert}.{proj}_proj",
                   out=lambda *_: None)
    assert [e for e, _ in rt[0]] == [0, 2] or [e for e, _ in rt[0]] == [2, 0]
    names = [pre.format(expert=1, proj=p) for p in ("gate", "down")]
    tab = hc.score(src, names, [qp], route=str(tmp_path / "route.pt"), prefix="model.layers.{layer}.mlp.experts.{expert}.{proj}_proj",
                   out=lambda *_: None)
    assert all(0 < tab[n][0] < 0.05 for n in names)
    mo = hc.moe(src, str(tmp_path / "route.pt"), [0], [qp, src], prefix="model.layers.{layer}.mlp.experts.{expert}.{proj}_proj",
                out=lambda *_: None)
    assert 0 < mo[0]["mean"][0] < 0.1 and mo[0]["mean"][1] == 0.0 and len(mo[0]["experts"][0]) == 3
    # the command line
    assert hc.main(["stats", str(da), str(db)]) == 0
    assert "files in both" in capsys.readouterr().out
    assert hc.main(["merge", str(tmp_path / "m2"), str(da), str(db), "--weights", "0.7,0.3"]) == 0
    h2, rows2 = hz.read_hessian(tmp_path / "m2" / "L00_s0_r0.f32")
    want = (0.7 * (Xa.t() @ Xa) / 512 + 0.3 * (Xb.t() @ Xb) / 768) * 1280
    assert rows2 == 1280 and torch.allclose(h2, want, rtol=1e-4, atol=1e-2)


def test_ppl_tool_scores_calibrates_and_measures_kl(tmp_path, capsys):
    import json
    import torch
    from volta_engine_b200.models.dense import DenseConfig
    from volta_engine_b200.models.factory import save_dense_checkpoint
    from volta_engine_b200.ops import hessian as hz
    from volta_engine_b200.tools import ppl
    from volta_engine_b200.tools.quantize import quantize_dir
    cfg = DenseConfig(n_layers=2, hidden=128, n_q=2, n_kv=1, head_dim=64, ffn=256, vocab=300)
    src = tmp_path / "src"
    save_dense_checkpoint(src, cfg, seed=5, fmt="bf16", std=0.08)
    g = torch.Generator().manual_seed(2)
    seqs = [torch.randint(0, 300, (n,), generator=g, dtype=torch.int32) for n in (70, 45)]
    torch.save(seqs, tmp_path / "tok.pt")
    cap, teacher = tmp_path / "cap", tmp_path / "teacher.pt"
    rc = ppl.main(["--model", str(src), "--tokens-file", str(tmp_path / "tok.pt"), "--chunk", "32", "--device", "cpu",
                   "--calibrate", "--hessian-dir", str(cap), "--hessian-layers", "1-1", "--topk-out", str(teacher),
                   "--topk", "8", "--inputs-out", str(tmp_path / "inputs.pt")])
    out = json.loads(capsys.readouterr().out.strip().splitlines()[-1])
    assert rc == 0 and out["tokens"] == 113 and 100 < out["ppl"] < 900          # random weights: near the vocabulary size
    files = sorted(f.name for f in cap.iterdir())
    assert files == ["L00_s4_r0.f32", "L01_s0_r0.f32", "L01_s1_r0.f32", "L01_s2_r0.f32", "L01_s3_r0.f32"]
    assert hz.read_hessian(cap / "L01_s1_r0.f32")[1] == 32 + 32 + 32       # whole chunks only: 6- and 13-row tails are decode-sized
    t = torch.load(teacher, weights_only=True)
    assert t["k"] == 8 and t["ids"][0].shape == (70, 8) and t["tail"][1].shape == (45,)
    assert torch.allclose(t["logp"][0].exp().sum(-1) + t["tail"][0].exp(), torch.ones(70), atol=1e-4)
    assert [len(s) for s in torch.load(tmp_path / "inputs.pt", weights_only=True)] == [70, 45]
    # the model against its own teacher: zero; a quantised copy: small and positive
    rc = ppl.main(["--model", str(src), "--tokens-file", str(tmp_path / "tok.pt"), "--chunk", "64", "--device", "cpu",
                   "--kl-teacher", str(teacher)])
    same = json.loads(capsys.readouterr().out.strip().splitlines()[-1])
    assert abs(same["kl"]) < 1e-4 and abs(same["ppl"] - out["ppl"]) / out["ppl"] < 1e-3
    q = tmp_path / "q"
    quantize_dir(src, q, "nvfp4", min_dim=64, log=lambda *_: None)
    ppl.main(["--model", str(q), "--tokens-file", str(tmp_path / "tok.pt"), "--chunk", "64", "--device", "cpu",
              "--kl-teacher", str(teacher)])
    quant = json.loads(capsys.readouterr().out.strip().splitlines()[-1])
    assert 1e-5 < quant["kl"] < 0.2


def test_tui_views_experts_speculation_memory():
    ex = {"ranks": 2, "layers": 2, "experts": 4, "total": [10, 30, 0, 60, 0, 0, 0, 0], "recent": []}
    f = tui.render_experts(ex, width=100)
    assert "2 layers x 4 experts" in f and " 3:60%" in f and " 1:30%" in f and f.count("\n") == 4     # layer 1 saw no routes
    assert "no routing histogram" in tui.render_experts({}, 80)
    stats = dict(STATS)
    stats["server"] = dict(stats.get("server", {}), speculation=True, speculator="draft")
    stats["speculation"] = {"rounds": 10, "proposed": 30, "accepted": 12, "accept_rate": 0.4, "tokens_per_round": 2.2,
                            "steps": [{"attempts": 10, "hits": 8}, {"attempts": 8, "hits": 3}, {"attempts": 3, "hits": 1}], "tree_rounds": 2, "tree_nodes": 9}
    f = tui.render_speculation(stats, 100)
    assert "accept 40.0%" in f and "80.0%" in f and "tree rounds 2 (9 nodes)" in f
    assert "off" in tui.render_speculation({"server": {}}, 80)
    f = tui.render_memory(stats, 100)
    assert f.startswith("memory") and "kv pool" in f
    assert tui.render_view("overview", stats, None, 100) == tui.render_frame(stats, 100)
    assert tui.render_view("experts", stats, ex, 100) == tui.render_experts(ex, 100)
    assert tui.VIEWS == ("overview", "experts", "speculation", "memory")
