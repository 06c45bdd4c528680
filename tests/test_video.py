"""Video diffusion transformer: INT8 rotated linears, the block's pieces, the sampler, and the sequence- / tensor-parallel
forms on two gloo ranks."""
import os
import socket
import subprocess
import sys

import pytest
import torch

from volta_engine_b200.video import dit as V

HERE = os.path.dirname(os.path.abspath(__file__))


def test_convrot_linear_round_trip_and_shards():
    g = torch.Generator().manual_seed(0)
    w = torch.randn(96, 512, generator=g) * 0.05
    lin = V.ConvRotLinear.from_dense(w)
    assert lin.q.dtype == torch.int8 and float((lin.dequant() - w).abs().max()) < 0.01          # 8-bit rows
    x = torch.randn(5, 512, generator=g)
    assert torch.allclose(lin.forward(x), x @ lin.dequant().t(), rtol=1e-4, atol=1e-5)
    # the rotation is orthonormal and an involution
    assert torch.allclose(V.hadamard_groups(V.hadamard_groups(x)), x, atol=1e-5)
    # shards: rows take their scales along, columns keep whole groups; the pieces add up to the whole product
    top, bot = lin.shard(rows=torch.arange(0, 48)), lin.shard(rows=torch.arange(48, 96))
    assert torch.allclose(torch.cat([top.forward(x), bot.forward(x)], 1), lin.forward(x), atol=1e-5)
    left, right = lin.shard(cols=(0, 256)), lin.shard(cols=(256, 512))
    assert torch.allclose(left.forward(x[:, :256]) + right.forward(x[:, 256:]), lin.forward(x), atol=1e-4)
    with pytest.raises(AssertionError):
        lin.shard(cols=(0, 128))


def test_timestep_table_rope_and_schedule():
    table = torch.arange(17 * 8, dtype=torch.float32).reshape(17, 8)
    e = V.timestep_embedding(table, torch.tensor([0.0, 1.0, 0.5, 1 / 32]))
    assert torch.equal(e[0], table[0]) and torch.equal(e[1], table[16]) and torch.allclose(e[2], table[8])
    assert torch.allclose(e[3], (table[0] + table[1]) / 2)
    x = torch.randn(6, 2, 64, generator=torch.Generator().manual_seed(1))
    pos = torch.tensor([[0, 0, 0], [1, 0, 0], [0, 2, 0], [0, 0, 3], [1, 2, 3], [4, 4, 4]], dtype=torch.float32)
    y = V.rope3d(x, pos, 8)
    assert torch.equal(y[0], x[0]) and torch.allclose(y.norm(dim=-1), x.norm(dim=-1), rtol=1e-5)
    assert torch.equal(y[1, :, 16:], x[1, :, 16:])            # a step along t rotates the first axis' dims only
    assert torch.equal(y[..., 48:], x[..., 48:])              # dims past 3 x 2 x freqs are never rotated
    s = V.sigma_schedule(4, shift=6.0)
    assert float(s[0]) == 1.0 and float(s[-1]) == 0.0 and torch.all(s[:-1] > s[1:])
    assert abs(float(s[2]) - 6 * 0.5 / (1 + 5 * 0.5)) < 1e-6


def test_denoise_is_deterministic_and_text_conditioned():
    cfg = V.H3Config.tiny()
    m = V.H3DiT(cfg).init_random(seed=2)
    g = torch.Generator().manual_seed(3)
    prompt = torch.randn(6, cfg.text_dim, generator=g)
    a = V.denoise(m, prompt, (2, 2, 2), 3, steps=3, seed=7)
    b = V.denoise(m, prompt, (2, 2, 2), 3, steps=3, seed=7)
    c = V.denoise(m, prompt * 2 + 1, (2, 2, 2), 3, steps=3, seed=7)
    assert torch.equal(a[0], b[0]) and torch.equal(a[1], b[1]) and not torch.allclose(a[0], c[0])
    assert a[0].shape == (8, cfg.latents) and a[1].shape == (3, cfg.audio_latents) and torch.isfinite(a[0]).all()
    frames = V.frames_rgb8(a[0], (2, 2, 2))
    assert frames.shape == (2, 4, 4, 3) and frames.dtype == torch.uint8


def test_dit_sequence_and_tensor_parallel_match_one_rank():
    s = socket.socket()
    s.bind(("127.0.0.1", 0))
    port = s.getsockname()[1]
    s.close()
    procs = []
    for r in range(2):
        env = dict(os.environ, RANK=str(r), WORLD_SIZE="2", MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port), OMP_NUM_THREADS="2")
        procs.append(subprocess.Popen([sys.executable, os.path.join(HERE, "h3_worker.py")], env=env, stdout=subprocess.PIPE,
                                      stderr=subprocess.STDOUT))
    logs = []
    for p in procs:
        try:
            o, _ = p.communicate(timeout=300)
        except subprocess.TimeoutExpired:
            p.kill()
            o, _ = p.communicate()
        logs.append(o.decode(errors="replace"))
    assert all(p.returncode == 0 for p in procs) and "H3_WORKER_OK" in logs[0], "\n---\n".join(l[-3000:] for l in logs)


@pytest.mark.gpu
def test_gpu_dit_matches_cpu():
    cfg = V.H3Config.tiny()
    mc = V.H3DiT(cfg).init_random(seed=2)
    mg = V.H3DiT(cfg, "cuda").init_random(seed=2)
    g = torch.Generator().manual_seed(3)
    video, audio, prompt = torch.randn(256, cfg.latents, generator=g), torch.randn(16, cfg.audio_latents, generator=g), torch.randn(16, cfg.text_dim, generator=g)
    rc = V.make_request(video, audio, prompt, (4, 8, 8), 0.6, 0.3)
    rg = V.make_request(video.cuda(), audio.cuda(), prompt.cuda(), (4, 8, 8), 0.6, 0.3)
    vc, ac = mc.forward(rc)
    vg, ag = mg.forward(rg)
    cos = torch.nn.functional.cosine_similarity(vg.cpu().flatten(), vc.flatten(), dim=0)
    assert float(cos) > 0.995, float(cos)


def _lora_files(tmp_path, cfg, rank=8, seed=0):
    """The same adapter (q / k / v, output, gate | up, down of block 0 and 1) written in the three key layouts."""
    from volta_engine_b200.loader.safetensors import write_safetensors
    g = torch.Generator().manual_seed(seed)
    qd, H, F = cfg.heads * cfg.head_dim, cfg.hidden, cfg.ffn
    rnd = lambda *s: (torch.randn(*s, generator=g) * 0.2).to(torch.bfloat16)
    pairs = {}
    for L in range(2):
        pairs[L] = {"q": (rnd(rank, H), rnd(qd, rank)), "k": (rnd(rank, H), rnd(qd, rank)), "v": (rnd(rank, H), rnd(qd, rank)),
                    "out": (rnd(rank, qd), rnd(H, rank)), "fc1": (rnd(rank, H), rnd(2 * F, rank)), "fc2": (rnd(rank, F), rnd(H, rank))}
    dif, koh, ait = {}, {}, {}
    for L, p in pairs.items():
        for n, suffix in (("q", "attn.to_q"), ("k", "attn.to_k"), ("v", "attn.to_v"), ("out", "attn.to_out.0"),
                          ("fc1", "ff.net.0.proj"), ("fc2", "ff.net.2")):
            dif[f"transformer_blocks.{L}.{suffix}.lora_A.default.weight"], dif[f"transformer_blocks.{L}.{suffix}.lora_B.default.weight"] = p[n]
        # the fused q | k | v of the native layouts: one A of rank 3r (stacked) and a block-diagonal B give the same delta
        a_qkv = torch.cat([p["q"][0], p["k"][0], p["v"][0]], 0)
        b_qkv = torch.zeros(3 * qd, 3 * rank, dtype=torch.bfloat16)
        for i, n in enumerate("qkv"):
            b_qkv[i * qd:(i + 1) * qd, i * rank:(i + 1) * rank] = p[n][1]
        native = {"attn.qkv_proj": (a_qkv, b_qkv), "attn.out_proj": p["out"], "mlp.fc1": p["fc1"], "mlp.fc2": p["fc2"]}
        for nn, (a, b) in native.items():
            k = f"lora_unet_blocks_{L}_" + nn.replace(".", "_")
            # diffusers scales by alpha / rank (alpha 4 in the metadata below); kohya by its alpha tensor / rank; ai-toolkit by 1
            koh[k + ".lora_down.weight"], koh[k + ".lora_up.weight"], koh[k + ".alpha"] = a, b, torch.tensor(4.0 * a.shape[0] / rank)
            ait[f"diffusion_model.blocks.{L}.{nn}.lora_A.weight"], ait[f"diffusion_model.blocks.{L}.{nn}.lora_B.weight"] = a, (b.float() * (4.0 / rank)).to(torch.bfloat16)
    write_safetensors(tmp_path / "h3_fl2v_turbo_4step.safetensors", dif, metadata={"alpha": "4"})
    write_safetensors(tmp_path / "style_kohya.safetensors", koh)
    write_safetensors(tmp_path / "style_aitk.safetensors", ait)
    return pairs


def test_lora_layouts_scales_and_tensor_parallel_parts(tmp_path):
    from volta_engine_b200.video import lora as LR
    cfg = V.H3Config.tiny()
    rank = 8
    pairs = _lora_files(tmp_path, cfg, rank)
    qd, H, F = cfg.heads * cfg.head_dim, cfg.hidden, cfg.ffn
    g = torch.Generator().manual_seed(5)
    x = torch.randn(6, H, generator=g)
    xo, xf = torch.randn(6, qd, generator=g), torch.randn(6, F, generator=g)
    f32 = lambda t: t.float()

    def want(L, slot, scale):
        p = pairs[L]
        d = lambda a, b, inp: (inp @ f32(a).t()) @ f32(b).t() * (scale * 4.0 / rank)
        if slot == 0:
            return torch.cat([d(*p["q"], x), d(*p["k"], x), d(*p["v"], x)], 1)
        return {1: d(*p["out"], xo), 2: d(*p["fc1"], x), 3: d(*p["fc2"], xf)}[slot]
    inputs = {0: x, 1: xo, 2: x, 3: xf}
    ads = {n: LR.load_adapter(tmp_path / n, cfg, scale=0.5, dtype=torch.float32)
           for n in ("h3_fl2v_turbo_4step.safetensors", "style_kohya.safetensors", "style_aitk.safetensors")}
    assert [a.layout for a in ads.values()] == ["diffusers", "kohya", "ai-toolkit"]
    assert ads["h3_fl2v_turbo_4step.safetensors"].targets() == 12 and ads["style_kohya.safetensors"].targets() == 8
    for name, ad in ads.items():
        for L in range(2):
            for slot in range(4):
                w = want(L, slot, 0.5)
                y = LR.apply_lora([ad], L, slot, inputs[slot], torch.zeros_like(w))
                tol = 2e-2 if name == "style_aitk.safetensors" else 1e-4          # (its B was rescaled in bf16)
                assert torch.allclose(y, w, atol=tol * float(w.abs().max())), (name, L, slot)
    # two adapters add; a scale of zero switches one off
    both = LR.apply_lora(list(ads.values())[:2], 0, 2, x, torch.zeros(6, 2 * F))
    assert torch.allclose(both, 2 * want(0, 2, 0.5), atol=1e-4 * float(both.abs().max()))
    ads["style_kohya.safetensors"].scale = 0.0
    assert torch.allclose(LR.apply_lora(list(ads.values())[:2], 0, 2, x, torch.zeros(6, 2 * F)), want(0, 2, 0.5), atol=1e-5)
    # tensor parallel, two ranks: column-parallel parts give this rank's columns, row-parallel partials add up to the delta
    ql, fl = qd // 2, F // 2
    for name in ("h3_fl2v_turbo_4step.safetensors", "style_kohya.safetensors"):
        parts = [LR.load_adapter(tmp_path / name, cfg, scale=0.5, tp_rank=r, tp_ranks=2, dtype=torch.float32) for r in range(2)]
        full = want(1, 0, 0.5)
        for r in range(2):
            y = LR.apply_lora([parts[r]], 1, 0, x, torch.zeros(6, 3 * ql))
            mine = torch.cat([full[:, s * qd + r * ql:s * qd + (r + 1) * ql] for s in range(3)], 1)
            assert torch.allclose(y, mine, atol=1e-4 * float(full.abs().max())), name
            y = LR.apply_lora([parts[r]], 1, 2, x, torch.zeros(6, 2 * fl))
            f1 = want(1, 2, 0.5)
            assert torch.allclose(y, torch.cat([f1[:, r * fl:(r + 1) * fl], f1[:, F + r * fl:F + (r + 1) * fl]], 1), atol=1e-4 * float(f1.abs().max()))
        tot = sum(LR.apply_lora([parts[r]], 1, 1, xo[:, r * ql:(r + 1) * ql], torch.zeros(6, H)) for r in range(2))
        assert torch.allclose(tot, want(1, 1, 0.5), atol=1e-4 * float(tot.abs().max()))
        tot = sum(LR.apply_lora([parts[r]], 1, 3, xf[:, r * fl:(r + 1) * fl], torch.zeros(6, H)) for r in range(2))
        assert torch.allclose(tot, want(1, 3, 0.5), atol=1e-4 * float(tot.abs().max()))
    with pytest.raises(ValueError):
        from volta_engine_b200.loader.safetensors import write_safetensors
        write_safetensors(tmp_path / "empty.safetensors", {"x": torch.zeros(1)})
        LR.load_adapter(tmp_path / "empty.safetensors", cfg)
    # the catalogue: formats, the turbo flag, reference-to-video turbo files only with that transformer configured
    (tmp_path / "h3_ref2v_turbo.safetensors").write_bytes((tmp_path / "h3_fl2v_turbo_4step.safetensors").read_bytes())
    cat = LR.AdapterCatalog().scan([tmp_path])
    assert {a.file: (a.format, a.turbo, a.task) for a in cat.all()} == {
        "h3_fl2v_turbo_4step.safetensors": ("diffusers", True, "fl2v"), "style_kohya.safetensors": ("kohya", False, "ref2va"),
        "style_aitk.safetensors": ("ai-toolkit", False, "ref2va")}
    assert LR.AdapterCatalog().scan([tmp_path], ref2va=True).find("h3_ref2v_turbo.safetensors").task == "ref2v"


def test_denoiser_with_adapters_and_job_staging(tmp_path):
    from volta_engine_b200.video import lora as LR
    from volta_engine_b200.video.pipeline import H3Job, H3Pipeline
    p = H3Pipeline.tiny()
    cfg = p.dit.cfg
    _lora_files(tmp_path, cfg, rank=8)
    job = H3Job(prompt="kite", width=32, height=16, frames=9, steps=2, seed=3)
    grid = job.grid(p.vae_cfg)
    prompt = p.encode_prompt(job)
    base, _ = p.denoise(job, prompt, grid, {})
    i = p.dit.add_lora(tmp_path / "style_kohya.safetensors", 1.0)
    with_ad, _ = p.denoise(job, prompt, grid, {})
    assert not torch.equal(base, with_ad)
    p.dit.set_lora_scale(i, 0.0)
    assert torch.equal(p.denoise(job, prompt, grid, {})[0], base)
    p.dit.clear_loras()
    assert p.dit.adapters == [] and p.dit.blocks[0].adapters is p.dit.adapters
    # jobs name adapters of the catalogue; the staged set is reused while the files stay the same
    p.catalog = LR.AdapterCatalog().scan([tmp_path])
    job.loras = [("style_kohya.safetensors", 1.0)]
    p.stage_adapters(job)
    first = p.dit.adapters[0]
    job.loras = [("style_kohya.safetensors", 0.25)]
    p.stage_adapters(job)
    assert p.dit.adapters[0] is first and first.scale == 0.25
    out = p.run(job, str(tmp_path / "job"))
    assert out["frames"] == 9
    job.loras = [("missing.safetensors", 1.0)]
    with pytest.raises(ValueError):
        p.stage_adapters(job)
    job.loras = []
    p.stage_adapters(job)
    assert p.dit.adapters == []
