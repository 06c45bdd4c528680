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
