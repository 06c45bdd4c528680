"""The rest of the video pipeline around the transformer: VAE encoder convolutions against the library convolution, tiled
decoding against whole-picture decoding, the audio stack's resamplers and shapes, the text tower, a whole job through the
stages, and the job service's HTTP routes."""
import base64
import json
import os
import time

import pytest
import torch
import torch.nn.functional as F

from volta_engine_b200.video import audio as A
from volta_engine_b200.video import vae as V
from volta_engine_b200.video.pipeline import H3Job, H3Pipeline, patchify, unpatchify
from volta_engine_b200.video.service import VideoService, serve


def test_causal_conv3d_equals_the_library_convolution_with_front_padding():
    g = torch.Generator().manual_seed(0)
    x = torch.randn(3, 6, 9, 10, generator=g)
    w = torch.randn(5, 3, 3, 3, 3, generator=g) * 0.2
    b = torch.randn(5, generator=g)
    for stride in ((1, 1, 1), (2, 2, 2), (1, 2, 2)):
        got = V.causal_conv3d(x, w, b, stride)
        want = F.conv3d(F.pad(x[None], (1, 1, 1, 1, 2, 0)), w, b, stride=stride)[0]
        assert got.shape == want.shape and torch.allclose(got, want, atol=1e-4), stride
    # causality: frame t of the output does not move when later input frames change
    x2 = x.clone()
    x2[:, 4:] += 1.0
    assert torch.allclose(V.causal_conv3d(x, w, b)[:, :4], V.causal_conv3d(x2, w, b)[:, :4])


def test_encoder_shapes_and_first_frame_block():
    cfg = V.VaeConfig.tiny()
    enc = V.VideoEncoder(cfg).init_random(1)
    frames = torch.randint(0, 255, (1 + 2 * cfg.t_up, 16, 24, 3), dtype=torch.uint8)
    z = enc.encode(frames)
    assert tuple(z.shape) == (3, 16 // cfg.s_up, 24 // cfg.s_up, cfg.latent)
    z1 = enc.encode(frames[:1])
    assert tuple(z1.shape) == (1, 4, 6, cfg.latent) and torch.allclose(z1[0], z[0], atol=1e-4)      # causal: frame 0 alone


def test_tiled_decode_blends_tiles_and_equals_whole_decode_where_one_tile_covers_it():
    cfg = V.VaeConfig.tiny(tile=8, overlap=2, chunk=4)
    dec = V.VideoDecoder(cfg).init_random(2)
    lat = torch.randn(2, 6, 8, cfg.latent, generator=torch.Generator().manual_seed(3))
    whole = dec.decode(lat)                                                        # 6 x 8 fits one tile
    assert whole.dtype == torch.uint8 and tuple(whole.shape) == (2 * cfg.t_up, 6 * cfg.s_up, 8 * cfg.s_up, 3)
    px = dec.decode_tile(lat)
    assert torch.equal(whole, ((px.clamp(-1, 1) + 1) * 127.5).round().to(torch.uint8))
    assert V.VideoDecoder.tile_starts(46, 16, 4) == [0, 12, 24, 30] and V.VideoDecoder.tile_starts(10, 16, 4) == [0]
    small = V.VideoDecoder(V.VaeConfig.tiny(tile=4, overlap=2, chunk=1)).init_random(2)
    calls = []
    tiled = small.decode(lat, on_tile=lambda d, t: calls.append((d, t)))
    assert tuple(tiled.shape) == tuple(whole.shape) and calls[-1][0] == calls[-1][1] == 2 * 2 * 3
    w = V.VideoDecoder._ramp(4, True, True, 2, 4)
    assert w[0] < w[7] and abs(float(w[7]) - 0.9375) < 1e-6 and float(w[8]) == float(w[7]) and torch.allclose(w, w.flip(0))
    assert float(V.VideoDecoder._ramp(6, True, False, 2, 4)[-1]) == 1.0            # an edge of the picture keeps full weight


def test_audio_resamplers_snake_and_shapes():
    t = torch.arange(256).float()
    lo = torch.sin(2 * torch.pi * 0.02 * t)[None]                                  # well below the band edge: passes
    up = A.upsample2(lo)
    assert up.shape[1] == 512 and torch.allclose(A.upsample2(torch.ones(1, 64)), torch.ones(1, 128), atol=1e-3)      # unit DC gain
    # (the even-length filter sits half a high-rate sample off the grid; the decimator's offset undoes it: the pair is aligned)
    back = A.downsample2(up)
    assert back.shape[1] == 256 and torch.allclose(back[0, 20:-20], lo[0, 20:-20], atol=0.03)
    hi = torch.cos(torch.pi * t)[None]                                             # the Nyquist tone is removed before decimation
    assert float(A.downsample2(hi).abs()[0, 20:-20].max()) < 0.02
    x = torch.randn(3, 50)
    la = torch.tensor([0.0, 0.5, -0.5])
    assert torch.allclose(A.snake(x, la), x + torch.sin(la.exp()[:, None] * x) ** 2 / la.exp()[:, None], atol=1e-6)
    cfg = A.AudioConfig.tiny()
    dec, enc = A.AudioDecoder(cfg).init_random(0), A.AudioEncoder(cfg).init_random(1)
    pcm = dec.decode(torch.randn(10, cfg.latent))
    assert tuple(pcm.shape) == (2, 10 * cfg.hop) and float(pcm.abs().max()) <= 1.0
    assert tuple(enc.encode(pcm).shape) == (10, cfg.latent)


def test_patch_layout_roundtrip_and_job_validation():
    lat = torch.randn(2, 4, 6, 5)
    rows = patchify(lat)
    assert tuple(rows.shape) == (2 * 2 * 3, 20) and torch.equal(unpatchify(rows, (2, 2, 3)), lat)
    vae = V.VaeConfig.tiny()
    H3Job(width=32, height=16, frames=9).validate(vae)
    for bad in (dict(width=30), dict(frames=8), dict(steps=0), dict(video_shift=0.1), dict(loras=[("a", 1)] * 7)):
        with pytest.raises(ValueError):
            H3Job(**dict(dict(width=32, height=16, frames=9), **bad)).validate(vae)
    assert H3Job(width=32, height=16, frames=9).grid(vae) == (3, 2, 4)


def test_a_job_runs_through_every_stage_and_keyframes_are_held(tmp_path):
    p = H3Pipeline.tiny()
    job = H3Job(prompt="a red kite over the sea", width=32, height=16, frames=9, steps=2, seed=3,
                images=[(torch.randint(0, 255, (16, 32, 3), dtype=torch.uint8), 0)])
    seen = []
    out = p.run(job, str(tmp_path / "job"), progress=lambda s, d, t: seen.append(s))
    assert out["frames"] == 9 and out["width"] == 32 and out["height"] == 16 and os.path.getsize(out["raw"]) == 9 * 16 * 32 * 3
    assert os.path.getsize(out["audio"]) > 44 and [s for i, s in enumerate(seen) if s not in seen[:i]] == ["plan", "references", "text", "denoise", "decode"]
    # the keyframe's latent rows come out of the sampler exactly as the encoder produced them
    grid = job.grid(p.vae_cfg)
    cond = p.encode_references(job, grid)
    xv, _ = p.denoise(job, p.encode_prompt(job), grid, cond)
    assert torch.allclose(xv[: grid[1] * grid[2]].cpu(), cond[0], atol=1e-6)
    # the same seed gives the same video; a cancelled job stops at the next boundary
    out2 = p.run(job, str(tmp_path / "job2"))
    assert open(out["raw"], "rb").read() == open(out2["raw"], "rb").read()
    with pytest.raises(InterruptedError):
        p.run(job, str(tmp_path / "job3"), cancelled=lambda: True)


def test_video_service_routes(tmp_path):
    svc = VideoService(H3Pipeline.tiny(), str(tmp_path / "out"), max_rows=64)
    try:
        st, ct, body, _ = svc.handle("GET", "/api/info")
        assert st == 200 and json.loads(body)["model"] == "minimax_h3"
        st, _, body, _ = svc.handle("POST", "/api/jobs", json.dumps({"prompt": "x", "width": 30, "height": 16, "frames": 9}).encode())
        assert st == 400
        st, _, body, _ = svc.handle("POST", "/api/jobs", json.dumps({"prompt": "x", "width": 320, "height": 160, "frames": 9}).encode())
        assert st == 400 and "rows" in json.loads(body)["error"]                    # over the row limit
        img = base64.b64encode(bytes(16 * 32 * 3)).decode()
        st, _, body, _ = svc.handle("POST", "/api/jobs", json.dumps({"prompt": "waves", "width": 32, "height": 16, "frames": 5, "steps": 1,
                                                                    "images": [{"data": img, "frame_index": 0}]}).encode())
        assert st == 200
        jid = json.loads(body)["id"]
        assert svc.handle("GET", "/api/jobs/" + jid + "/video")[0] in (200, 409)
        done = svc.wait(jid, 120)
        assert done["status"] == "done", done
        st, _, body, _ = svc.handle("GET", "/api/jobs")
        assert [j["id"] for j in json.loads(body)["jobs"]] == [jid]
        st, ct, data, extra = svc.handle("GET", f"/api/jobs/{jid}/video", headers={"range": "bytes=10-19"})
        assert st == 206 and len(data) == 10 and extra["Content-Range"].startswith("bytes 10-19/")
        assert svc.handle("GET", f"/api/jobs/{jid}/thumb")[0] == 200
        assert svc.handle("GET", "/api/jobs/nope")[0] == 404
        # a queued job can be cancelled before the worker reaches it; deleting removes it
        slow = json.loads(svc.handle("POST", "/api/jobs", json.dumps({"prompt": "a", "width": 32, "height": 16, "frames": 9, "steps": 3}).encode())[2])
        nxt = json.loads(svc.handle("POST", "/api/jobs", json.dumps({"prompt": "b", "width": 32, "height": 16, "frames": 5, "steps": 1}).encode())[2])
        st, _, body, _ = svc.handle("POST", f"/api/jobs/{nxt['id']}/cancel")
        assert json.loads(body)["status"] in ("cancelled", "running", "done")
        svc.wait(slow["id"], 120)
        assert svc.handle("DELETE", f"/api/jobs/{slow['id']}")[0] == 200 and slow["id"] not in svc.jobs
    finally:
        svc.stop()


def test_video_service_over_http(tmp_path):
    import urllib.request
    svc = VideoService(H3Pipeline.tiny(), str(tmp_path / "out"))
    stop = []
    srv = serve(svc, "127.0.0.1", 0, stop=lambda: bool(stop))
    try:
        base = f"http://127.0.0.1:{srv.port}"
        info = json.loads(urllib.request.urlopen(base + "/api/info", timeout=10).read())
        assert info["model"] == "minimax_h3"
        req = urllib.request.Request(base + "/api/jobs", data=json.dumps({"prompt": "hi", "width": 32, "height": 16, "frames": 5, "steps": 1}).encode(),
                                     method="POST", headers={"Content-Type": "application/json"})
        jid = json.loads(urllib.request.urlopen(req, timeout=10).read())["id"]
        assert svc.wait(jid, 120)["status"] == "done"
        got = json.loads(urllib.request.urlopen(base + "/api/jobs/" + jid, timeout=10).read())
        assert got["status"] == "done" and got["result"]["frames"] == 5
    finally:
        stop.append(1)
        time.sleep(0.3)
        srv.stop()
        svc.stop()


def test_launcher_recognises_a_video_model_directory_and_the_generate_tool_runs(tmp_path, capsys):
    from volta_engine_b200.server.cli import build_video_service, is_video_model_dir
    from volta_engine_b200.video.generate import main as h3_generate
    root = tmp_path / "h3"
    root.mkdir()
    assert not is_video_model_dir(str(root))
    (root / "model_index.json").write_text(json.dumps({"_class_name": "MiniMaxH3Pipeline"}))
    assert is_video_model_dir(str(root))
    with pytest.raises(NotImplementedError):
        build_video_service(str(root), device="cpu")
    (root / "model_index.json").write_text(json.dumps({"_class_name": "MiniMaxH3Pipeline", "synthetic_weights": 4, "shape": "tiny"}))
    rc = h3_generate(["--root", str(root), "--prompt", "a boat", "--size", "32x16", "--frames", "5", "--steps", "1", "--out",
                      str(tmp_path / "o"), "--device", "cpu"])
    line = json.loads(capsys.readouterr().out.strip().splitlines()[-1])
    assert rc == 0 and line["frames"] == 5 and os.path.exists(line["raw"])
    assert h3_generate(["--root", str(root), "--size", "30x16", "--frames", "5", "--out", str(tmp_path / "o2"), "--device", "cpu"]) == 2


@pytest.mark.gpu
def test_gpu_full_attention_and_vae_decoder_match_the_cpu_statement():
    from volta_engine_b200.ops import kernels as K
    from volta_engine_b200.video.common import full_attention
    g = torch.Generator().manual_seed(5)
    for heads, hd, n in ((4, 128, 300), (3, 64, 150)):                       # the tcgen05 kernel and the mma.sync kernel
        q, k, v = (torch.randn(n, heads * hd, generator=g).to(torch.bfloat16) for _ in range(3))
        want = full_attention(q, k, v, heads, hd).float()
        got = full_attention(q.cuda(), k.cuda(), v.cuda(), heads, hd).float().cpu()
        cos = torch.nn.functional.cosine_similarity(got.flatten().double(), want.flatten().double(), dim=0)
        assert float(cos) > 0.9995, (hd, float(cos))
    cfg = V.VaeConfig.tiny(head_dim=64, heads=2, dim=128)
    dc, dg = V.VideoDecoder(cfg).init_random(2), V.VideoDecoder(cfg, "cuda").init_random(2)
    lat = torch.randn(2, 4, 4, cfg.latent, generator=g)
    a, b = dc.decode_tile(lat).float(), dg.decode_tile(lat.cuda()).float().cpu()
    assert float(torch.nn.functional.cosine_similarity(a.flatten(), b.flatten(), dim=0)) > 0.99
    assert K.check_status(torch.device("cuda")) == 0


@pytest.mark.gpu
def test_gpu_video_job_runs(tmp_path):
    p = H3Pipeline.tiny("cuda")
    out = p.run(H3Job(prompt="tide pools", width=32, height=16, frames=5, steps=2, seed=1), str(tmp_path / "j"))
    assert out["frames"] == 5 and os.path.getsize(out["raw"]) == 5 * 16 * 32 * 3


def test_captions_through_the_text_tower_and_the_service(tmp_path):
    """A tower built with its last layers and head writes text: the condition rows stay those of the shorter tower, greedy
    decoding continues the same whether the first half of an answer was decoded or prefilled, sampling is seeded, a picture
    changes the answer; the service runs caption requests on its worker."""
    import base64
    import io
    import json
    from PIL import Image
    from volta_engine_b200.loader.image import VisionParams
    from volta_engine_b200.models.vision import VisionConfig, VisionTower
    from volta_engine_b200.runtime.multimodal import MultimodalFrontend
    from volta_engine_b200.video.service import VideoService
    from volta_engine_b200.video.text import H3Captioner, H3TextTower
    t, short = H3TextTower.tiny(captioner=True).init_random(1), H3TextTower.tiny().init_random(1)
    assert t.can_generate and not short.can_generate and t.cfg.n_layers == short.cfg.n_layers + 1
    ids = [5, 6, 7, 8, 9, 10]
    assert torch.equal(t.encode(ids), short.encode(ids))
    prompt = list(range(10, 40))
    a = t.generate(prompt, 12)
    assert len(a) == 12 and t.generate(prompt + a[:6], 6) == a[6:]
    assert t.generate(prompt, 12, forced=a[:5]) == a
    assert t.generate(prompt, 12, eos_ids=(a[3],)) == a[:4]
    s1, s2 = t.generate(prompt, 12, temperature=0.7, seed=1), t.generate(prompt, 12, temperature=0.7, seed=1)
    assert s1 == s2 and t.generate(prompt, 12, temperature=5.0, seed=2) != s1
    assert "user's idea" in H3Captioner.instruction("a  kite\n") and "a kite" in H3Captioner.instruction("a  kite\n")
    p = H3Pipeline.tiny(captioner=True)
    vt = VisionTower(VisionConfig(out_hidden=64), "cpu").init_random(2)
    fe = MultimodalFrontend(vt, VisionParams(min_pixels=32 * 32, max_pixels=64 * 64), image_token_id=400)
    cap = p.attach_captioner(lambda ids: bytes(32 + (i % 90) for i in ids).decode(), fe, 400, eos_ids=(0,), max_new=10)
    buf = io.BytesIO()
    Image.fromarray(torch.randint(0, 255, (48, 64, 3), dtype=torch.uint8).numpy()).save(buf, format="PNG")
    with_pic, without = cap.caption(buf.getvalue(), "", greedy=True), cap.caption(None, "", greedy=True)
    assert with_pic and without and with_pic != without and cap.caption(buf.getvalue(), "", greedy=True) == with_pic
    svc = VideoService(p, str(tmp_path / "out"))
    try:
        st, _, body, _ = svc.handle("POST", "/api/caption", json.dumps({"image": base64.b64encode(buf.getvalue()).decode(), "greedy": True}).encode())
        cid = json.loads(body)["id"]
        assert st == 200
        for _ in range(500):
            rec = json.loads(svc.handle("GET", f"/api/caption/{cid}")[2])
            if rec["status"] in ("done", "failed"):
                break
            import time
            time.sleep(0.02)
        assert rec["status"] == "done" and rec["text"] == with_pic and "_image" not in rec
        assert svc.handle("POST", "/api/caption", b"{}")[0] == 400 and svc.handle("GET", "/api/caption/nope")[0] == 404
        assert json.loads(svc.handle("GET", "/api/info")[2])["captioner"] is True
    finally:
        svc.stop()
    plain = VideoService(H3Pipeline.tiny(), str(tmp_path / "out2"))
    try:
        assert plain.handle("POST", "/api/caption", json.dumps({"prompt": "x"}).encode())[0] == 400
    finally:
        plain.stop()
