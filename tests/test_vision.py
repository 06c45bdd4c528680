"""Vision tower: patch positions in merge-block order, 2-D rope properties, CPU forward shapes, GPU vs CPU."""
import numpy as np
import pytest
import torch

from volta_engine_b200.loader.image import VisionParams, prepare_image
from volta_engine_b200.models.util import to_device
from volta_engine_b200.models.vision import VisionConfig, VisionTower, rope2d


def test_patch_positions_follow_the_merge_block_order():
    t = VisionTower(VisionConfig(), "cpu")
    r, c = t.patch_positions(4, 6)
    assert r[:4].tolist() == [0, 0, 1, 1] and c[:4].tolist() == [0, 1, 0, 1]          # first 2x2 block
    assert r[4:8].tolist() == [0, 0, 1, 1] and c[4:8].tolist() == [2, 3, 2, 3]        # next block to the right
    assert r[12:16].tolist() == [2, 2, 3, 3] and c[12:16].tolist() == [0, 1, 0, 1]    # first block of the second band
    assert sorted(zip(r.tolist(), c.tolist())) == [(i, j) for i in range(4) for j in range(6)]


def test_rope2d_is_a_rotation_that_depends_on_row_and_column():
    g = torch.Generator().manual_seed(0)
    x = torch.randn(3, 2 * 64, generator=g)
    zero = torch.zeros(3, dtype=torch.int32)
    assert torch.allclose(rope2d(x.clone(), zero, zero, 2, 64, 1e4), x, atol=1e-6)
    rows = torch.tensor([1, 5, 9], dtype=torch.int32)
    y = rope2d(x.clone(), rows, zero, 2, 64, 1e4)
    assert torch.allclose(y.reshape(3, 2, 64).norm(dim=-1), x.reshape(3, 2, 64).norm(dim=-1), atol=1e-4)
    yh, xh = y.reshape(3, 2, 2, 32), x.reshape(3, 2, 2, 32)
    assert not torch.allclose(yh[..., :16], xh[..., :16]) and torch.allclose(yh[..., 16:], xh[..., 16:], atol=1e-6)
    # relative property: <rope(q, p), rope(k, p)> does not depend on p
    q, k = torch.randn(1, 64, generator=g), torch.randn(1, 64, generator=g)
    dots = []
    for p in (0, 7):
        pp = torch.tensor([p], dtype=torch.int32)
        dots.append(float((rope2d(q.clone(), pp, pp, 1, 64, 1e4) * rope2d(k.clone(), pp, pp, 1, 64, 1e4)).sum()))
    assert abs(dots[0] - dots[1]) < 1e-3


def _image_patches():
    rgb = np.random.default_rng(0).integers(0, 255, (96, 160, 3), dtype=np.uint8)
    return prepare_image(rgb, VisionParams(patch_size=16, merge_size=2, min_pixels=1024, max_pixels=65536))


def test_cpu_forward_shapes_and_determinism():
    pre = _image_patches()
    cfg = VisionConfig()
    t = VisionTower(cfg, "cpu").init_random(seed=1)
    out = t.forward(pre.patches, pre.grid_h, pre.grid_w)
    assert out.shape == (pre.tokens(2), cfg.out_hidden) and torch.isfinite(out.float()).all()
    assert torch.equal(out, t.forward(pre.patches, pre.grid_h, pre.grid_w))
    # every patch influences every token (bidirectional attention): perturb the last patch, the first token moves
    p2 = pre.patches.clone()
    p2[-1] += 1.0
    out2 = t.forward(p2, pre.grid_h, pre.grid_w)
    assert not torch.allclose(out2[0].float(), out[0].float(), atol=1e-4)


@pytest.mark.gpu
def test_gpu_tower_matches_cpu():
    pre = _image_patches()
    cfg = VisionConfig(depth=2, hidden=128, heads=2, mlp=256, out_hidden=256)      # head_dim 64: the paged attention kernel
    tc = VisionTower(cfg, "cpu").init_random(seed=2, std=0.05)
    tg = to_device(tc, "cuda:0")
    want = tc.forward(pre.patches, pre.grid_h, pre.grid_w).float()
    got = tg.forward(pre.patches, pre.grid_h, pre.grid_w).float().cpu()
    cos = torch.nn.functional.cosine_similarity(got.flatten(), want.flatten(), dim=0)
    assert cos > 0.998, float(cos)


def test_vision_tower_loads_from_a_checkpoint_directory_and_the_launcher_builds_the_frontend(tmp_path):
    """The tower's tensors under their checkpoint names round-trip through a safetensors directory; the launcher's
    frontend caps the image size by max_image_tokens and switches image input off at 0."""
    import json
    from types import SimpleNamespace
    from volta_engine_b200.loader.safetensors import write_safetensors
    from volta_engine_b200.models.factory import TensorSource
    from volta_engine_b200.models.vision import VisionConfig, VisionTower
    from volta_engine_b200.server.cli import load_vision_frontend
    vc = {"depth": 2, "hidden_size": 64, "num_heads": 2, "intermediate_size": 128, "patch_size": 16, "temporal_patch_size": 2,
          "spatial_merge_size": 2, "out_hidden_size": 96}
    cfg = VisionConfig.from_hf(vc)
    assert (cfg.depth, cfg.hidden, cfg.heads, cfg.mlp, cfg.out_hidden) == (2, 64, 2, 128, 96)
    t = VisionTower(cfg, "cpu").init_random(seed=3)
    write_safetensors(tmp_path / "vision.safetensors", t.state_tensors())
    (tmp_path / "config.json").write_text(json.dumps({"model_type": "qwen3_vl", "vision_config": vc, "image_token_id": 77}))
    (tmp_path / "preprocessor_config.json").write_text(json.dumps({"patch_size": 16, "merge_size": 2, "min_pixels": 4096, "max_pixels": 1 << 20}))
    t2 = VisionTower(cfg, "cpu").load(TensorSource(tmp_path))
    patches = torch.randn(4 * 6, cfg.patch_dim, generator=torch.Generator().manual_seed(1))
    assert torch.equal(t.forward(patches, 4, 6), t2.forward(patches, 4, 6))
    hf = json.loads((tmp_path / "config.json").read_text())
    o = SimpleNamespace(vision_dir="", max_image_tokens=16)
    front = load_vision_frontend(str(tmp_path), hf, o, "cpu")
    assert front is not None and front.image_token_id == 77 and front.params.max_pixels == 16 * 32 * 32
    assert load_vision_frontend(str(tmp_path), hf, SimpleNamespace(vision_dir="", max_image_tokens=0), "cpu") is None
    other = tmp_path / "elsewhere"
    other.mkdir()
    (other / "config.json").write_text(json.dumps({"model_type": "x"}))
    assert load_vision_frontend(str(other), {"model_type": "x"}, SimpleNamespace(vision_dir=str(tmp_path), max_image_tokens=64), "cpu") is not None


def test_vision_tower_loads_from_a_llama_cpp_projector_file(tmp_path):
    """vision_mmproj: the tower's weights under llama.cpp's clip tensor names (split temporal patch kernel, merged or
    separate q / k / v) give the same image tokens as the tower they were written from."""
    import json
    from types import SimpleNamespace
    from volta_engine_b200.loader.gguf_file import GGUFFile, write_gguf
    from volta_engine_b200.models.vision import VisionConfig, VisionTower
    from volta_engine_b200.quant import gguf as gq
    from volta_engine_b200.server.cli import load_vision_frontend
    vc = {"depth": 2, "hidden_size": 64, "num_heads": 2, "intermediate_size": 128, "patch_size": 16, "temporal_patch_size": 2,
          "spatial_merge_size": 2, "out_hidden_size": 96}
    cfg = VisionConfig.from_hf(vc)
    t = VisionTower(cfg, "cpu").init_random(seed=5)
    bf = lambda x: (x.to(torch.bfloat16), gq.GGML_BF16, tuple(x.shape))
    f32 = lambda x: (x.float(), gq.GGML_F32, tuple(x.shape))
    pe = t.patch_embed.weight.reshape(cfg.hidden, 3, cfg.temporal, cfg.patch, cfg.patch)
    tensors = {"v.patch_embd.weight": bf(pe[:, :, 0].contiguous()), "v.patch_embd.weight.1": bf(pe[:, :, 1].contiguous()),
               "v.patch_embd.bias": f32(t.patch_bias)}
    for i, b in enumerate(t.blocks):
        q = f"v.blk.{i}."
        tensors.update({q + "ln1.weight": f32(b["ln1_w"]), q + "ln1.bias": f32(b["ln1_b"]), q + "ln2.weight": f32(b["ln2_w"]),
                        q + "ln2.bias": f32(b["ln2_b"]), q + "attn_out.weight": bf(b["proj"].weight), q + "attn_out.bias": f32(b["proj_b"]),
                        q + "ffn_up.weight": bf(b["fc1"].weight), q + "ffn_up.bias": f32(b["fc1_b"]),
                        q + "ffn_down.weight": bf(b["fc2"].weight), q + "ffn_down.bias": f32(b["fc2_b"])})
        if i == 0:                                     # one block merged, one with separate q / k / v
            tensors.update({q + "attn_qkv.weight": bf(b["qkv"].weight), q + "attn_qkv.bias": f32(b["qkv_b"])})
        else:
            for j, n in enumerate("qkv"):
                tensors[q + f"attn_{n}.weight"] = bf(b["qkv"].weight[j * cfg.hidden:(j + 1) * cfg.hidden].contiguous())
                tensors[q + f"attn_{n}.bias"] = f32(b["qkv_b"][j * cfg.hidden:(j + 1) * cfg.hidden].contiguous())
    m = t.merger
    tensors.update({"v.post_ln.weight": f32(m["ln_w"]), "v.post_ln.bias": f32(m["ln_b"]), "mm.0.weight": bf(m["fc1"].weight),
                    "mm.0.bias": f32(m["fc1_b"]), "mm.2.weight": bf(m["fc2"].weight), "mm.2.bias": f32(m["fc2_b"])})
    write_gguf(tmp_path / "model-mmproj-bf16.gguf", {"general.architecture": "clip"}, tensors)
    t2 = VisionTower(cfg, "cpu").load_mmproj(GGUFFile(tmp_path / "model-mmproj-bf16.gguf"))
    patches = torch.randn(4 * 6, cfg.patch_dim, generator=torch.Generator().manual_seed(1))
    assert torch.equal(t.forward(patches, 4, 6), t2.forward(patches, 4, 6))
    (tmp_path / "config.json").write_text(json.dumps({"model_type": "qwen3_vl", "vision_config": vc}))
    front = load_vision_frontend(str(tmp_path), {"vision_config": vc}, SimpleNamespace(vision_dir="", max_image_tokens=64,
                                                                                       vision_mmproj=str(tmp_path)), "cpu")
    assert front is not None and torch.equal(front.tower.forward(patches, 4, 6), t.forward(patches, 4, 6))
