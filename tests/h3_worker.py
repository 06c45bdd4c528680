"""Child process of tests/test_video.py: one CPU rank of a gloo world; sequence- and tensor-parallel DiT against one rank."""
import datetime
import os
import sys

import torch
import torch.distributed as dist

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))

from volta_engine_b200.video import dit as V  # noqa: E402


def main():
    dist.init_process_group("gloo", timeout=datetime.timedelta(seconds=120))
    rank, world = dist.get_rank(), dist.get_world_size()
    cfg = V.H3Config.tiny(heads=8, head_dim=64, ffn=1024, hidden=256)       # 8 heads x 64 = 512: shards of 256 channels
    g = torch.Generator().manual_seed(5)
    grid = (2, 2, 3)
    video, audio, prompt = torch.randn(12, cfg.latents, generator=g), torch.randn(4, cfg.audio_latents, generator=g), torch.randn(8, cfg.text_dim, generator=g)
    req = V.make_request(video, audio, prompt, grid, 0.7, 0.4)
    one = V.H3DiT(cfg).init_random(seed=3)
    want_v, want_a = one.forward(req)
    sp = V.H3DiT(cfg).init_random(seed=3)
    sp.set_sp(None, rank, world)
    got_v, got_a = sp.forward(req)
    assert torch.allclose(got_v, want_v, rtol=1e-4, atol=1e-5) and torch.allclose(got_a, want_a, rtol=1e-4, atol=1e-5), "sequence parallel"
    tp = V.H3DiT(cfg, tp_rank=rank, tp_ranks=world).init_random(seed=3)
    assert tp.blocks[0].qkv.out_features == 3 * cfg.heads * cfg.head_dim // world
    tv, ta = tp.forward(req)
    assert torch.allclose(tv, want_v, rtol=1e-3, atol=1e-4) and torch.allclose(ta, want_a, rtol=1e-3, atol=1e-4), "tensor parallel"
    # the sampler over the sequence-parallel model reproduces the single-rank latents
    a = V.denoise(one, prompt, grid, 4, steps=3, seed=1, pad_to=world)
    b = V.denoise(sp, prompt, grid, 4, steps=3, seed=1, pad_to=world)
    assert torch.allclose(a[0], b[0], rtol=1e-3, atol=1e-4) and torch.allclose(a[1], b[1], rtol=1e-3, atol=1e-4)
    dist.barrier()
    if rank == 0:
        print("H3_WORKER_OK", flush=True)
    dist.destroy_process_group()


if __name__ == "__main__":
    main()
