"""Child process of tests/test_gdn.py: one CPU rank of a 2-rank gloo world running the tiny hybrid (GDN or KDA + gated
attention) model tensor parallel."""
import datetime
import os
import sys

import torch
import torch.distributed as dist

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))

from volta_engine_b200.models.hybrid import HybridConfig, HybridModel  # noqa: E402
from volta_engine_b200.parallel.host import HostComm  # noqa: E402
from volta_engine_b200.runtime.batch import BatchRows, LOGITS_ALL  # noqa: E402
from volta_engine_b200.runtime.kv_cache import PagedKVCache  # noqa: E402


def main():
    out_path, mixer = sys.argv[1], sys.argv[2]
    rank, world = int(os.environ["RANK"]), int(os.environ["WORLD_SIZE"])
    store = dist.TCPStore("127.0.0.1", int(os.environ["MASTER_PORT"]), world, rank == 0, timeout=datetime.timedelta(seconds=60))
    dist.init_process_group("gloo", store=store, rank=rank, world_size=world, timeout=datetime.timedelta(seconds=60))
    if mixer == "glm5":             # KDA mixers + latent attention: the GLM-5-Next-style assembly
        from volta_engine_b200.models.glm5 import Glm5NextConfig, Glm5NextModel
        cfg = Glm5NextConfig.tiny_glm5(vocab=256, gdn_k_heads=4, gdn_v_heads=4)
        m = Glm5NextModel(cfg, "cpu", HostComm()).init_random(seed=0, search=False)
        kv = m.make_cache(16, 2, 512)
    else:
        kw = {"linear_mixer": "kda", "gdn_k_heads": 4} if mixer == "kda" else {}
        cfg = HybridConfig.tiny_hybrid(vocab=256, **kw)
        m = HybridModel(cfg, "cpu", HostComm()).init_random(seed=0, search=False)
        kv = PagedKVCache(m.kv_layers, m.nkv, cfg.head_dim, 16, 2, 512, "cpu")
    toks = torch.randint(0, 256, (40,), generator=torch.Generator().manual_seed(11)).tolist()
    kv.reserve(0, 64)
    outs = []
    for lo, hi in ((0, 30), (30, 34), (34, 35), (35, 40)):          # a prefill chunk, verify rows, one decode row, more rows
        b = BatchRows.make(toks[lo:hi], list(range(lo, hi)), [0] * (hi - lo), "cpu", LOGITS_ALL, m.nq // m.nkv, prefill=hi - lo > 16)
        outs.append(m.forward(b, kv).float())
    torch.save({"rank": rank, "logits": torch.cat(outs), "heads": (m.dims.n_k, m.dims.n_v)}, f"{out_path}.{rank}")
    dist.barrier()
    dist.destroy_process_group()


if __name__ == "__main__":
    main()
