"""Child process of tests/test_dsv4.py: one CPU rank of a 2-rank gloo world running the tiny DeepSeek-V4.1-style model."""
import datetime
import os
import sys

import torch
import torch.distributed as dist

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))

from volta_engine_b200.models.dsv4 import DSV4Config, DSV4Model  # noqa: E402
from volta_engine_b200.parallel.host import HostComm  # noqa: E402
from volta_engine_b200.runtime.batch import BatchRows, LOGITS_ALL  # noqa: E402
from volta_engine_b200.runtime.kv_cache import PagedKVCache  # noqa: E402


def main():
    out_path = sys.argv[1]
    rank, world = int(os.environ["RANK"]), int(os.environ["WORLD_SIZE"])
    store = dist.TCPStore("127.0.0.1", int(os.environ["MASTER_PORT"]), world, rank == 0, timeout=datetime.timedelta(seconds=60))
    dist.init_process_group("gloo", store=store, rank=rank, world_size=world, timeout=datetime.timedelta(seconds=60))
    cfg = DSV4Config.tiny_dsv4()
    m = DSV4Model(cfg, "cpu", HostComm()).init_random(seed=5, std=0.05)
    kv = PagedKVCache(1, 1, 64, 16, 2, 512, "cpu")
    g = torch.Generator().manual_seed(11)
    toks = torch.randint(0, 1024, (48,), generator=g).tolist()
    kv.reserve(0, 64)
    outs = []
    for lo, hi in ((0, 40), (40, 48)):
        b = BatchRows.make(toks[lo:hi], list(range(lo, hi)), [0] * (hi - lo), "cpu", LOGITS_ALL, m.nq, prefill=True)
        outs.append(m.forward(b, kv).float())
    torch.save({"rank": rank, "logits": torch.cat(outs), "heads": m.heads, "groups": m.groups, "e_local": m.e_local}, f"{out_path}.{rank}")
    dist.barrier()
    dist.destroy_process_group()


if __name__ == "__main__":
    main()
