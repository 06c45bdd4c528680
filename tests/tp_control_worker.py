"""Child process of tests/test_tp_control.py: one CPU rank of a 2-rank gloo world."""
import datetime
import json
import os
import sys
import time

import torch
import torch.distributed as dist

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))

from volta_engine_b200.models.dense import DenseConfig, DenseModel  # noqa: E402
from volta_engine_b200.parallel.host import HostComm  # noqa: E402
from volta_engine_b200.runtime.engine import Engine  # noqa: E402
from volta_engine_b200.runtime.generator import Generator, Request  # noqa: E402
from volta_engine_b200.runtime.kv_cache import PagedKVCache  # noqa: E402
from volta_engine_b200.runtime.options import Options  # noqa: E402
from volta_engine_b200.runtime.prefix_cache import PrefixCache  # noqa: E402
from volta_engine_b200.runtime.tp_control import (ControlChannel, Heartbeat, LeaderEngine, RankFailure,  # noqa: E402
                                                  follower_loop)


class ByteTok:
    eos_ids = [0]

    def decode_bytes(self, ids, skip_special=False):
        return bytes(i & 0xFF for i in ids)

    def encode(self, text, allow_special=True):
        return list(text.encode())


def main():
    mode, out_path = sys.argv[1], sys.argv[2]
    rank, world = int(os.environ["RANK"]), int(os.environ["WORLD_SIZE"])
    store = dist.TCPStore("127.0.0.1", int(os.environ["MASTER_PORT"]), world, rank == 0,
                          timeout=datetime.timedelta(seconds=30))
    dist.init_process_group("gloo", store=store, rank=rank, world_size=world, timeout=datetime.timedelta(seconds=4))
    hb = Heartbeat(store, rank, world, period_s=0.1, timeout_s=1.0).start()
    cfg = DenseConfig.tiny(vocab=256)
    model = DenseModel(cfg, "cpu", HostComm()).init_random(seed=0, search=False)
    kv = PagedKVCache(cfg.n_layers, model.nkv, cfg.head_dim, 40, 2, 512, "cpu")
    eng = Engine(model, kv, use_graphs=False, prefill_chunk=32)
    chan = ControlChannel(heartbeat=hb if rank == 0 else None)
    result = {"rank": rank, "mode": mode}
    dist.barrier()
    if mode == "serve":
        if rank == 0:
            lead = LeaderEngine(eng, chan)
            gen = Generator(lead, ByteTok(), Options.resolve({"max_slots": 2, "prefix_interval": 64}, env={}),
                            prefix_cache=PrefixCache(64 << 20), eos_ids=[])
            prompt = [(7 * i + 3) % 256 for i in range(150)]
            a = gen.generate(Request(prompt=prompt, max_tokens=6))
            b = gen.generate(Request(prompt=prompt + a["tokens"] + [5, 6], max_tokens=4))   # resumes from a snapshot
            result.update(tokens=a["tokens"], tokens2=b["tokens"], cached=b["usage"].get("cached_tokens", 0))
            lead.shutdown()
        else:
            result["commands"] = follower_loop(eng, chan)
    elif mode == "drafter":
        # tensor-parallel block drafter: the leader's generator drafts through LeaderDrafter, the follower mirrors it
        from volta_engine_b200.runtime import dflash_runner as DF
        from volta_engine_b200.runtime.tp_control import LeaderDrafter
        dc = DF.DFlashConfig(block_size=4, n_layers=2, hidden=cfg.hidden, n_q=cfg.n_q, n_kv=cfg.n_kv, head_dim=cfg.head_dim,
                             ffn=cfg.ffn, target_layer_ids=(0, cfg.n_layers - 1), sliding_window=64, rope_theta=1e4,
                             mask_token_id=255, tap_cap=64, quant="bf16")
        runner = DF.DFlashRunner(eng, dc)
        eng.drafter = runner
        result["drafter_tp"] = runner.model.comm.size
        if rank == 0:
            lead = LeaderEngine(eng, chan)
            o = Options.resolve({"max_slots": 2, "prefix_interval": 0, "speculator": "draft", "spec_ctrl": False, "spec_depth": 3}, env={})
            gen = Generator(lead, ByteTok(), o, eos_ids=[])
            gen.drafter = LeaderDrafter(runner, lead)
            prompt = [(7 * i + 3) % 255 + 1 for i in range(45)]
            a = gen.generate(Request(prompt=prompt, max_tokens=10, cache_prefix=False))
            result.update(tokens=a["tokens"], rounds=gen.metrics.spec["rounds"], proposed=gen.metrics.spec["proposed"])
            lead.shutdown()
        else:
            seen = []
            result["commands"] = follower_loop(eng, chan, on_command=lambda n, a, k: seen.append(n))
            result["drafter_calls"] = sum(1 for n in seen if n.startswith("drafter."))
    elif mode == "follower_dies":
        # the follower leaves between steps (no kernel or collective in flight); the leader must notice on the host
        if rank == 0:
            lead = LeaderEngine(eng, chan)
            lead.prefill_rows(0, list(range(20)), 0, True)
            time.sleep(2.0)
            try:
                lead.step([1], [20], [0])
                result["error"] = None
            except RankFailure as e:
                result["error"] = str(e)
        else:
            (name, a, k), _ = chan.recv()
            getattr(eng, name)(*a, **k)
            hb.stop()
            result["left"] = True
            with open(out_path + f".{rank}", "w") as f:
                json.dump(result, f)
            os._exit(0)
    elif mode == "leader_dies":
        if rank == 0:
            lead = LeaderEngine(eng, chan)
            lead.prefill_rows(0, list(range(20)), 0, True)
            result["left"] = True
            with open(out_path + f".{rank}", "w") as f:
                json.dump(result, f)
            os._exit(0)
        else:
            try:
                follower_loop(eng, chan)
                result["error"] = None
            except RankFailure as e:
                result["error"] = str(e)
    with open(out_path + f".{rank}", "w") as f:
        json.dump(result, f)
    hb.stop()
    os._exit(0)          # skip the process-group teardown: a peer may already be gone


if __name__ == "__main__":
    main()
