"""Child process of tests/test_tools.py: one CPU rank of a gloo world running the sequence-parallel training form of
volta_e2e against the single-rank form (loss, gradients, a few optimiser steps)."""
import datetime
import os
import sys

import torch
import torch.distributed as dist

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))

from volta_engine_b200.models.dense import DenseConfig, DenseModel  # noqa: E402
from volta_engine_b200.tools import e2e as E  # noqa: E402


def main():
    dist.init_process_group("gloo", timeout=datetime.timedelta(seconds=120))
    rank, world = dist.get_rank(), dist.get_world_size()
    torch.manual_seed(0)
    cfg = DenseConfig(n_layers=2, hidden=64, n_q=4, n_kv=2, head_dim=16, ffn=128, vocab=96, quant="bf16")
    model = DenseModel(cfg, "cpu").init_random(seed=3, std=0.08, search=False)
    g = torch.Generator().manual_seed(1)
    seqs = [torch.randint(0, cfg.vocab, (24,), generator=g) for _ in range(3)]
    teachers = [torch.randn(24, cfg.vocab, generator=g) for _ in range(3)]

    one = E.build_from_engine_model(model)
    sp = E.TunedModelSP(E.build_from_engine_model(model), rank, world)
    # --- one loss and its gradients
    one.train()
    sp.train()
    loss1 = E.kl_teacher(one(seqs[0]), teachers[0])
    loss1.backward()
    rows = sp.rows(24)
    loss_sp = E.kl_teacher(sp(seqs[0]), teachers[0][rows]) / world
    loss_sp.backward()
    sp.sync_grads()
    tot = loss_sp.detach().clone()
    dist.all_reduce(tot)
    assert torch.allclose(tot, loss1.detach(), rtol=1e-5, atol=1e-7), (float(tot), float(loss1))
    L1, Ls = one.layers[1], sp.layers[1]
    assert torch.allclose(Ls.n1.delta.grad, L1.n1.delta.grad, rtol=1e-3, atol=1e-7), "replicated norm gradient"
    assert torch.allclose(Ls.qkv.a_u.grad, L1.qkv.a_u.grad, rtol=1e-3, atol=1e-7), "replicated input-scale gradient"
    assert torch.allclose(Ls.o.a_v.grad, L1.o.a_v.grad, rtol=1e-3, atol=1e-7), "replicated output-scale gradient"
    hd, nq = cfg.head_dim, cfg.n_q // world
    q = slice(rank * nq * hd, (rank + 1) * nq * hd)
    assert torch.allclose(Ls.qkv.a_v.grad[: nq * hd], L1.qkv.a_v.grad[q], rtol=1e-3, atol=1e-7), "sharded output-scale gradient"
    assert torch.allclose(Ls.o.a_u.grad, L1.o.a_u.grad[q], rtol=1e-3, atol=1e-7), "sharded input-scale gradient"
    f = cfg.ffn // world
    assert torch.allclose(Ls.dn.a_u.grad, L1.dn.a_u.grad[rank * f:(rank + 1) * f], rtol=1e-3, atol=1e-7)
    # --- the tuning loop: the same held-out KL trajectory as the single-rank form
    o = E.E2EOptions(steps=4, batch=2, lr=5e-3, warmup=1, eval_every=2)
    h1 = E.tune(E.build_from_engine_model(model), seqs, teachers, o, log=lambda *_: None)
    hs = E.tune(E.TunedModelSP(E.build_from_engine_model(model), rank, world), seqs, teachers, o, log=lambda *_: None)
    for (s1, k1), (s2, k2) in zip(h1["eval"], hs["eval"]):
        assert s1 == s2 and abs(k1 - k2) < 2e-4 * max(1.0, abs(k1)), (h1["eval"], hs["eval"])
    assert hs["eval"][-1][1] < hs["eval"][0][1]
    # --- the scales put back into whole vectors
    spm = E.TunedModelSP(E.build_from_engine_model(model), rank, world)
    whole = E.gather_tuned_model(spm)
    su, sv = whole.layers[0].qkv.tuned_scales()
    assert su.shape[0] == cfg.hidden and sv.shape[0] == (cfg.n_q + 2 * cfg.n_kv) * cfg.head_dim
    assert whole.layers[0].dn.tuned_scales()[0].shape[0] == cfg.ffn
    dist.barrier()
    if rank == 0:
        print("E2E_SP_OK", flush=True)
    dist.destroy_process_group()


if __name__ == "__main__":
    main()
