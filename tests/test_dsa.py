"""Sparse-attention indexer: list construction rules on CPU, kernels against the PyTorch statement, and a latent-attention
model that decodes over the indexer's list."""
import pytest
import torch

from volta_engine_b200.models.mla import MLAConfig, MLAModel
from volta_engine_b200.models.util import to_device
from volta_engine_b200.ops import dsa as D
from volta_engine_b200.ops.linear import LinearBF16
from volta_engine_b200.runtime.batch import BatchRows
from volta_engine_b200.runtime.engine import Engine
from volta_engine_b200.runtime.kv_cache import PagedKVCache


def test_select_rules():
    g = torch.Generator().manual_seed(0)
    assert D.select_reference(torch.zeros(10), 37) == list(range(37))                  # few pools: dense
    vis = 2600 * 4 + 2
    sc = torch.randn(2600, generator=g)
    sc[100], sc[7], sc[2000] = 9.0, 9.0, 9.0
    toks = D.select_reference(sc, vis)
    assert len(toks) == D.TOPK + 2 and toks[-2:] == [vis - 2, vis - 1]
    pools = [t // 4 for t in toks[:D.TOPK:4]]
    assert pools[:-1] == sorted(pools[:-1]) and {7, 100, 2000} <= set(pools)           # pool order (threshold pool last)
    assert toks[:4] == [pools[0] * 4 + j for j in range(4)]
    # ties at the threshold are taken in pool order
    tie = torch.zeros(1000)
    tie[500:] = 1.0                                                                     # 500 above, the rest tie at 0
    toks = D.select_reference(tie, 4000)
    pools = [t // 4 for t in toks[:D.TOPK:4]]
    assert pools == list(range(500, 1000)) + list(range(12))


def _weights(H, qlat, dev="cpu", seed=1):
    g = torch.Generator().manual_seed(seed)
    bf = torch.bfloat16
    return D.DSAWeights(proj=LinearBF16((torch.randn(D.PROJ, H, generator=g) * 0.2).to(bf).to(dev)),
                        q_proj=LinearBF16((torch.randn(D.HEADS * D.DIM, qlat, generator=g) * 0.2).to(bf).to(dev)),
                        ln_w=(1 + 0.1 * torch.randn(D.DIM, generator=g)).to(bf).to(dev),
                        ln_b=(0.1 * torch.randn(D.DIM, generator=g)).to(bf).to(dev),
                        ape=torch.randn(D.POOL, D.DIM, generator=g).to(bf).to(dev))


def test_short_context_model_with_indexer_equals_the_dense_model():
    cfg = MLAConfig.tiny_mla(vocab=256, mtp_layers=0, dsa=True)
    m = MLAModel(cfg, "cpu").init_random(seed=1)
    plain = to_device(m, "cpu")
    for L in plain.layers:
        L.dsa = None
    p = torch.randint(1, 250, (50,), generator=torch.Generator().manual_seed(2)).tolist()
    outs = []
    for mod in (m, plain):
        kv = PagedKVCache(cfg.n_layers, 1, 576, 8, 1, 256, "cpu", v_head_dim=8)
        out, _ = Engine(mod, kv, use_graphs=False, prefill_chunk=32).generate(p, 6)
        outs.append(out)
    assert outs[0] == outs[1]
    assert m.dsa_states and float(m.dsa_states[0].pools[0, :12].abs().sum()) > 0      # 50 tokens: 12 complete pools were built


# ------------------------------------------------------------------------------------------------ GPU
DEV = torch.device("cuda:0")


@pytest.mark.gpu
def test_indexer_kernels_match_reference():
    H, qlat, slots, max_seq = 512, 128, 2, 16384
    Wc, Wg = _weights(H, qlat), _weights(H, qlat, DEV)
    sc_, sg_ = D.DSAState(slots, max_seq, "cpu"), D.DSAState(slots, max_seq, DEV)
    g = torch.Generator().manual_seed(3)
    n0 = 3000                                                   # slot 0 holds positions 0..2999, slot 1 a short sequence
    x = (torch.randn(n0 + 40, H, generator=g)).to(torch.bfloat16)
    slot = torch.cat([torch.zeros(n0, dtype=torch.int32), torch.ones(40, dtype=torch.int32)])
    pos = torch.cat([torch.arange(n0, dtype=torch.int32), torch.arange(40, dtype=torch.int32)])
    wc = D.update(sc_, Wc, x, slot, pos)
    wg = D.update(sg_, Wg, x.to(DEV), slot.to(DEV), pos.to(DEV))
    assert torch.allclose(wg.cpu(), wc, atol=0.05, rtol=0.02)
    assert torch.allclose(sg_.pools.cpu().float(), sc_.pools.float(), atol=0.06, rtol=0.03)
    assert float(sc_.pools[0, n0 // 4 - 1].abs().sum()) > 0 and float(sc_.pools[0, n0 // 4].abs().sum()) == 0
    # scores of two query rows (same pooled keys on both sides so the comparison isolates the score kernel)
    sg_.pools.copy_(sc_.pools)
    q = torch.randn(3, D.HEADS * D.DIM, generator=g).to(torch.bfloat16)
    w = torch.randn(3, D.HEADS, generator=g)
    qs, qp = torch.tensor([0, 1, -1], dtype=torch.int32), torch.tensor([n0 - 1, 39, 0], dtype=torch.int32)
    want = D.score_reference(q[:2], w[:2], sc_, qs, qp)
    got = D.score(sg_, q.to(DEV), w.to(DEV), qs.to(DEV), qp.to(DEV)).cpu()
    for r in range(2):
        assert torch.allclose(got[r, :len(want[r])], want[r], atol=2e-3, rtol=2e-3), f"scores row {r}"
    # selection from the device scores: same list as the rule applied to those scores
    idx, nk = D.select_from_scores(got.to(DEV), qs.to(DEV), qp.to(DEV))
    assert nk.tolist() == [D.TOPK + n0 % 4, 40, 0]
    assert idx[0, :int(nk[0])].tolist() == D.select_reference(got[0], n0)
    assert idx[1, :40].tolist() == list(range(40))
    # ties and negative scores
    tie = torch.full((1, 4096), -1.0)
    tie[0, 500:1000] = 2.0
    tie[0, 3000] = -0.5
    i2, n2 = D.select_from_scores(tie.to(DEV), torch.zeros(1, dtype=torch.int32, device=DEV),
                                  torch.tensor([4096 * 4 - 1], dtype=torch.int32, device=DEV))
    assert i2[0, :int(n2[0])].tolist() == D.select_reference(tie[0], 4096 * 4)
    # gather into scratch pages
    pool = torch.randn(60, 1, 64, 576, generator=g).to(torch.bfloat16)
    table = torch.randperm(59, generator=g)[:50].to(torch.int32).reshape(1, 50) + 1
    scr_c = torch.zeros(D.PAGES_PER_ROW, 1, 64, 576, dtype=torch.bfloat16)
    scr_g = torch.zeros(D.PAGES_PER_ROW, 1, 64, 576, dtype=torch.bfloat16, device=DEV)
    s0 = torch.zeros(1, dtype=torch.int32)
    D.gather_rows(pool, table, s0, idx[:1].cpu(), nk[:1].cpu(), scr_c)
    D.gather_rows(pool.to(DEV), table.to(DEV), s0.to(DEV), idx[:1], nk[:1], scr_g)
    assert torch.equal(scr_g.cpu(), scr_c)


@pytest.mark.gpu
def test_latent_attention_model_decodes_over_the_indexer_list():
    cfg = MLAConfig.tiny_mla(vocab=256, mtp_layers=0, dsa=True)
    mg = MLAModel(cfg, DEV).init_random(seed=1)
    mc = to_device(mg, "cpu")
    n = 2300                                                   # more than 512 complete pools: the list is sparse
    p = torch.randint(1, 250, (n,), generator=torch.Generator().manual_seed(4)).tolist()
    kvg = PagedKVCache(cfg.n_layers, 1, 576, 48, 1, 4096, DEV, v_head_dim=8)
    kvc = PagedKVCache(cfg.n_layers, 1, 576, 48, 1, 4096, "cpu", v_head_dim=8)
    eg, ec = Engine(mg, kvg, prefill_chunk=1024), Engine(mc, kvc, use_graphs=False, prefill_chunk=1024)
    eg.prefill(0, p)
    ec.prefill(0, p)
    bg = BatchRows.make([p[5]], [n], [0], DEV, "all", 1, nsplit=2)
    bc = BatchRows.make([p[5]], [n], [0], "cpu", "all", 1)
    kvg.reserve(0, n + 8)
    kvc.reserve(0, n + 8)
    lg, lc = mg.forward(bg, kvg), mc.forward(bc, kvc)
    a, b = lg.float().cpu().flatten(), lc.float().flatten()
    assert float(torch.dot(a, b) / (a.norm() * b.norm())) > 0.99
    out, _ = Engine(mg, PagedKVCache(cfg.n_layers, 1, 576, 48, 1, 4096, DEV, v_head_dim=8), prefill_chunk=1024).generate(p, 5)
    assert len(out) == 5


# ------------------------------------------------------------------------------------------------ block-sparse indexer
def _qsa_weights(H, dev="cpu", seed=2):
    g = torch.Generator().manual_seed(seed)
    bf = torch.bfloat16
    return D.QSAWeights(proj=LinearBF16((torch.randn(5 * D.DIM, H, generator=g) * 0.2).to(bf).to(dev)),
                        q_norm=(0.1 * torch.randn(D.DIM, generator=g)).to(bf).to(dev),
                        k_norm=(0.1 * torch.randn(D.DIM, generator=g)).to(bf).to(dev), rot=64, theta=1e4)


def test_hybrid_model_with_block_sparse_indexer_equals_dense_on_short_context():
    from volta_engine_b200.models.hybrid import HybridConfig, HybridModel
    cfg = HybridConfig.tiny_hybrid(vocab=256, qsa=True)
    m = HybridModel(cfg, "cpu").init_random(seed=1)
    plain = to_device(m, "cpu")
    for L in plain.layers:
        L.qsa = None
    p = torch.randint(1, 250, (50,), generator=torch.Generator().manual_seed(2)).tolist()
    outs = []
    for mod in (m, plain):
        kv = PagedKVCache(mod.kv_layers, mod.nkv, cfg.head_dim, 8, 1, 256, "cpu")
        out, _ = Engine(mod, kv, use_graphs=False, prefill_chunk=32).generate(p, 6)
        outs.append(out)
    assert outs[0] == outs[1] and m.qsa_states


@pytest.mark.gpu
def test_block_sparse_indexer_kernels_and_model():
    H, slots, max_seq = 256, 2, 8192
    Wc, Wg = _qsa_weights(H), _qsa_weights(H, DEV)
    sc_, sg_ = D.QSAState(slots, max_seq, "cpu"), D.QSAState(slots, max_seq, DEV)
    g = torch.Generator().manual_seed(5)
    n0 = 2500
    x = torch.randn(n0, H, generator=g).to(torch.bfloat16)
    slot = torch.ones(n0, dtype=torch.int32)
    pos = torch.arange(n0, dtype=torch.int32)
    qc = D.qsa_update(sc_, Wc, x, slot, pos)
    qg = D.qsa_update(sg_, Wg, x.to(DEV), slot.to(DEV), pos.to(DEV))
    assert torch.allclose(qg.cpu().float(), qc.float(), atol=0.06, rtol=0.03)
    assert torch.allclose(sg_.pools.cpu().float(), sc_.pools.float(), atol=0.06, rtol=0.03)
    assert torch.allclose(sg_.ring.cpu().float(), sc_.ring.float(), atol=0.06, rtol=0.03)
    sg_.pools.copy_(sc_.pools)
    qs, qp = torch.ones(1, dtype=torch.int32), torch.tensor([n0 - 1], dtype=torch.int32)
    want = D.qsa_score_reference(qc[-1:], sc_, qs, qp)[0]
    got = D.score(sg_, qc[-1:].to(DEV), None, qs.to(DEV), qp.to(DEV)).cpu()[0, :len(want)]
    assert torch.allclose(got, want, atol=2e-3, rtol=2e-3)
    idx, nk = D.qsa_select(sg_, qc[-1:].to(DEV), qs.to(DEV), qp.to(DEV))
    assert int(nk[0]) == D.TOPK + n0 % 4 and idx[0, :int(nk[0])].tolist() == D.select_reference(got, n0)
    # gather with several kv heads
    pool = torch.randn(50, 2, 64, 64, generator=g).to(torch.bfloat16)
    table = (torch.randperm(49, generator=g)[:40].to(torch.int32) + 1).reshape(1, 40).repeat(2, 1)
    scr_c = torch.zeros(D.PAGES_PER_ROW, 2, 64, 64, dtype=torch.bfloat16)
    scr_g = scr_c.to(DEV)
    D.gather_rows(pool, table, qs, idx.cpu(), nk.cpu(), scr_c)
    D.gather_rows(pool.to(DEV), table.to(DEV), qs.to(DEV), idx, nk, scr_g)
    assert torch.equal(scr_g.cpu(), scr_c)
    # a hybrid model decoding a row past 2048 tokens: GPU and CPU agree on the logits
    from volta_engine_b200.models.hybrid import HybridConfig, HybridModel
    cfg = HybridConfig.tiny_hybrid(vocab=256, qsa=True)
    mg = HybridModel(cfg, DEV).init_random(seed=1)
    mc = to_device(mg, "cpu")
    n = 2200
    p = torch.randint(1, 250, (n,), generator=torch.Generator().manual_seed(4)).tolist()
    kvg = PagedKVCache(mg.kv_layers, mg.nkv, cfg.head_dim, 48, 1, 4096, DEV)
    kvc = PagedKVCache(mc.kv_layers, mc.nkv, cfg.head_dim, 48, 1, 4096, "cpu")
    eg, ec = Engine(mg, kvg, prefill_chunk=1024), Engine(mc, kvc, use_graphs=False, prefill_chunk=1024)
    tg, tc = eg.prefill(0, p), ec.prefill(0, p)
    G = mg.nq // mg.nkv
    kvg.reserve(0, n + 8)
    kvc.reserve(0, n + 8)
    lg = mg.forward(BatchRows.make([p[5]], [n], [0], DEV, "all", G, nsplit=2), kvg)
    lc = mc.forward(BatchRows.make([p[5]], [n], [0], "cpu", "all", G), kvc)
    a, b = lg.float().cpu().flatten(), lc.float().flatten()
    assert float(torch.dot(a, b) / (a.norm() * b.norm())) > 0.99
