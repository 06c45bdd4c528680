"""Scaled KV cache formats (k8v4: int8 keys + 4-bit rotated values; nvfp4: E2M1 with E4M3 scales): codec properties and a
CPU engine over the quantised cache; on a GPU the quantising store and attention over the byte cache against the
PyTorch codecs reading the same bytes."""
import math

import pytest
import torch

from volta_engine_b200.models.dense import DenseConfig, DenseModel
from volta_engine_b200.ops import kernels as K
from volta_engine_b200.ops import reference as ref
from volta_engine_b200.quant import kv_codec as C
from volta_engine_b200.runtime.engine import Engine
from volta_engine_b200.runtime.kv_cache import PagedKVCache


def test_codecs_round_trip_within_their_step():
    g = torch.Generator().manual_seed(0)
    x = torch.randn(4, 3, 128, generator=g)
    assert torch.allclose(C.fwht64(C.fwht64(x.reshape(4, 3, 2, 64))).reshape(4, 3, 128), x, atol=1e-5)
    for q, rel in ((C.Q_I8, 0.01), (C.Q_Q4, 0.15), (C.Q_FP4, 0.13)):
        d, s = C.encode(x, q)
        assert d.shape[-1] == C.data_bytes(q, 128) and s.shape[-1] == C.scale_bytes(q, 128) and d.dtype == torch.uint8
        y = C.decode(d, s, q, 128)
        assert float((y - x).norm() / x.norm()) < rel
    z = torch.zeros(2, 64)
    for q in (C.Q_I8, C.Q_Q4, C.Q_FP4):
        assert float(C.decode(*C.encode(z, q), q, 64).abs().sum()) == 0      # zero scale: zero, not NaN


@pytest.mark.parametrize("fmt", ["k8v4", "nvfp4"])
def test_engine_over_a_quantised_cache_on_cpu(fmt):
    cfg = DenseConfig.tiny(vocab=256)
    cfg.quant = "bf16"
    m = DenseModel(cfg, "cpu").init_random(seed=0)
    p = torch.randint(1, 250, (70,), generator=torch.Generator().manual_seed(1)).tolist()
    kv_ref = PagedKVCache(cfg.n_layers, m.nkv, cfg.head_dim, 8, 1, 256, "cpu")
    kv_q = PagedKVCache(cfg.n_layers, m.nkv, cfg.head_dim, 8, 1, 256, "cpu", dtype=fmt)
    assert kv_q.bytes_per_token() < 0.5 * kv_ref.bytes_per_token()
    from volta_engine_b200.runtime.batch import BatchRows
    G = m.nq // m.nkv
    outs = []
    for kv in (kv_ref, kv_q):
        kv.reserve(0, 128)
        outs.append(m.forward(BatchRows.make(p, list(range(70)), [0] * 70, "cpu", "all", G, prefill=True), kv))
    a, b = outs[0].flatten(), outs[1].flatten()
    assert float(torch.dot(a, b) / (a.norm() * b.norm())) > 0.98
    out, _ = Engine(m, PagedKVCache(cfg.n_layers, m.nkv, cfg.head_dim, 8, 1, 256, "cpu", dtype=fmt), use_graphs=False,
                    prefill_chunk=32).generate(p, 5)
    assert len(out) == 5
    snap = kv_q.save_rows(0, 0, 70)                     # snapshots carry the scale pools
    kv2 = PagedKVCache(cfg.n_layers, m.nkv, cfg.head_dim, 8, 1, 256, "cpu", dtype=fmt)
    kv2.load_rows(0, snap)
    pg, pg2 = int(kv_q.host_table[0, 0]), int(kv2.host_table[0, 0])
    assert torch.equal(kv2.ks[:, pg2], kv_q.ks[:, pg]) and torch.equal(kv2.v[:, pg2], kv_q.v[:, pg])


# ------------------------------------------------------------------------------------------------ GPU
DEV = torch.device("cuda:0")


def _pools(fmt, pages, nkv, hd, dev):
    kv = PagedKVCache(1, nkv, hd, pages, 4, 2048, dev, dtype=fmt)
    return kv, kv.layer(0)


@pytest.mark.gpu
@pytest.mark.parametrize("fmt", ["k8v4", "nvfp4"])
@pytest.mark.parametrize("hd,nq,nkv", [(128, 40, 8), (256, 16, 2)])
def test_store_and_attention_over_the_scaled_cache(fmt, hd, nq, nkv):
    g = torch.Generator().manual_seed(3)
    n = 300
    kvc, (kc, vc) = _pools(fmt, 24, nkv, hd, "cpu")
    kvg, (kg, vg) = _pools(fmt, 24, nkv, hd, DEV)
    for kv in (kvc, kvg):
        kv.reserve(1, n + 1)
    assert torch.equal(kvc.host_table, kvg.host_table)
    qkv = (torch.randn(n, (nq + 2 * nkv) * hd, generator=g) * 0.8).to(torch.bfloat16)
    pos = torch.arange(n, dtype=torch.int32)
    slot = torch.ones(n, dtype=torch.int32)
    qc, qg = qkv.clone(), qkv.clone().to(DEV)
    K.rope_store(qc, pos, slot, kvc.page_table, kc, vc, nq, nkv, hd, hd, 1e6, False)
    K.rope_store(qg, pos.to(DEV), slot.to(DEV), kvg.page_table, kg, vg, nq, nkv, hd, hd, 1e6, False)
    kq, vq = C.FORMATS[kvc.fmt]
    # values are not rotated by rope: the stored values equal the codec's up to a code step where the butterfly's fp32
    # rounding moved a scale or a tie
    dv_c, dv_g = C.decode(vc, vc.kv_scale, vq, hd), C.decode(vg.cpu(), vg.kv_scale.cpu(), vq, hd)
    assert float((dv_g - dv_c).norm() / dv_c.norm()) < 0.02
    assert float((vg.kv_scale.cpu() != vc.kv_scale).float().mean()) < 0.02
    dk_c, dk_g = C.decode(kc, kc.kv_scale, kq, hd), C.decode(kg.cpu(), kg.kv_scale.cpu(), kq, hd)
    assert float((dk_g - dk_c).norm() / dk_c.norm()) < 0.02                   # rope rounding can move a code by one step
    # attention reads the same bytes on both sides
    for t in (kc, vc):
        pass
    kg.copy_(kc.to(DEV)), vg.copy_(vc.to(DEV))
    kg.kv_scale.copy_(kc.kv_scale.to(DEV)), vg.kv_scale.copy_(vc.kv_scale.to(DEV))
    rows_pos = torch.tensor([0, 63, 64, 200, n - 1, 5], dtype=torch.int32)
    rows_slot = torch.tensor([1, 1, 1, 1, 1, -1], dtype=torch.int32)
    q = (torch.randn(6, (nq + 2 * nkv) * hd, generator=g)).to(torch.bfloat16)
    scale = 1 / math.sqrt(hd)
    want = K.attention(q, rows_pos, rows_slot, kvc.page_table, kc, vc, nq, nkv, hd, scale)
    ws = K.AttnWorkspace(6, nq, hd, 8, DEV)
    for nsplit in (1, 3):
        got = K.attention(q.to(DEV), rows_pos.to(DEV), rows_slot.to(DEV), kvg.page_table, kg, vg, nq, nkv, hd, scale,
                          nsplit=nsplit, ws=ws)
        a, b = got[:5].float().cpu().flatten(), want[:5].float().flatten()
        assert float(torch.dot(a, b) / (a.norm() * b.norm())) > 0.999, f"{fmt} decode nsplit={nsplit}"
        assert float((a - b).abs().max()) < 0.05
    # a prefill tile over the same cache
    G = nq // nkv
    pp, ps = torch.arange(100, 140, dtype=torch.int32), torch.ones(40, dtype=torch.int32)
    qp = (torch.randn(40, (nq + 2 * nkv) * hd, generator=g)).to(torch.bfloat16)
    wantp = K.attention(qp, pp, ps, kvc.page_table, kc, vc, nq, nkv, hd, scale)
    tiles = K.make_prefill_tiles([1] * 40, G, DEV)
    gotp = K.attention(qp.to(DEV), pp.to(DEV), ps.to(DEV), kvg.page_table, kg, vg, nq, nkv, hd, scale, tiles=tiles)
    a, b = gotp.float().cpu().flatten(), wantp.float().flatten()
    assert float(torch.dot(a, b) / (a.norm() * b.norm())) > 0.999 and float((a - b).abs().max()) < 0.05
    assert K.check_status(DEV) == 0


@pytest.mark.gpu
@pytest.mark.parametrize("fmt", ["k8v4", "nvfp4"])
def test_engine_with_a_scaled_cache_on_the_gpu(fmt):
    from volta_engine_b200.runtime.batch import BatchRows
    cfg = DenseConfig(n_layers=2, hidden=512, n_q=8, n_kv=2, head_dim=128, ffn=1024, vocab=1024)
    m = DenseModel(cfg, DEV).init_random(seed=3)
    p = torch.randint(1, 1000, (200,), generator=torch.Generator().manual_seed(1)).tolist()
    G = m.nq // m.nkv
    logits = []
    for dt in (torch.bfloat16, fmt):
        kv = PagedKVCache(cfg.n_layers, m.nkv, cfg.head_dim, 16, 1, 512, DEV, dtype=dt)
        eng = Engine(m, kv, prefill_chunk=64)
        eng.prefill(0, p)
        kv.reserve(0, 210)
        lg = m.forward(BatchRows.make([p[3]], [200], [0], DEV, "all", G, nsplit=2), kv)       # a decode row over the cache
        logits.append(lg.float().cpu().flatten())
        out, _ = Engine(m, PagedKVCache(cfg.n_layers, m.nkv, cfg.head_dim, 16, 1, 512, DEV, dtype=dt), prefill_chunk=64).generate(p, 8)
        assert len(out) == 8                                   # CUDA-graph decode over the format
    a, b = logits
    assert float(torch.dot(a, b) / (a.norm() * b.norm())) > 0.97
    assert K.check_status(DEV) == 0
