"""Models with multi-stream residuals (gated residual streams, hyper-connections): chunked prefill + decode agree with
one full forward on CPU; the GPU forward agrees with the CPU one."""
import pytest
import torch

from volta_engine_b200.models.dense import DenseConfig, DenseModel
from volta_engine_b200.models.util import to_device
from volta_engine_b200.runtime.batch import BatchRows
from volta_engine_b200.runtime.engine import Engine
from volta_engine_b200.runtime.kv_cache import PagedKVCache


def _model(residual, device="cpu", quant="bf16"):
    cfg = DenseConfig.tiny(vocab=512)
    cfg.residual, cfg.hc_rank, cfg.quant = residual, 32, quant
    return DenseModel(cfg, device).init_random(seed=2).init_stream_weights(seed=3)


def _prompt(n):
    return torch.randint(1, 500, (n,), generator=torch.Generator().manual_seed(1)).tolist()


@pytest.mark.parametrize("residual", ["gated", "hc"])
def test_chunked_prefill_and_decode_match_a_single_forward(residual):
    m = _model(residual)
    cfg = m.cfg
    p = _prompt(40)
    kv = PagedKVCache(cfg.n_layers, m.nkv, cfg.head_dim, 8, 1, 256, "cpu")
    kv.reserve(0, 64)
    full = m.forward(BatchRows.make(p, list(range(40)), [0] * 40, "cpu", "all", m.nq // m.nkv, prefill=True), kv)
    assert m.last_streams.shape[1] == 4 and m.last_streams.dtype == torch.float32
    kv2 = PagedKVCache(cfg.n_layers, m.nkv, cfg.head_dim, 8, 1, 256, "cpu")
    eng = Engine(m, kv2, use_graphs=False, prefill_chunk=16)
    first = eng.prefill(0, p)
    assert first == int(full[-1].argmax())
    # decode the same continuation row by row and compare with the teacher-forced rows of the full forward
    step = m.forward(BatchRows.make([p[20]], [20], [0], "cpu", "all", m.nq // m.nkv), kv)
    assert torch.allclose(step[0], full[20], atol=2e-2, rtol=2e-2)
    out, _ = Engine(m, PagedKVCache(cfg.n_layers, m.nkv, cfg.head_dim, 8, 1, 256, "cpu"), use_graphs=False).generate(p, 5)
    assert len(out) == 5


@pytest.mark.gpu
@pytest.mark.parametrize("residual,quant", [("gated", "bf16"), ("hc", "bf16"), ("gated", "nvfp4")])
def test_stream_model_gpu_matches_cpu(residual, quant):
    dev = torch.device("cuda:0")
    mg = _model(residual, dev, quant)
    mc = to_device(mg, "cpu")
    cfg = mg.cfg
    p = _prompt(40)
    kvg = PagedKVCache(cfg.n_layers, mg.nkv, cfg.head_dim, 8, 1, 256, dev)
    kvc = PagedKVCache(cfg.n_layers, mc.nkv, cfg.head_dim, 8, 1, 256, "cpu")
    kvg.reserve(0, 64)
    kvc.reserve(0, 64)
    G = mg.nq // mg.nkv
    lg = mg.forward(BatchRows.make(p, list(range(40)), [0] * 40, dev, "all", G, prefill=True), kvg)
    lc = mc.forward(BatchRows.make(p, list(range(40)), [0] * 40, "cpu", "all", G, prefill=True), kvc)
    a, b = lg.float().cpu().flatten(), lc.float().flatten()
    assert float(torch.dot(a, b) / (a.norm() * b.norm())) > 0.995
    sg = mg.forward(BatchRows.make([p[7]], [40], [0], dev, "all", G), kvg)           # a decode row through the mat-vec paths
    sc = mc.forward(BatchRows.make([p[7]], [40], [0], "cpu", "all", G), kvc)
    a, b = sg.float().cpu().flatten(), sc.float().flatten()
    assert float(torch.dot(a, b) / (a.norm() * b.norm())) > 0.995
    out, _ = Engine(mg, PagedKVCache(cfg.n_layers, mg.nkv, cfg.head_dim, 8, 1, 256, dev)).generate(p, 6)       # CUDA graphs
    assert len(out) == 6
