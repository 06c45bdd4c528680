"""Training primitives: central-difference gradient checks on the CPU forms, Adam parameterisations, and the CUDA
kernels against the CPU forms."""
import pytest
import torch

from volta_engine_b200.train import grad as G


def _num_grad(f, x, eps=1e-3):
    g = torch.zeros_like(x)
    flat, gf = x.view(-1), g.view(-1)
    for i in range(flat.numel()):
        old = float(flat[i])
        flat[i] = old + eps; up = f()
        flat[i] = old - eps; dn = f()
        flat[i] = old
        gf[i] = (up - dn) / (2 * eps)
    return g


def test_swiglu_backward_matches_central_differences():
    gen = torch.Generator().manual_seed(0)
    for limit in (0.0, 1.0):
        g, u = torch.randn(3, 5, generator=gen, dtype=torch.float64) * 2, torch.randn(3, 5, generator=gen, dtype=torch.float64) * 2
        da = torch.randn(3, 5, generator=gen, dtype=torch.float64)
        dg, du = G.swiglu_backward(g, u, da, limit)
        ng = _num_grad(lambda: float((G.swiglu_forward(g, u, limit) * da).sum()), g, 1e-5)
        nu = _num_grad(lambda: float((G.swiglu_forward(g, u, limit) * da).sum()), u, 1e-5)
        assert torch.allclose(dg, ng, atol=1e-5) and torch.allclose(du, nu, atol=1e-5)


def test_scaled_linear_gradients():
    gen = torch.Generator().manual_seed(1)
    k, n, rows = 6, 4, 5
    T = torch.randn(k, n, generator=gen, dtype=torch.float64)
    su, sv = torch.rand(k, generator=gen, dtype=torch.float64) + 0.5, torch.rand(n, generator=gen, dtype=torch.float64) + 0.5
    X = torch.randn(rows, k, generator=gen, dtype=torch.float64)
    tgt = torch.randn(rows, n, generator=gen, dtype=torch.float64)
    w = torch.rand(rows, generator=gen, dtype=torch.float64)
    l = G.ScaledLinear(T, su, sv, torch.zeros(k, dtype=torch.float64), torch.zeros(n, dtype=torch.float64))

    def loss():
        return G.weighted_sq_error(G.scaled_linear_forward(l, X)[0], tgt, w)[0]
    Y, Z = G.scaled_linear_forward(l, X)
    _, dY = G.weighted_sq_error(Y, tgt, w, want_dy=True)
    dX = G.scaled_linear_backward(l, X, Z, dY)
    assert torch.allclose(l.dsu, _num_grad(loss, su, 1e-6), atol=1e-5)
    assert torch.allclose(l.dsv, _num_grad(loss, sv, 1e-6), atol=1e-5)
    assert torch.allclose(dX, _num_grad(loss, X, 1e-6), atol=1e-5)
    assert abs(G.weighted_sq_norm(tgt, w) - float(((tgt ** 2).sum(1) * w).sum())) < 1e-9


def test_adam_parameterisations_descend():
    o = G.AdamOptions(lr=0.05)
    # plain: minimise |p - 3|^2
    p, m, v = torch.zeros(4), torch.zeros(4), torch.zeros(4)
    for step in range(1, 300):
        G.adam_step(p, 2 * (p - 3.0), m, v, step, o)
    assert torch.allclose(p, torch.full((4,), 3.0), atol=0.05)
    # log-scale: s = s0 e^a towards 2
    s0, a, s, m, v = torch.ones(4), torch.zeros(4), torch.ones(4), torch.zeros(4), torch.zeros(4)
    for step in range(1, 400):
        G.adam_log_scales(s0, a, s, 2 * (s - 2.0), m, v, step, 1.0, o)
    assert torch.allclose(s, torch.full((4,), 2.0), atol=0.05) and torch.allclose(s, s0 * torch.exp(a))
    # additive: w = w0 + a towards -1
    w0, a, w, m, v = torch.ones(4), torch.zeros(4), torch.ones(4), torch.zeros(4), torch.zeros(4)
    for step in range(1, 400):
        G.adam_deltas(w0, a, w, 2 * (w + 1.0), m, v, step, 1.0, o)
    assert torch.allclose(w, torch.full((4,), -1.0), atol=0.05) and torch.allclose(w, w0 + a)
    # first step of plain Adam moves every parameter by lr against the gradient's sign
    p, m, v = torch.zeros(3), torch.zeros(3), torch.zeros(3)
    G.adam_step(p, torch.tensor([1.0, -2.0, 0.5]), m, v, 1, G.AdamOptions(lr=0.1))
    assert torch.allclose(p, torch.tensor([-0.1, 0.1, -0.1]), atol=1e-5)


def test_gather_scatter():
    src = torch.arange(12.0).reshape(4, 3)
    idx = torch.tensor([2, 0], dtype=torch.int32)
    w = torch.tensor([2.0, 0.5])
    got = G.gather_rows(src, idx, w)
    assert torch.equal(got, torch.stack([src[2] * 2, src[0] * 0.5]))
    dst = torch.zeros(4, 3)
    G.scatter_add_rows_(dst, got, idx, w)
    assert torch.equal(dst[2], src[2] * 4) and torch.equal(dst[0], src[0] * 0.25) and float(dst[1].abs().sum()) == 0


@pytest.mark.gpu
def test_gpu_kernels_match_cpu_forms():
    dev = torch.device("cuda:0")
    gen = torch.Generator().manual_seed(2)
    g, u, da = (torch.randn(7, 33, generator=gen) * 2 for _ in range(3))
    for limit in (0.0, 1.5):
        assert torch.allclose(G.swiglu_forward(g.to(dev), u.to(dev), limit).cpu(), G.swiglu_forward(g, u, limit), atol=1e-5)
        dg, du = G.swiglu_backward(g.to(dev), u.to(dev), da.to(dev), limit)
        rg, ru = G.swiglu_backward(g, u, da, limit)
        assert torch.allclose(dg.cpu(), rg, atol=1e-5) and torch.allclose(du.cpu(), ru, atol=1e-5)
    w = torch.rand(7, generator=gen)
    lc, dyc = G.weighted_sq_error(g, u, w, want_dy=True, scale=0.5)
    lg, dyg = G.weighted_sq_error(g.to(dev), u.to(dev), w.to(dev), want_dy=True, scale=0.5)
    assert abs(lc - lg) < 1e-3 * abs(lc) and torch.allclose(dyg.cpu(), dyc, atol=1e-5)
    assert abs(G.weighted_sq_norm(u.to(dev), w.to(dev)) - G.weighted_sq_norm(u, w)) < 1e-3
    for mode in range(3):
        base = torch.rand(50, generator=gen) + 0.5
        grad = torch.randn(50, generator=gen)
        st_c = [torch.zeros(50), base.clone(), torch.zeros(50), torch.zeros(50)]
        st_g = [t.clone().to(dev) for t in st_c]
        for step in (1, 2, 3):
            for (a, d, m, v), dv_ in ((st_c, "cpu"), (st_g, dev)):
                b, gr = base.to(dv_), grad.to(dv_)
                if mode == 0:
                    G.adam_step(a, gr, m, v, step)
                elif mode == 1:
                    G.adam_log_scales(b, a, d, gr, m, v, step, 0.7)
                else:
                    G.adam_deltas(b, a, d, gr, m, v, step, 0.7)
        for c, gq in zip(st_c, st_g):
            assert torch.allclose(gq.cpu(), c, atol=1e-5)
    src = torch.randn(9, 16, generator=gen)
    idx = torch.tensor([4, 1, 7], dtype=torch.int32)
    ww = torch.rand(3, generator=gen)
    assert torch.allclose(G.gather_rows(src.to(dev), idx.to(dev), ww.to(dev)).cpu(), G.gather_rows(src, idx, ww))
    assert torch.allclose(G.gather_rows(src.half().to(dev), idx.to(dev)).cpu(), src.half()[idx.long()].float())
    d1, d2 = torch.zeros(9, 16), torch.zeros(9, 16, device=dev)
    G.scatter_add_rows_(d1, src[:3].contiguous(), idx, ww)
    G.scatter_add_rows_(d2, src[:3].contiguous().to(dev), idx.to(dev), ww.to(dev))
    assert torch.allclose(d2.cpu(), d1)
    x = torch.randn(5, 8, generator=gen)
    s = torch.rand(5, generator=gen)
    assert torch.allclose(G.scale_rows_(x.clone().to(dev), s.to(dev)).cpu(), x * s[:, None])
    assert torch.allclose(G.exp_scale(x.to(dev), (x * 0.1).to(dev)).cpu(), x * torch.exp(x * 0.1), atol=1e-5)


def test_hessian_accumulator_cpu():
    from volta_engine_b200.ops.hessian import HessianAccumulator
    g = torch.Generator().manual_seed(5)
    a, b = torch.randn(10, 16, generator=g), torch.randn(7, 16, generator=g)
    h = HessianAccumulator(16, "cpu").add(a).add(b)
    x = torch.cat([a, b])
    assert torch.allclose(h.H, x.t() @ x, atol=1e-4) and h.rows == 17
    assert torch.allclose(h.mean(), x.t() @ x / 17, atol=1e-5)


@pytest.mark.gpu
def test_hessian_accumulator_gpu():
    from volta_engine_b200.ops.hessian import HessianAccumulator
    dev = torch.device("cuda:0")
    g = torch.Generator().manual_seed(6)
    x = torch.randn(200, 256, generator=g).to(torch.bfloat16)
    h = HessianAccumulator(256, dev).add(x[:70].to(dev)).add(x[70:].to(dev))
    ref = x.float().t() @ x.float()
    assert torch.allclose(h.H.cpu(), ref, atol=0.05, rtol=1e-2)


@pytest.mark.gpu
def test_model_hessian_capture_gpu_matches_cpu_capture(tmp_path):
    """The capture taps of the dense model on the device (tcgen05 x^T x) against the same model's capture on the CPU."""
    from volta_engine_b200.models.dense import DenseConfig
    from volta_engine_b200.models.factory import load_model, save_dense_checkpoint
    from volta_engine_b200.runtime.engine import Engine
    from volta_engine_b200.runtime.kv_cache import PagedKVCache
    cfg = DenseConfig.tiny(n_layers=2)
    save_dense_checkpoint(tmp_path / "m", cfg, seed=4, fmt="bf16", std=0.05)
    sums = {}
    for dev in ("cpu", "cuda"):
        m, _ = load_model(tmp_path / "m", dev)
        hs = m.enable_hessians()
        kv = PagedKVCache(cfg.n_layers, cfg.n_kv, cfg.head_dim, 8, 1, 256, dev)
        Engine(m, kv, use_graphs=False, prefill_chunk=128).generate(list(range(3, 99)), 2)
        sums[dev] = {k: (a.H.float().cpu(), a.rows) for k, a in hs.sites.items()}
    assert set(sums["cpu"]) == set(sums["cuda"])
    for k, (hc, rows) in sums["cpu"].items():
        hg, rg = sums["cuda"][k]
        assert rows == rg == 96, k
        cos = float((hc * hg).sum() / (hc.norm() * hg.norm()))
        assert cos > 0.995, (k, cos)
