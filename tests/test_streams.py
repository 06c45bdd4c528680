"""Multi-stream residual modules (hyper-connections, gated residual, n-gram layer, row epilogues): properties of the
PyTorch statement on CPU, and the CUDA kernels against it on a GPU."""
import pytest
import torch

from volta_engine_b200.ops import streams as S


def _g(seed):
    return torch.Generator().manual_seed(seed)


def _hc_inputs(rows, D, seed=0):
    g = _g(seed)
    streams = torch.randn(rows, 4, D, generator=g)
    fn = torch.randn(24, 4 * D, generator=g) * 0.05
    base = torch.randn(24, generator=g) * 0.5
    scale = torch.tensor([0.7, 1.1, 0.9])
    return streams, fn, base, scale


def _gr_weights(H, hc, rank, seed=1, inject=True):
    g = _g(seed)
    bf = torch.bfloat16
    return S.GatedResidualWeights(
        norm=(torch.randn(hc, H, generator=g) * 0.1).to(bf),
        down=(torch.randn(rank, hc * H, generator=g) * 0.05).to(bf),
        up=(torch.randn(hc * H, rank, generator=g) * 0.2).to(bf),
        inject=(torch.randn(hc, hc * H, generator=g) * 0.05).to(bf) if inject else None)


def _to(dev, obj):
    if isinstance(obj, torch.Tensor):
        return obj.to(dev)
    if isinstance(obj, S.GatedResidualWeights):
        return S.GatedResidualWeights(*[None if t is None else t.to(dev) for t in (obj.norm, obj.down, obj.up, obj.inject)])
    return obj


# ------------------------------------------------------------------------------------------------ CPU properties
def test_hc_collapse_gates_and_sinkhorn_are_well_formed():
    streams, fn, base, scale = _hc_inputs(3, 64)
    m = S.hc_collapse(streams, fn, base, scale)
    assert m.comb.shape == (3, 4, 4) and torch.all(m.comb > 0)
    assert torch.allclose(m.comb.sum(1), torch.ones(3, 4), atol=1e-3)            # columns normalised last
    assert torch.allclose(m.comb.sum(2), torch.ones(3, 4), atol=2e-2)            # rows nearly, after 20 rounds
    assert torch.all((m.post > 0) & (m.post < 2)) and torch.all((m.pre > 0) & (m.pre < 1.001))
    want = torch.einsum("rh,rhd->rd", m.pre, streams)
    assert torch.allclose(m.collapsed.float(), want, atol=0.02, rtol=0.01)
    lag = S.hc_collapse(streams, fn, base, scale, pre_in=torch.full((3, 4), 0.25), post_scale=0.5)
    assert torch.allclose(lag.collapsed.float(), streams.mean(1), atol=0.02, rtol=0.01)
    assert torch.allclose(lag.post, m.post * 0.5) and torch.equal(lag.pre, m.pre)


def test_hc_update_with_identity_mix_is_a_plain_residual_add():
    g = _g(2)
    streams = torch.randn(2, 4, 32, generator=g)
    y = torch.randn(2, 32, generator=g).to(torch.bfloat16)
    before = streams.clone()
    S.hc_update(y, streams, torch.ones(2, 4), torch.eye(4).repeat(2, 1, 1))
    assert torch.allclose(streams, before + y.float()[:, None, :])
    assert torch.equal(S.head_mean(S.init_streams(y, 4)), y)


def test_gated_residual_deferred_apply_equals_apply_then_mix():
    H, hc, rank = 64, 4, 32
    W = _gr_weights(H, hc, rank)
    g = _g(3)
    a = torch.randn(3, hc, H, generator=g)
    b = a.clone()
    post = torch.rand(3, hc, generator=g)
    y = torch.randn(3, H, generator=g).to(torch.bfloat16)
    S.gated_stream_update(y, a, post)                                  # apply now ...
    m1, p1 = S.gr_mix(a, W, 1e-6)
    m2, p2 = S.gr_mix(b, W, 1e-6, prev_post=post, prev_y=y)            # ... or folded into the next mixer's norm
    assert torch.equal(m1, m2) and torch.equal(p1, p2) and torch.equal(a, b)
    assert p1.shape == (3, hc) and torch.all((p1 > 0) & (p1 < 2))
    # the per-stream norm returned by the update is the next mixer's input
    n = S.gated_stream_update(y, a, post, norm_w=W.norm)
    assert torch.allclose(n, S.gr_norm(a, W.norm, 1e-6))


def test_ple_conv_over_one_chunk_equals_token_by_token_through_the_ring():
    hc, H, T, dil = 2, 16, 12, 3
    C = hc * H
    g = _g(4)
    normed = (torch.randn(T, C, generator=g)).to(torch.bfloat16)
    gated = torch.randn(T, hc, H, generator=g)
    conv_w = (torch.randn(C, 4, generator=g) * 0.5).to(torch.bfloat16)
    slot = torch.zeros(T, dtype=torch.int32)
    pos = torch.arange(T, dtype=torch.int32)
    a = torch.zeros(T, hc, H)
    ring_a = torch.zeros(1, S.PLE_RING, C, dtype=torch.bfloat16)
    S.ple_conv_apply(normed, conv_w, ring_a, slot, pos, gated, a, dil)
    b = torch.zeros(T, hc, H)
    ring_b = torch.zeros(1, S.PLE_RING, C, dtype=torch.bfloat16)
    for t in range(T):
        S.ple_conv_apply(normed[t:t + 1], conv_w, ring_b, slot[t:t + 1], pos[t:t + 1], gated[t:t + 1], b[t:t + 1], dil)
    assert torch.allclose(a, b, atol=1e-6) and torch.equal(ring_a, ring_b)
    # the first position sees only its own tap
    acc = conv_w[:, 3].float() * normed[0].float()
    assert torch.allclose(a[0].reshape(-1), gated[0].reshape(-1) + acc * torch.sigmoid(acc), atol=1e-6)


def test_sandwich_epilogue_matches_its_three_step_form():
    g = _g(5)
    H = 48
    y = torch.randn(2, H, generator=g).to(torch.bfloat16)
    w1, w2 = (torch.randn(H, generator=g) * 0.1).to(torch.bfloat16), (torch.randn(H, generator=g) * 0.1).to(torch.bfloat16)
    for dt in (torch.float32, torch.bfloat16):
        r = torch.randn(2, H, generator=g).to(dt)
        keep = r.clone()
        out = S.sandwich_add_norm(y, r, w1, w2, 1e-6, wbias=1.0, scale=0.5)
        yf = y.float()
        t = (yf * torch.rsqrt(yf.pow(2).mean(-1, keepdim=True) + 1e-6) * (w1.float() + 1)).to(torch.bfloat16).float()
        want_r = ((keep.float() + t) * 0.5).to(dt)
        assert torch.equal(r, want_r)
        wf = want_r.float()
        assert torch.allclose(out.float(), wf * torch.rsqrt(wf.pow(2).mean(-1, keepdim=True) + 1e-6) * (w2.float() + 1),
                              atol=0.02, rtol=0.01)


# ------------------------------------------------------------------------------------------------ GPU kernels
DEV = torch.device("cuda:0")


def _close(a, b, atol, rtol=1e-3, name=""):
    a, b = a.float().cpu(), b.float().cpu()
    assert torch.allclose(a, b, atol=atol, rtol=rtol), f"{name}: max diff {float((a - b).abs().max())}"


@pytest.mark.gpu
@pytest.mark.parametrize("rows,D", [(1, 4096), (5, 5120), (3, 512)])
def test_hc_collapse_kernel(rows, D):
    streams, fn, base, scale = _hc_inputs(rows, D, seed=rows)
    want = S.hc_collapse(streams, fn, base, scale)
    got = S.hc_collapse(*[t.to(DEV) for t in (streams, fn, base, scale)])
    _close(got.mix_logits, want.mix_logits, 2e-3, name="mix logits")
    _close(got.inv_rms, want.inv_rms, 1e-5, name="inv rms")
    _close(got.pre, want.pre, 1e-4, name="pre")
    _close(got.post, want.post, 1e-4, name="post")
    _close(got.comb, want.comb, 1e-4, name="comb")
    _close(got.collapsed, want.collapsed, 0.03, 0.01, name="collapsed")
    nw = (torch.randn(D, generator=_g(9)) * 0.1).to(torch.bfloat16)
    pre_in = torch.rand(rows, 4, generator=_g(10))
    want = S.hc_collapse(streams, fn, base, scale, norm_w=nw, norm_bias=1.0, pre_in=pre_in, post_scale=0.5)
    got = S.hc_collapse(*[t.to(DEV) for t in (streams, fn, base, scale)], norm_w=nw.to(DEV), norm_bias=1.0,
                        pre_in=pre_in.to(DEV), post_scale=0.5)
    _close(got.collapsed, want.collapsed, 0.03, 0.01, name="lagged collapse + norm")
    _close(got.post, want.post, 1e-4, name="scaled post")


@pytest.mark.gpu
def test_stream_epilogue_kernels():
    g = _g(11)
    rows, H = 5, 2560
    y = torch.randn(rows, H, generator=g).to(torch.bfloat16)
    # hyper-connection update
    xs = torch.randn(rows, 4, H, generator=g)
    post, comb = torch.rand(rows, 4, generator=g) * 2, torch.rand(rows, 4, 4, generator=g)
    want = S.hc_update(y, xs.clone(), post, comb)
    got = S.hc_update(y.to(DEV), xs.to(DEV), post.to(DEV), comb.to(DEV))
    _close(got, want, 1e-4, name="hc update")
    # gated streams with the shared-expert addend and the next mixer's norm
    hc = 4
    nw = (torch.randn(hc, H, generator=g) * 0.1).to(torch.bfloat16)
    add, gate = torch.randn(rows, H, generator=g).to(torch.bfloat16), torch.rand(rows, generator=g)
    a = torch.randn(rows, hc, H, generator=g)
    b = a.to(DEV)
    wn = S.gated_stream_update(y, a, post, nw, 1e-6, add, gate)
    gn = S.gated_stream_update(y.to(DEV), b, post.to(DEV), nw.to(DEV), 1e-6, add.to(DEV), gate.to(DEV))
    _close(b, a, 0.02, name="gated streams")
    _close(gn, wn, 0.02, 0.01, name="gated normed")
    g16 = S.gated_stream_update(y.to(DEV), a.to(DEV), torch.zeros(rows, hc, device=DEV), nw.to(DEV), 1e-6, out_dtype=torch.bfloat16)
    _close(g16, S.stream_norm(a, nw, 1e-6).reshape(rows, hc, H), 0.03, 0.01, name="bf16 stream norm")
    _close(S.stream_norm(a.to(DEV), nw.to(DEV), 1e-6), S.stream_norm(a, nw, 1e-6), 0.03, 0.01, name="stream_norm")
    # sandwich norm on both residual types
    w1, w2 = (torch.randn(H, generator=g) * 0.1).to(torch.bfloat16), (torch.randn(H, generator=g) * 0.1).to(torch.bfloat16)
    for dt in (torch.float32, torch.bfloat16):
        r = torch.randn(rows, H, generator=g).to(dt)
        rd = r.to(DEV)
        want = S.sandwich_add_norm(y, r, w1, w2, 1e-6, 1.0, 0.7)
        got = S.sandwich_add_norm(y.to(DEV), rd, w1.to(DEV), w2.to(DEV), 1e-6, 1.0, 0.7)
        _close(rd, r, 0.02, 0.01, name=f"sandwich residual {dt}")
        _close(got, want, 0.03, 0.01, name=f"sandwich out {dt}")
    _close(S.head_mean(S.init_streams(y.to(DEV), 4)), y, 0, name="init + mean")
    e = torch.randn(rows, H, generator=g).to(torch.bfloat16)
    h = torch.randn(rows * hc, H, generator=g).to(torch.bfloat16)
    _close(S.add_broadcast(h.to(DEV), e.to(DEV), hc), S.add_broadcast(h, e, hc), 1e-6, name="add_broadcast")


@pytest.mark.gpu
@pytest.mark.parametrize("rows", [1, 7, 40, 200])
def test_gated_residual_mix_kernels(rows):
    H, hc, rank = 2560, 4, 320
    W = _gr_weights(H, hc, rank, inject=rows != 7)
    g = _g(20 + rows)
    xs = torch.randn(rows, hc, H, generator=g)
    post = torch.rand(rows, hc, generator=g)
    y = torch.randn(rows, H, generator=g).to(torch.bfloat16)
    a, b = xs.clone(), xs.to(DEV)
    wm, wp = S.gr_mix(a, W, 1e-6, post, y)
    gm, gp = S.gr_mix(b, _to(DEV, W), 1e-6, post.to(DEV), y.to(DEV))
    _close(b, a, 1e-5, name="deferred apply")
    _close(gm, wm, 0.02, 0.02, name="mixed")
    if wp is not None:
        _close(gp, wp, 2e-3, name="post")
    x16 = torch.randn(rows, H, generator=g).to(torch.bfloat16)
    wv = (torch.randn(H, generator=g) * 0.05).to(torch.bfloat16)
    _close(S.shared_gate(x16.to(DEV), wv.to(DEV)), S.shared_gate(x16, wv), 2e-3, name="shared gate")


@pytest.mark.gpu
def test_ple_kernels():
    hc, H, T, dil = 4, 640, 10, 3
    C = hc * H
    g = _g(30)
    bf = torch.bfloat16
    key = torch.randn(T, C, generator=g).to(bf)
    value = torch.randn(T, H, generator=g).to(bf)
    xs = torch.randn(T, hc, H, generator=g)
    nk, nq, nc = [(torch.randn(hc, H, generator=g) * 0.1).to(bf) for _ in range(3)]
    wg, wn = S.ple_gate_and_norm(key, value, xs, nk, nq, nc, 1e-6, 0.05)
    gg, gn = S.ple_gate_and_norm(*[t.to(DEV) for t in (key, value, xs, nk, nq, nc)], 1e-6, 0.05)
    _close(gg, wg, 5e-3, 5e-3, name="ple gated")
    _close(gn, wn, 0.03, 0.01, name="ple normed")
    conv_w = (torch.randn(C, 4, generator=g) * 0.5).to(bf)
    # two slots interleaved in one chunk, the second one continuing from ring contents
    slot = torch.tensor([0, 1, 0, 1, 0, 1, 0, 1, 0, -1], dtype=torch.int32)
    pos = torch.tensor([0, 20, 1, 21, 2, 22, 3, 23, 4, 0], dtype=torch.int32)
    ring = torch.randn(2, S.PLE_RING, C, generator=g).to(bf)
    a, ra = xs.clone(), ring.clone()
    S.ple_conv_apply(wn, conv_w, ra, slot, pos, wg, a, dil)
    b, rb = xs.to(DEV), ring.to(DEV)
    S.ple_conv_apply(wn.to(DEV), conv_w.to(DEV), rb, slot.to(DEV), pos.to(DEV), wg.to(DEV), b, dil)
    _close(b, a, 2e-3, name="ple conv")
    assert torch.equal(rb.cpu(), ra)
