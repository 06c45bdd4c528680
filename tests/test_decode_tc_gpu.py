"""tcgen05 block-scaled FP4 decode linear: in-kernel residual expansion of bf16 activations, split-K tickets,
residual / fp32 outputs, agreement with the stand-alone expansion kernel and with the fp32 reference."""
import pytest
import torch

pytestmark = pytest.mark.gpu


def _dequant_expansion(xp, xs, M, K, terms):
    from volta_engine_b200.quant import nvfp4 as qn
    codes = qn.e2m1_decode(qn.unpack_codes(xp[: M * terms].cpu())).reshape(M * terms, K // 16, 16)
    atoms = xs.cpu().reshape(-1, 512)[: K // 64]
    v = torch.arange(M * terms)
    idx = (v % 32) * 16 + (v // 32) * 4
    sc = torch.stack([atoms[:, idx + j] for j in range(4)], dim=-1)          # [K/64, rows, 4]
    sc = qn.e4m3_decode(sc.permute(1, 0, 2).reshape(M * terms, K // 16))
    rows = (codes * sc[..., None]).reshape(M, terms, K)
    coef = torch.tensor([8.0 ** -t for t in range(terms)])
    return (rows * coef[None, :, None]).sum(1)


def test_expansion_reaches_bf16_accuracy():
    from volta_engine_b200.ops import kernels as K
    dev = torch.device("cuda:0")
    g = torch.Generator(device="cpu").manual_seed(0)
    x = (torch.randn(5, 1024, generator=g) * torch.rand(5, 1024, generator=g).pow(3) * 4).to(torch.bfloat16)
    for terms, bound in ((1, 0.12), (2, 0.012), (4, 1e-4)):
        xp, xs = K.nvfp4_expand_rows(x.to(dev), terms)
        torch.cuda.synchronize()
        xh = _dequant_expansion(xp, xs, 5, 1024, terms)
        rel = float((xh - x.float()).norm() / x.float().norm())
        assert rel < bound, (terms, rel)


@pytest.mark.parametrize("Kd", [640, 2176])
def test_decode_linear_with_a_half_k_tile(Kd):
    """K that is a multiple of 128 but not of 256 (the row-parallel shards of the 27B model on 8 GPUs: 640 and 2176): the
    last k-tile is half weights, half zero fill, and the scale atoms are padded to whole tiles."""
    from volta_engine_b200.ops.linear import LinearNVFP4
    from volta_engine_b200.quant import nvfp4 as qn
    dev = torch.device("cuda:0")
    g = torch.Generator(device="cpu").manual_seed(Kd)
    lin = LinearNVFP4.from_dense((torch.randn(512, Kd, generator=g) * 0.05).to(dev), search=False).prepare()
    assert lin.tc_ready()
    wd = qn.dequantize_nvfp4(lin.packed, lin.scales, lin.gscale).double().cpu()
    for M in (1, 4, 16):
        x = (torch.randn(M, Kd, generator=g) * 2).to(torch.bfloat16)
        ref = x.double() @ wd.t()
        y = lin.forward(x.to(dev)).double().cpu()
        assert float((y - ref).norm() / ref.norm()) < 5e-3, (M, float((y - ref).norm() / ref.norm()))
        y1 = lin.forward(x[:1].to(dev)).double().cpu()
        assert torch.equal(y1[0], y[0])                  # row 0 does not depend on how many rows ride along


@pytest.mark.parametrize("M", [1, 3, 8, 16])
def test_decode_linear_matches_reference(M):
    from volta_engine_b200.ops import kernels as K
    from volta_engine_b200.quant import nvfp4 as qn
    dev = torch.device("cuda:0")
    g = torch.Generator(device="cpu").manual_seed(M)
    N, Kd = 384, 3072          # 12 k-tiles: with one split every pipeline stage is reused three times
    w = torch.randn(N, Kd, generator=g) * 0.05
    p, s, gs = qn.quantize_nvfp4(w, search=False)
    wd = qn.dequantize_nvfp4(p, s, gs).double()
    at = qn.scales_atoms_512(s).to(dev)
    x = (torch.randn(M, Kd, generator=g) * torch.rand(M, Kd, generator=g) * 3).to(torch.bfloat16)
    res = torch.randn(M, N, generator=g).to(torch.bfloat16)
    ref = x.double() @ wd.t()
    xp, xs = K.nvfp4_expand_rows(x.to(dev), 4)
    torch.cuda.synchronize()
    ref_exp = _dequant_expansion(xp, xs, M, Kd, 4).double() @ wd.t()     # what the tensor core is asked to compute
    outs = {}
    for ks in (1, 2, 3, None):
        for pdl in (False, True):
            y = K.decode_w4a4(p.to(dev), at, gs, x.to(dev), out_f32=True, ks=ks, pdl=pdl).double().cpu()
            assert float((y - ref_exp).abs().max()) < 2e-5 * float(ref.abs().max()) + 1e-6, (ks, pdl)
            assert float((y - ref).norm() / ref.norm()) < 2e-4
            outs[(ks, pdl)] = y
    assert torch.equal(outs[(2, False)], outs[(2, True)])       # split order is fixed, launch mode does not matter
    yb = K.decode_w4a4(p.to(dev), at, gs, x.to(dev), residual=res.to(dev), ks=2).float().cpu()
    want = (ref + res.double()).float()
    assert torch.allclose(yb, want, atol=2e-2 * float(want.abs().max()), rtol=1e-2)
    # rows are independent of the batch they ride in
    y1 = K.decode_w4a4(p.to(dev), at, gs, x[:1].to(dev), out_f32=True, ks=2).cpu()
    assert torch.equal(y1[0], outs[(2, False)][0].float())
    assert K.check_status(dev) == 0


def test_linear_layer_uses_the_tensor_core_path_for_decode_rows():
    from volta_engine_b200.ops import kernels as K, linear as L
    dev = torch.device("cuda:0")
    g = torch.Generator(device="cpu").manual_seed(9)
    w = torch.randn(256, 512, generator=g) * 0.05
    lin = L.LinearNVFP4.from_dense(w.to(dev), search=False).prepare()
    assert lin._sf_atoms is not None or L.GEMV_KERNEL not in ("auto", "tc")
    x = torch.randn(2, 512, generator=g).to(torch.bfloat16).to(dev)
    ref = x.float().cpu() @ lin.dequant().float().cpu().t()
    before = K.native_launches()
    y = lin.forward(x).float().cpu()
    assert torch.allclose(y, ref, atol=2e-2 * float(ref.abs().max()), rtol=2e-2)
    if L.GEMV_KERNEL in ("auto", "tc"):
        assert K.native_launches() - before == 1       # one launch: expansion happens inside the kernel


@pytest.mark.parametrize("act", [0, 1])
def test_fused_gated_activation_matches_separate_kernels(act):
    from volta_engine_b200.ops import kernels as K, linear as L
    dev = torch.device("cuda:0")
    g = torch.Generator(device="cpu").manual_seed(21)
    I, H = 384, 512
    w = torch.randn(2 * I, H, generator=g) * 0.05
    plain = L.LinearNVFP4.from_dense(w.to(dev), search=False).prepare()
    fused = L.LinearNVFP4.from_dense(w.to(dev), search=False).prepare().interleave_gated()
    assert fused.gated and torch.equal(fused.packed[:64], plain.packed[:64]) and torch.equal(fused.packed[64:128], plain.packed[I:I + 64])
    for rows in (1, 5, 40):                       # decode kernel epilogue, and the GEMM + interleaved activation kernel
        x = torch.randn(rows, H, generator=g).to(torch.bfloat16).to(dev)
        want = K.gated_act(plain.forward(x), I, act, 2.0).float().cpu()
        got = fused.forward_gated(x, act, 2.0).float().cpu()
        assert got.shape == (rows, I)
        assert torch.allclose(got, want, atol=2e-2 * float(want.abs().max()) + 1e-3, rtol=2e-2), rows
    assert K.check_status(dev) == 0


def test_fused_prenorm_matches_norm_kernel_then_linear():
    from volta_engine_b200.ops import kernels as K, linear as L
    dev = torch.device("cuda:0")
    g = torch.Generator(device="cpu").manual_seed(31)
    H, N = 1024, 512
    lin = L.LinearNVFP4.from_dense((torch.randn(N, H, generator=g) * 0.05).to(dev), search=False).prepare()
    gated = L.LinearNVFP4.from_dense((torch.randn(N, H, generator=g) * 0.05).to(dev), search=False).prepare().interleave_gated()
    w = (torch.rand(H, generator=g) + 0.5).to(torch.bfloat16).to(dev)
    for M in (1, 3, 4):
        resid = torch.randn(M, H, generator=g).to(torch.bfloat16).to(dev)
        delta = (torch.randn(M, H, generator=g) * 0.3).to(torch.bfloat16).to(dev)
        # reference: the norm kernel (updates the residual in place), then the plain decode linear
        r_ref = resid.clone()
        x_ref = K.rmsnorm(delta, w, 1e-6, 0.0, residual=r_ref)
        want = lin.forward(x_ref).float().cpu()
        r_out = torch.empty_like(resid)
        got = lin.forward_prenorm(resid, delta, w, 1e-6, 0.0, r_out).float().cpu()
        assert torch.equal(r_out, r_ref)
        assert torch.allclose(got, want, atol=2e-2 * float(want.abs().max()), rtol=2e-2)
        # no delta: plain norm of the residual, nothing written
        x0 = K.rmsnorm(resid, w, 1e-6, 1.0)
        got0 = lin.forward_prenorm(resid, None, w, 1e-6, 1.0, None).float().cpu()
        assert torch.allclose(got0, lin.forward(x0).float().cpu(), atol=2e-2 * float(want.abs().max()), rtol=2e-2)
        # together with the gated activation
        wantg = gated.forward_gated(x_ref, 0, 0.0).float().cpu()
        gotg = gated.forward_prenorm(resid, delta, w, 1e-6, 0.0, torch.empty_like(resid), act=0).float().cpu()
        assert torch.allclose(gotg, wantg, atol=2e-2 * float(wantg.abs().max()) + 1e-3, rtol=3e-2)
    assert K.check_status(dev) == 0


def test_dense_model_step_agrees_with_and_without_fused_norms(monkeypatch):
    from volta_engine_b200.models import dense
    from volta_engine_b200.runtime.engine import Engine
    from volta_engine_b200.runtime.kv_cache import PagedKVCache
    dev = torch.device("cuda:0")
    cfg = dense.DenseConfig(n_layers=3, hidden=512, n_q=4, n_kv=2, head_dim=128, ffn=1024, vocab=2048)
    m = dense.DenseModel(cfg, dev).init_random(seed=5)
    prompt = list(range(100, 180))
    hidden = []
    for fuse in (True, False):
        monkeypatch.setattr(dense, "FUSE_PRENORM", fuse)
        assert m._prenorm_ok(type("B", (), {"n": 1})()) == fuse
        kv = PagedKVCache(cfg.n_layers, m.nkv, cfg.head_dim, 8, 1, 512, dev)
        eng = Engine(m, kv, use_graphs=False, prefill_chunk=64)
        eng.prefill(0, prompt)                          # prefill rows never take the fused path
        eng.step([7], [len(prompt)], [0])               # one decode row on top of identical caches
        hidden.append(m.last_hidden.float().cpu().clone())
    cos = torch.nn.functional.cosine_similarity(hidden[0].flatten(), hidden[1].flatten(), dim=0)
    assert cos > 0.999, float(cos)


def test_fused_add_norm_behind_the_linear_matches_linear_then_norm_kernel():
    """The tile that finishes last adds the product into the residual and normalises the rows: same residual bits as the
    stand-alone norm kernel, normalised rows to rounding; the launch-wide ticket is back at zero after every call."""
    from volta_engine_b200.ops import kernels as K, linear as L
    dev = torch.device("cuda:0")
    g = torch.Generator(device="cpu").manual_seed(41)
    for (N, Kd) in ((1024, 512), (5120, 3072)):
        lin = L.LinearNVFP4.from_dense((torch.randn(N, Kd, generator=g) * 0.05).to(dev), search=False).prepare()
        w = (torch.rand(N, generator=g) + 0.5).to(torch.bfloat16).to(dev)
        for M in (1, 4, 16):
            assert lin.addnorm_ready(M)
            x = torch.randn(M, Kd, generator=g).to(torch.bfloat16).to(dev)
            resid = torch.randn(M, N, generator=g).to(torch.bfloat16).to(dev)
            r_ref = resid.clone()
            want = K.rmsnorm(lin.forward(x), w, 1e-6, 1.0, residual=r_ref)
            for _ in range(2):                                   # twice: the ticket must have been reset
                r_got = resid.clone()
                got = lin.forward_addnorm(x, r_got, w, 1e-6, 1.0)
                assert torch.equal(r_got, r_ref), f"residual differs N={N} M={M}"
                assert torch.allclose(got.float(), want.float(), atol=2e-2, rtol=2e-2)
            assert int(K.dw_scratch(dev)[3][1024].item()) == 0
    assert K.check_status(dev) == 0


@pytest.mark.parametrize("kv_dtype", [torch.bfloat16, torch.float8_e5m2])
@pytest.mark.parametrize("rot", [128, 64])
def test_fused_rope_and_cache_write_match_linear_then_rotation_kernel(kv_dtype, rot):
    from volta_engine_b200.ops import kernels as K, linear as L
    dev = torch.device("cuda:0")
    g = torch.Generator(device="cpu").manual_seed(51)
    nq, nkv, hd, H = 6, 2, 128, 768
    lin = L.LinearNVFP4.from_dense((torch.randn((nq + 2 * nkv) * hd, H, generator=g) * 0.05).to(dev), search=False).prepare()
    table = (torch.randperm(15, generator=g)[:12].to(torch.int32) + 1).reshape(3, 4).to(dev)
    for M, pos, slot in ((1, [130], [1]), (5, [0, 63, 64, 200, 7], [0, 0, 1, 2, -1]), (16, list(range(100, 116)), [2] * 16)):
        assert lin.rope_ready(M, hd)
        x = torch.randn(M, H, generator=g).to(torch.bfloat16).to(dev)
        p = torch.tensor(pos, dtype=torch.int32, device=dev)
        s = torch.tensor(slot, dtype=torch.int32, device=dev)
        k1, v1 = (torch.zeros(16, nkv, 64, hd, dtype=kv_dtype, device=dev) for _ in range(2))
        k2, v2 = (torch.zeros(16, nkv, 64, hd, dtype=kv_dtype, device=dev) for _ in range(2))
        want = lin.forward(x)
        K.rope_store(want, p, s, table, k1, v1, nq, nkv, hd, rot, 1e6, False)
        got = lin.forward_rope(x, p, s, table, k2, v2, nq, nkv, rot, 1e6)
        assert torch.equal(got, want), f"rotated rows differ M={M}"
        assert torch.equal(k2.view(torch.uint8), k1.view(torch.uint8)) and torch.equal(v2.view(torch.uint8), v1.view(torch.uint8))
    assert K.check_status(dev) == 0


def test_dense_model_decode_agrees_with_and_without_the_fused_rope(monkeypatch):
    from volta_engine_b200.models import dense
    from volta_engine_b200.runtime.engine import Engine
    from volta_engine_b200.runtime.kv_cache import PagedKVCache
    dev = torch.device("cuda:0")
    cfg = dense.DenseConfig(n_layers=3, hidden=512, n_q=4, n_kv=2, head_dim=128, ffn=1024, vocab=2048)
    m = dense.DenseModel(cfg, dev).init_random(seed=5)
    prompt = list(range(100, 180))
    outs = []
    for fuse in (True, False):
        monkeypatch.setattr(dense, "FUSE_ROPE", fuse)
        kv = PagedKVCache(cfg.n_layers, m.nkv, cfg.head_dim, 8, 1, 512, dev)
        out, _ = Engine(m, kv, prefill_chunk=64).generate(prompt, 8)
        outs.append(out)
    assert outs[0] == outs[1]                               # same bits: same tokens


@pytest.mark.parametrize("shape", ["tiny", "wide"])
def test_graph_replay_decodes_the_same_tokens_as_eager_launches(shape):
    """CUDA-graph replay runs the step's kernels back to back (programmatic launches really overlap there); the greedy
    tokens must be those of eager launches, run after run."""
    from volta_engine_b200.models import dense
    from volta_engine_b200.ops import kernels as K
    from volta_engine_b200.runtime.engine import Engine
    from volta_engine_b200.runtime.kv_cache import PagedKVCache
    dev = torch.device("cuda:0")
    if shape == "tiny":
        cfg = dense.DenseConfig(n_layers=3, hidden=512, n_q=4, n_kv=2, head_dim=128, ffn=1024, vocab=2048)
    else:
        cfg = dense.DenseConfig(n_layers=4, hidden=2048, n_q=16, n_kv=4, head_dim=128, ffn=8192, vocab=4096)
    m = dense.DenseModel(cfg, dev).init_random(seed=5)
    prompt = list(range(100, 180))
    outs = []
    for graphs in (False, True, True, True):
        kv = PagedKVCache(cfg.n_layers, m.nkv, cfg.head_dim, 8, 1, 512, dev)
        out, _ = Engine(m, kv, prefill_chunk=64, use_graphs=graphs).generate(prompt, 12)
        outs.append(out)
    assert outs[1] == outs[0] and outs[2] == outs[0] and outs[3] == outs[0], outs
    assert K.check_status(dev) == 0
