"""EXL3 trellis format: CPU oracle properties, Viterbi encoder quality, and the CUDA kernels against the oracle."""
import pytest
import torch

from volta_engine_b200.quant import exl3 as ex


def test_had128_is_an_orthonormal_involution():
    g = torch.Generator().manual_seed(0)
    x = torch.randn(5, 384, generator=g)
    y = ex.had128(x)
    assert torch.allclose(ex.had128(y), x, atol=1e-5)
    assert torch.allclose(y.norm(dim=-1), x.norm(dim=-1), rtol=1e-5)
    # natural (Sylvester) order: row 1 of H alternates signs
    e = torch.zeros(128); e[1] = 1
    h = ex.had128(e) * 128 ** 0.5
    assert torch.allclose(h, torch.tensor([1.0, -1.0]).repeat(64), atol=1e-5)


def test_window_extraction_matches_a_bit_by_bit_reader():
    g = torch.Generator().manual_seed(1)
    for bits in (2, 3, 4, 5, 8):
        codes = ex.random_codes(16, 16, bits, g)[0, 0]
        words = [(int(codes[2 * i]) & 0xFFFF) | ((int(codes[2 * i + 1]) & 0xFFFF) << 16) for i in range(8 * bits)]
        stream = [(w >> (31 - b)) & 1 for w in words for b in range(32)]
        total = 256 * bits
        win = ex.tile_windows(codes[None], bits)[0]
        for p in (0, 1, 7, 100, 255):
            s = (p * bits + bits - 16) % total
            v = 0
            for j in range(16):
                v = (v << 1) | stream[(s + j) % total]
            assert int(win[p]) == v


def test_half_integer_rate_windows_follow_the_funnel_shift_reader(tmp_path):
    """Rates K + 0.5 (16 K + 8 code words per tile): the windows advance by K and K + 1 bits alternately. The vectorised
    reader is checked against a literal 64-bit funnel-shift reader of the same stream (two 32-bit words merged high word
    first, shifted so that the window's end bit lands at bit 0), then through a linear loaded from a checkpoint."""
    g = torch.Generator().manual_seed(4)
    for K in (1, 2, 3, 4):
        codes = ex.random_codes(16, 16, K + 0.5, g)[0, 0]
        assert codes.numel() == 16 * K + 8 and ex.is_half_rate(codes)
        nwords = 4 * (2 * K + 1)
        words = [(int(codes[2 * i]) & 0xFFFF) | ((int(codes[2 * i + 1]) & 0xFFFF) << 16) for i in range(nwords)]
        win = ex.tile_windows(codes[None], K)[0]
        bits2 = 2 * K + 1
        for p in (0, 1, 2, 3, 6, 7, 100, 101, 254, 255):
            end = (p // 2 + 1) * bits2 - (0 if p % 2 else K + 1) + 128 * bits2          # one tile ahead: the stream wraps
            hi, lo = (end - 1) // 32, (end - 16) // 32
            merged = (words[lo % nwords] << 32) | words[hi % nwords] if hi != lo else (words[lo % nwords] << 32) | words[lo % nwords]
            shift = (hi + 1) * 32 - end
            if hi == lo:
                v = (words[lo % nwords] >> shift) & 0xFFFF
            else:
                v = (merged >> shift) & 0xFFFF
            assert int(win[p]) == v, (K, p)
    # a 2.5 bit linear: the map is that of its decoded tiles, and a checkpoint with such a tensor loads
    from volta_engine_b200.loader.safetensors import SafeTensorsRepo, write_safetensors
    from volta_engine_b200.ops.linear_exl3 import LinearEXL3
    codes = ex.random_codes(128, 256, 2.5, g)
    suh = (torch.randint(0, 2, (128,), generator=g).float() * 2 - 1).half()
    svh = ((torch.randint(0, 2, (256,), generator=g).float() * 2 - 1) * 0.05).half()
    write_safetensors(tmp_path / "m.safetensors", {"l.trellis": codes, "l.suh": suh, "l.svh": svh, "l.mul1": torch.zeros(1, dtype=torch.int32)},
                      unsigned16=("l.trellis",))
    lin = SafeTensorsRepo(tmp_path).load_linear("l")
    assert isinstance(lin, LinearEXL3) and lin.bits == 2 and lin.half and lin.cb == ex.CB_MUL1
    W = ex.reconstruct(codes, 2, ex.CB_MUL1)
    assert W.shape == (128, 256) and 0.8 < float(W.std()) < 1.2           # random windows decode to a near-unit Gaussian
    x = torch.randn(3, 128, generator=g)
    want = ex.had128(ex.had128(x * suh.float()) @ W) * svh.float()
    assert torch.allclose(lin.forward(x, out_f32=True), want, atol=1e-5)


def test_extended_trellis_start_states_and_tile_gains(tmp_path):
    """Open-trellis tiles: the windows are those of the plain (not cyclic) bit string "16 bits of start state + the tile's
    stream"; a gain code c scales a tile by (896 + c) / 1024; a checkpoint with the two side tensors loads and slices."""
    from volta_engine_b200.loader.safetensors import SafeTensorsRepo, write_safetensors
    g = torch.Generator().manual_seed(6)
    for bits in (2, 3, 4, 5, 8):
        codes = ex.random_codes(16, 16, bits, g)[0, 0]
        start = int(torch.randint(0, 65536, (1,), generator=g))
        words = [(int(codes[2 * i]) & 0xFFFF) | ((int(codes[2 * i + 1]) & 0xFFFF) << 16) for i in range(8 * bits)]
        string = [(start >> (15 - b)) & 1 for b in range(16)] + [(w >> (31 - b)) & 1 for w in words for b in range(32)]
        win = ex.tile_windows(codes[None], bits, torch.tensor([start]))[0]
        ring = ex.tile_windows(codes[None], bits)[0]
        for p in range(256):
            v = 0
            for bit in string[(p + 1) * bits:(p + 1) * bits + 16]:
                v = (v << 1) | bit
            assert int(win[p]) == v, (bits, p)
            if (p + 1) * bits >= 16:
                assert int(ring[p]) == v                     # past the first 16 bits the two readers agree
    K, N, bits = 128, 256, 3
    codes, suh, svh = ex.synth_linear(K, N, bits, 0.05, g)
    tstart = torch.randint(0, 65536, (K // 16, N // 16), generator=g, dtype=torch.int32).to(torch.int16)
    tgain = torch.randint(0, 256, (K // 16, N // 16), generator=g, dtype=torch.int32).to(torch.uint8)
    plain, ext = ex.reconstruct(codes, bits), ex.reconstruct(codes, bits, tstart=tstart, tgain=tgain)
    gains = ex.tile_gain(tgain)
    assert float(gains.min()) >= 0.875 and float(gains.max()) <= 1151 / 1024
    t_plain = plain.reshape(K // 16, 16, N // 16, 16).permute(0, 2, 1, 3)
    t_ext = ex.reconstruct(codes, bits, tstart=tstart).reshape(K // 16, 16, N // 16, 16).permute(0, 2, 1, 3)
    changed = (t_plain != t_ext).reshape(K // 16, N // 16, -1).sum(-1)
    assert int(changed.max()) <= 5 and int(changed.sum()) > 0          # only a tile's first windows (16 / bits of them) see the start state
    want = (t_ext * gains[..., None, None]).to(torch.float16).float().permute(0, 2, 1, 3).reshape(K, N)
    assert torch.equal(ext, want)
    write_safetensors(tmp_path / "m.safetensors", {"l.trellis": codes, "l.suh": suh, "l.svh": svh, "l.tstart": tstart.reshape(-1),
                                                  "l.tgain": tgain.reshape(-1), "l.mul1": torch.zeros(1, dtype=torch.int32)},
                      unsigned16=("l.trellis", "l.tstart"))
    repo = SafeTensorsRepo(tmp_path)
    lin = repo.load_linear("l")
    x = torch.randn(2, K, generator=g)
    full = lin.forward(x, out_f32=True)
    assert torch.allclose(full, ex.had128(ex.had128(x * suh.float()) @ ext) * svh.float(), atol=1e-5)
    assert not torch.allclose(full, ex.had128(ex.had128(x * suh.float()) @ plain) * svh.float(), atol=1e-4)
    cols = torch.cat([repo.load_linear("l", "col", r, 2).forward(x, out_f32=True) for r in range(2)], -1)
    assert torch.allclose(cols, full, atol=1e-4)
    assert torch.allclose(lin.dequant().t(), ex.effective_weight(codes, bits, suh, svh, tstart=tstart, tgain=tgain), atol=1e-6)


def test_codebooks_are_near_unit_gaussians():
    w = torch.arange(65536)
    for cb, lo, hi in ((ex.CB_MUL1, 0.95, 1.05), (ex.CB_3INST, 1.1, 1.4), (ex.CB_MCG, 1.1, 1.4)):
        v = ex.decode_windows(w, cb)
        assert abs(float(v.mean())) < 0.05 and lo < float(v.std()) < hi


def test_viterbi_encoder_reaches_trellis_quality_and_round_trips():
    g = torch.Generator().manual_seed(2)
    t = torch.randn(256, generator=g)
    for bits, bound in ((2, 0.09), (4, 0.008)):
        code = ex.viterbi_encode_tile(t, bits)
        w = ex.decode_windows(ex.tile_windows(code[None], bits))[0]
        assert float(((w - t) ** 2).mean()) < bound


def test_quantize_small_matrix_reproduces_the_linear_map():
    g = torch.Generator().manual_seed(3)
    W = torch.randn(128, 128, generator=g) * 0.05
    codes, suh, svh = ex.quantize(W, 2)
    x = torch.randn(4, 128, generator=g)
    y = ex.linear_reference(x, codes, 2, suh, svh)
    ref = x @ W
    cos = torch.nn.functional.cosine_similarity(y.flatten(), ref.flatten(), dim=0)
    assert cos > 0.96


@pytest.mark.gpu
@pytest.mark.parametrize("bits", [1, 2, 3, 4, 5, 6, 8])
def test_gpu_reconstruct_and_gemv_match_oracle(bits):
    from volta_engine_b200.ops import linear_exl3 as L
    dev = torch.device("cuda:0")
    g = torch.Generator().manual_seed(bits)
    Kf, N = 640, 384          # 40 k-tiles: the warps' last iteration is a partial one
    for cb in (0, 1, 2):
        codes = ex.random_codes(Kf, N, bits, g)
        Wref = ex.reconstruct(codes, bits, cb)                   # [K, N]
        w = L.exl3_reconstruct(codes.to(dev), Kf, N, bits, cb).float().cpu()
        assert torch.equal(w, Wref.t().to(torch.bfloat16).float())
        for M in (1, 5, 16):
            x = (torch.randn(M, Kf, generator=g)).to(torch.float16)
            y = L.exl3_gemv(codes.to(dev), x.to(dev), M, Kf, N, bits, cb).cpu()
            ref = x.float() @ Wref
            assert torch.allclose(y, ref, atol=2e-2, rtol=2e-3), (bits, cb, M, float((y - ref).abs().max()))


@pytest.mark.gpu
def test_gpu_had128_and_linear_paths():
    from volta_engine_b200.ops import linear_exl3 as L
    dev = torch.device("cuda:0")
    g = torch.Generator().manual_seed(11)
    x = torch.randn(7, 640, generator=g).to(torch.bfloat16)
    s = (torch.rand(640, generator=g) + 0.5).to(torch.float16)
    y = L.had128(x.to(dev), s.to(dev), out_dtype=torch.float16).float().cpu()
    assert torch.allclose(y, ex.had128(x.float() * s.float()), atol=2e-2, rtol=1e-2)
    y2 = L.had128(x.float().to(dev), s.to(dev), post=True, out_dtype=torch.bfloat16).float().cpu()
    assert torch.allclose(y2, ex.had128(x.float()) * s.float(), atol=3e-2, rtol=2e-2)
    lin = L.LinearEXL3.synth(640, 512, bits=4, std=0.05, gen=g)
    ref1 = lin.forward(x[:3].float(), out_f32=True)
    xl = torch.randn(48, 640, generator=g).to(torch.bfloat16)
    ref2 = lin.forward(xl.float(), out_f32=True)
    lin.to(dev)
    o1 = lin.forward(x[:3].to(dev)).float().cpu()
    o2 = lin.forward(xl.to(dev)).float().cpu()
    cs = torch.nn.functional.cosine_similarity
    assert cs(o1.flatten(), ref1.flatten(), dim=0) > 0.9995
    assert cs(o2.flatten(), ref2.flatten(), dim=0) > 0.999
    # decode rows are batch-invariant: row 0 alone equals row 0 inside a 3-row batch
    a = lin.forward(x[:1].to(dev)); b = lin.forward(x[:3].to(dev))[:1]
    assert torch.equal(a, b)


def test_moe_model_with_exl3_experts_runs_on_cpu_and_its_bank_matches_dense_weights():
    from volta_engine_b200.models.moe import MoEConfig, MoEModel
    from volta_engine_b200.ops.moe_exl3 import EXL3ExpertBank
    from volta_engine_b200.runtime.engine import Engine
    from volta_engine_b200.runtime.kv_cache import PagedKVCache
    bank = EXL3ExpertBank.random(3, 128, 256, 3, e0=2, seed=1, std=0.05)
    x = (torch.randn(2, 256, generator=torch.Generator().manual_seed(0)) * 0.5).to(torch.bfloat16)
    ids = torch.tensor([[2, 9], [4, 3]], dtype=torch.int32)                  # expert 9 lives on another rank
    d = bank.routes(x, ids, 0, 0.0).float()
    assert float(d[1].abs().max()) == 0.0 and float(d[0].abs().max()) > 0
    # the statement through dense effective weights
    for r, (t, e) in enumerate(((0, 0), (0, None), (1, 2), (1, 1))):
        if e is None:
            continue
        gu, dn = bank.dequant("gu", e), bank.dequant("dn", e)
        h = x[t].float() @ gu.t()
        a = torch.nn.functional.silu(h[:128]) * h[128:]
        want = a @ dn.t()
        assert torch.allclose(d[r], want, atol=3e-2 * float(want.abs().max()) + 1e-5), (r, float((d[r] - want).abs().max()))
    cfg = MoEConfig.tiny_moe(expert_quant="exl3_4", hidden=256, expert_ffn=128)
    m = MoEModel(cfg, "cpu").init_random(seed=3)
    assert isinstance(m.layers[0].bank, EXL3ExpertBank) and m.layers[0].bank.bits == 4
    kv = PagedKVCache(2, m.nkv, 64, 16, 1, 512, "cpu")
    out, _ = Engine(m, kv, use_graphs=False, prefill_chunk=16).generate(list(range(1, 25)), 4)
    assert len(out) == 4


@pytest.mark.gpu
@pytest.mark.parametrize("bits", [2, 4, 5])
def test_gpu_routed_experts_in_exl3(bits):
    from volta_engine_b200.ops.moe_exl3 import EXL3ExpertBank
    from volta_engine_b200.ops import kernels as K
    dev = "cuda"
    E, I, H, k = 8, 256, 512, 2
    bank_c = EXL3ExpertBank.random(E, I, H, bits, e0=4, seed=9, std=0.05)
    bank_g = bank_c.to(dev)
    g = torch.Generator().manual_seed(2)
    for rows in (1, 7, 16, 150):
        x = (torch.randn(rows, H, generator=g) * 0.5).to(torch.bfloat16)
        ids = torch.randint(0, 16, (rows, k), generator=g, dtype=torch.int32)
        if rows == 150:
            ids[:, 0] = 5                                  # one crowded expert: several tiles of the grouped GEMM
        want = bank_c.routes(x[:24], ids[:24], 0, 0.0).float()       # (the CPU statement is slow: the first 24 rows)
        got = bank_g.routes(x.to(dev), ids.to(dev), 0, 0.0).float().cpu()
        scale = float(want.abs().max()) + 1e-6
        n = want.shape[0]
        assert float((got[:n] - want).abs().max()) < 4e-2 * scale, (bits, rows, float((got[:n] - want).abs().max()), scale)
        away = ((ids < 4) | (ids >= 12)).reshape(-1)
        assert float(got[away].abs().max()) == 0.0 if away.any() else True
    assert K.check_status(dev) == 0


@pytest.mark.gpu
@pytest.mark.parametrize("bits,cb", [(2, ex.CB_MUL1), (3, ex.CB_MUL1), (4, ex.CB_MUL1), (4, ex.CB_3INST), (6, ex.CB_MCG)])
def test_gpu_viterbi_encoder_matches_the_host_statement(bits, cb):
    """The device encoder runs the same search as quant.exl3.viterbi_encode_tile: the same code words (or, where two
    paths tie to the last bit, the same squared error), and its streams are tail-biting (they decode to 256 windows)."""
    from volta_engine_b200.ops.linear_exl3 import exl3_viterbi
    g = torch.Generator().manual_seed(bits * 10 + cb)
    targets = torch.randn(3, 256, generator=g)
    got = exl3_viterbi(targets.cuda(), bits, cb).cpu()
    for i in range(3 if bits >= 4 else 1):                       # (the host search is slow at low rates: 2^(16 + bits) per step)
        want = ex.viterbi_encode_tile(targets[i], bits, cb)
        vg = ex.decode_windows(ex.tile_windows(got[i], bits), cb)
        vw = ex.decode_windows(ex.tile_windows(want, bits), cb)
        eg, ew = float(((vg - targets[i]) ** 2).sum()), float(((vw - targets[i]) ** 2).sum())
        assert torch.equal(got[i], want) or abs(eg - ew) < 1e-4 * max(1.0, ew), (bits, cb, i, eg, ew)
        if bits <= 4:
            assert eg < 256 * (4.0 ** -bits) * 6, (bits, eg)             # the rate-distortion ballpark of a trellis code


@pytest.mark.gpu
def test_gpu_quantize_whole_matrix_with_the_device_encoder():
    W = torch.randn(256, 384, generator=torch.Generator().manual_seed(1)) * 0.03
    codes, suh, svh = ex.quantize(W.cuda(), 4)
    assert codes.shape == (16, 24, 64) and codes.is_cuda
    eff = ex.effective_weight(codes.cpu(), 4, suh.cpu(), svh.cpu())
    rel = float((eff - W).norm() / W.norm())
    assert rel < 0.12, rel                                         # 4 bits per weight: about 7-9 % relative error
