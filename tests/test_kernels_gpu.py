"""CUDA kernels against the fp32 PyTorch oracle (volta_engine_b200.ops.reference)."""
import math

import pytest
import torch

from volta_engine_b200.ops import kernels as K
from volta_engine_b200.ops import reference as ref
from volta_engine_b200.quant import nvfp4 as qn
from util import assert_close, cos

pytestmark = pytest.mark.gpu
DEV = "cuda"


def rnd(*shape, std=1.0, seed=0, dtype=torch.bfloat16):
    g = torch.Generator(device=DEV).manual_seed(seed)
    return (torch.randn(*shape, generator=g, device=DEV) * std).to(dtype)


@pytest.mark.parametrize("rows,H", [(1, 512), (7, 5120), (33, 2048)])
def test_rmsnorm_plain_and_fused(rows, H):
    x, w = rnd(rows, H, seed=1), rnd(H, std=0.1, seed=2)
    got = K.rmsnorm(x, w, 1e-6, 1.0)
    want, _ = ref.rmsnorm(x.cpu(), w.cpu(), 1e-6, 1.0)
    assert_close(got.cpu(), want, name="rmsnorm")
    res = rnd(rows, H, seed=3)
    res_ref = res.cpu().clone()
    got = K.rmsnorm(x, w, 1e-6, 0.0, residual=res)
    want, new_res = ref.rmsnorm(x.cpu(), w.cpu(), 1e-6, 0.0, residual=res_ref)
    assert_close(got.cpu(), want, name="rmsnorm fused")
    assert torch.equal(res.cpu(), new_res)


def test_rmsnorm_fp32_residual():
    x, w = rnd(5, 1024, seed=1), rnd(1024, std=0.1, seed=2)
    res = rnd(5, 1024, seed=3, dtype=torch.float32)
    want, new_res = ref.rmsnorm(x.cpu(), w.cpu(), 1e-6, 0.0, residual=res.cpu().clone())
    got = K.rmsnorm(x, w, 1e-6, 0.0, residual=res)
    assert_close(got.cpu(), want, name="rmsnorm f32 res")
    assert_close(res.cpu(), new_res, cos_min=0.999999, rel=1e-6, abs_=1e-6)


def test_embed_and_gated_act():
    table = rnd(1000, 256, seed=4)
    ids = torch.tensor([0, 5, 999, 17], dtype=torch.int32, device=DEV)
    assert torch.equal(K.embed(ids, table), table[ids.long()])
    gu = rnd(9, 2 * 1408, seed=5)
    for act, lim in ((0, 0.0), (0, 1.0), (1, 0.0)):
        assert_close(K.gated_act(gu, 1408, act, lim).cpu(), ref.gated_act(gu.cpu(), 1408, act, lim), name="act")


def _kv_setup(nkv, hd, slots, max_seq, pages, seed=0):
    kpool = torch.zeros(pages, nkv, 64, hd, dtype=torch.bfloat16, device=DEV)
    vpool = torch.zeros_like(kpool)
    maxp = (max_seq + 63) // 64
    table = torch.zeros(slots, maxp, dtype=torch.int32)
    perm = torch.randperm(pages - 1, generator=torch.Generator().manual_seed(seed)) + 1
    table.view(-1)[: min(slots * maxp, pages - 1)] = perm[: slots * maxp].int()
    return kpool, vpool, table.to(DEV)


@pytest.mark.parametrize("interleaved,rot", [(False, 128), (True, 128), (False, 64)])
def test_rope_store(interleaved, rot):
    nq, nkv, hd, rows = 8, 2, 128, 6
    kpool, vpool, table = _kv_setup(nkv, hd, 2, 256, 16)
    qkv = rnd(rows, (nq + 2 * nkv) * hd, seed=6)
    pos = torch.tensor([0, 1, 63, 64, 130, 7], dtype=torch.int32, device=DEV)
    slot = torch.tensor([0, 0, 0, 0, 1, 1], dtype=torch.int32, device=DEV)
    q_ref, k_ref, v_ref = qkv.cpu().clone(), kpool.cpu().clone(), vpool.cpu().clone()
    ref.rope_store(q_ref, pos.cpu(), slot.cpu(), table.cpu(), k_ref, v_ref, nq, nkv, hd, rot, 1e6, interleaved)
    K.rope_store(qkv, pos, slot, table, kpool, vpool, nq, nkv, hd, rot, 1e6, interleaved)
    assert_close(qkv.cpu(), q_ref, name="rope q/k")
    assert_close(kpool.cpu(), k_ref, name="k cache")
    assert torch.equal(vpool.cpu(), v_ref)


def _fill_cache(kpool, vpool, seed):
    g = torch.Generator(device=DEV).manual_seed(seed)
    kpool.copy_(torch.randn(kpool.shape, generator=g, device=DEV).to(torch.bfloat16))
    vpool.copy_(torch.randn(vpool.shape, generator=g, device=DEV).to(torch.bfloat16))


@pytest.mark.parametrize("hd,nq,nkv", [(128, 40, 8), (64, 8, 2), (256, 16, 2)])
@pytest.mark.parametrize("nsplit", [1, 8])
def test_attention_decode(hd, nq, nkv, nsplit):
    kpool, vpool, table = _kv_setup(nkv, hd, 3, 1024, 64)
    _fill_cache(kpool, vpool, 7)
    pos = torch.tensor([0, 63, 64, 500, 1000, 129], dtype=torch.int32, device=DEV)
    slot = torch.tensor([0, 1, 2, 0, 1, -1], dtype=torch.int32, device=DEV)
    rows = pos.numel()
    q = rnd(rows, (nq + 2 * nkv) * hd, seed=8)
    ws = K.AttnWorkspace(rows, nq, hd, 8, DEV)
    got = K.attention(q, pos, slot, table, kpool, vpool, nq, nkv, hd, 1 / math.sqrt(hd), nsplit=nsplit, ws=ws)
    want = ref.attention(q.cpu(), pos.cpu(), slot.cpu(), table.cpu(), kpool.cpu(), vpool.cpu(), nq, nkv, hd,
                         1 / math.sqrt(hd))
    assert_close(got[:5].cpu(), want[:5], name="attn decode")
    assert K.check_status(DEV) == 0


def test_attention_window_and_gate():
    hd, nq, nkv = 128, 8, 2
    kpool, vpool, table = _kv_setup(nkv, hd, 2, 1024, 40)
    _fill_cache(kpool, vpool, 9)
    pos = torch.tensor([700, 20], dtype=torch.int32, device=DEV)
    slot = torch.tensor([0, 1], dtype=torch.int32, device=DEV)
    q = rnd(2, (nq + 2 * nkv) * hd, seed=10)
    gate = rnd(2, nq * hd, seed=11)
    ws = K.AttnWorkspace(2, nq, hd, 4, DEV)
    for nsplit in (1, 4):
        got = K.attention(q, pos, slot, table, kpool, vpool, nq, nkv, hd, 0.1, window=128, gate=gate,
                          nsplit=nsplit, ws=ws)
        want = ref.attention(q.cpu(), pos.cpu(), slot.cpu(), table.cpu(), kpool.cpu(), vpool.cpu(), nq, nkv, hd,
                             0.1, window=128, gate=gate.cpu())
        assert_close(got.cpu(), want, name="attn window+gate")


@pytest.mark.parametrize("hd,nq,nkv,n", [(128, 40, 8, 150), (64, 8, 2, 200), (256, 16, 2, 70)])
def test_attention_prefill(hd, nq, nkv, n):
    kpool, vpool, table = _kv_setup(nkv, hd, 2, 512, 20)
    _fill_cache(kpool, vpool, 12)
    start = 37
    pos = torch.arange(start, start + n, dtype=torch.int32, device=DEV)
    slots = [1] * n
    slot = torch.tensor(slots, dtype=torch.int32, device=DEV)
    q = rnd(n, (nq + 2 * nkv) * hd, seed=13)
    tiles = K.make_prefill_tiles(slots, nq // nkv, DEV)
    got = K.attention(q, pos, slot, table, kpool, vpool, nq, nkv, hd, 1 / math.sqrt(hd), tiles=tiles)
    want = ref.attention(q.cpu(), pos.cpu(), slot.cpu(), table.cpu(), kpool.cpu(), vpool.cpu(), nq, nkv, hd,
                         1 / math.sqrt(hd))
    assert_close(got.cpu(), want, rel=0.01, name="attn prefill")  # P is rounded to bf16 for the PV MMA


@pytest.mark.parametrize("nq,nkv,start,n,window,gated", [(40, 8, 0, 40, 0, False), (40, 8, 1000, 700, 0, False),
                                                         (16, 16, 300, 300, 0, False), (32, 4, 500, 260, 192, True)])
def test_attention_prefill_tcgen05(nq, nkv, start, n, window, gated):
    """The tcgen05 prefill kernel (128-row tiles, two softmax streams, lazy rescale) against the fp32 oracle and the
    mma.sync kernel: one-page tiles, many pages, G = 1 and G = 8, sliding window with a sigmoid gate, two sequences."""
    hd = 128
    kpool, vpool, table = _kv_setup(nkv, hd, 2, 2048, 70)
    _fill_cache(kpool, vpool, 21)
    half = n // 2
    slots = [1] * half + [0] * (n - half)                     # two sequences in one launch
    pos = torch.tensor([start + i for i in range(half)] + [start // 2 + i for i in range(n - half)], dtype=torch.int32, device=DEV)
    slot = torch.tensor(slots, dtype=torch.int32, device=DEV)
    q = rnd(n, (nq + 2 * nkv) * hd, seed=22)
    gate = rnd(n, nq * hd, seed=23) if gated else None
    tiles = K.make_prefill_tiles(slots, nq // nkv, DEV)
    assert len(tiles) == 4 and tiles[3][2] <= tiles[2]
    got = K.attention(q, pos, slot, table, kpool, vpool, nq, nkv, hd, 1 / math.sqrt(hd), tiles=tiles, window=window, gate=gate)
    old = K.ATTN_PREFILL_TC
    K.ATTN_PREFILL_TC = False
    try:
        mma = K.attention(q, pos, slot, table, kpool, vpool, nq, nkv, hd, 1 / math.sqrt(hd), tiles=tiles, window=window, gate=gate)
    finally:
        K.ATTN_PREFILL_TC = old
    want = ref.attention(q.cpu(), pos.cpu(), slot.cpu(), table.cpu(), kpool.cpu(), vpool.cpu(), nq, nkv, hd,
                         1 / math.sqrt(hd), window, None, gate.cpu() if gated else None)
    assert K.check_status(torch.device(DEV)) == 0
    assert_close(got.cpu(), want, rel=0.01, name="attn prefill tcgen05")
    assert_close(mma.cpu(), want, rel=0.01, name="attn prefill mma.sync")


def test_attention_prefill_tcgen05_key_end():
    """Bidirectional rows (key_end past the row's own position) on the tcgen05 kernel."""
    hd, nq, nkv, n, start = 128, 8, 2, 90, 100
    kpool, vpool, table = _kv_setup(nkv, hd, 2, 512, 20)
    _fill_cache(kpool, vpool, 31)
    pos = torch.arange(start, start + n, dtype=torch.int32, device=DEV)
    slot = torch.ones(n, dtype=torch.int32, device=DEV)
    key_end = pos.clone()
    key_end[20:60] = start + 59                                # an image span: every row sees the whole span
    q = rnd(n, (nq + 2 * nkv) * hd, seed=32)
    tiles = K.make_prefill_tiles([1] * n, nq // nkv, DEV)
    got = K.attention(q, pos, slot, table, kpool, vpool, nq, nkv, hd, 1 / math.sqrt(hd), tiles=tiles, key_end=key_end)
    want = ref.attention(q.cpu(), pos.cpu(), slot.cpu(), table.cpu(), kpool.cpu(), vpool.cpu(), nq, nkv, hd,
                         1 / math.sqrt(hd), 0, key_end.cpu())
    assert_close(got.cpu(), want, rel=0.01, name="attn prefill tcgen05 key_end")


def test_argmax_topk():
    logits = rnd(5, 151936 // 8, seed=14, dtype=torch.float32)
    logits[2, 100] = logits[2, 7] = 50.0  # tie -> lowest id
    idx, val = K.argmax(logits, id_offset=1000)
    ridx, rval = ref.argmax(logits.cpu(), 1000)
    assert torch.equal(idx.cpu(), ridx) and torch.equal(val.cpu(), rval)
    assert int(idx[2]) == 1007
    ids, vals, lse = K.topk(logits, 16)
    rids, rvals, rlse = ref.topk(logits.cpu(), 16)
    assert torch.equal(ids.cpu(), rids) and torch.equal(vals.cpu(), rvals)
    assert_close(lse.cpu(), rlse, rel=1e-5, abs_=1e-4)


def test_nvfp4_dequant_and_quant_rows():
    w = rnd(256, 512, std=0.02, seed=15, dtype=torch.float32)
    p, s, g = qn.quantize_nvfp4(w)
    want = qn.dequantize_nvfp4(p.cpu(), s.cpu(), g)
    got = K.nvfp4_dequant(p, s, g)
    assert_close(got.cpu(), want, cos_min=0.9999, rel=0.004, name="dequant")
    x = rnd(40, 512, seed=16)
    xp, xs = K.nvfp4_quant_rows(x, blocked=False)
    rp, rs = qn.quantize_rows_nvfp4(x.cpu())
    assert torch.equal(xs.cpu(), rs)
    assert (xp.cpu() != rp).float().mean() < 1e-3  # identical up to rare division rounding
    xp2, xs2 = K.nvfp4_quant_rows(x, blocked=True)
    assert torch.equal(xs2.cpu(), qn.scales_atoms_512(rs))


@pytest.mark.parametrize("N,Kd", [(5120, 5120), (1024, 17408), (130, 256)])
def test_nvfp4_gemv_rows_and_batch_invariance(N, Kd):
    w = rnd(N, Kd, std=0.02, seed=17, dtype=torch.float32)
    p, s, g = qn.quantize_nvfp4(w, search=False)
    wd = qn.dequantize_nvfp4(p.cpu(), s.cpu(), g)
    x = rnd(16, Kd, seed=18)
    res = rnd(16, N, seed=19)
    full = K.nvfp4_gemv(p, s, g, x)
    want = x.cpu().float() @ wd.t()
    assert_close(full.cpu(), want, name="gemv M=16")
    for m in (1, 2, 3, 5):
        part = K.nvfp4_gemv(p, s, g, x[:m])
        assert torch.equal(part, full[:m]), f"row result depends on batch size (M={m})"
    wres = K.nvfp4_gemv(p, s, g, x[:3], residual=res[:3])
    assert_close(wres.cpu(), want[:3] + res[:3].cpu().float(), name="gemv residual")


def test_bf16_gemv_f32():
    W, x = rnd(4096 + 3, 1024, std=0.05, seed=20), rnd(6, 1024, seed=21)
    got = K.bf16_gemv_f32(W, x)
    assert_close(got.cpu(), x.cpu().float() @ W.cpu().float().t(), rel=1e-3, name="lm head gemv")


@pytest.mark.parametrize("N,Kd", [(5120, 5120), (1024, 17408), (7168, 5120), (48, 128)])
def test_nvfp4_gemv_mma_exact_and_batch_invariant(N, Kd):
    w = rnd(N, Kd, std=0.02, seed=27, dtype=torch.float32)
    p, s, g = qn.quantize_nvfp4(w, search=False)
    s[0, 0] = 3       # force E4M3 subnormal scales and zero scales through the decode path
    s[1, 1] = 0
    wd = qn.dequantize_nvfp4(p.cpu(), s.cpu(), g)
    wg, sg = qn.prepack_gv(p, s)
    x = rnd(16, Kd, seed=28)
    x[0, :8] = 0
    res = rnd(16, N, seed=29)
    want = x.cpu().float() @ wd.t()
    full = K.nvfp4_gemv_mma(wg, sg, g, x, N, Kd)
    assert_close(full.cpu(), want, name="gemv mma M=16")
    for m in (1, 2, 5, 8, 9):
        part = K.nvfp4_gemv_mma(wg, sg, g, x[:m], N, Kd)
        assert torch.equal(part, full[:m]), f"row result depends on batch size (M={m})"
    for ks in (1, 2, 4):
        if ks <= (Kd // 64) // 4 or ks == 1:
            alt = K.nvfp4_gemv_mma(wg, sg, g, x[:3], N, Kd, ks=ks)
            assert_close(alt.cpu(), want[:3], name=f"gemv mma ks={ks}")
    wres = K.nvfp4_gemv_mma(wg, sg, g, x[:3], N, Kd, residual=res[:3])
    assert_close(wres.cpu(), want[:3] + res[:3].cpu().float(), name="gemv mma residual")
    # products are exact and accumulated in fp32: compare against the fp64 product at fp32-level tolerance
    one = K.nvfp4_gemv_mma(wg, sg, g, x[:1], N, Kd).float().cpu()
    ref64 = (x[:1].cpu().double() @ wd.double().t()).float()
    assert (one - ref64.to(torch.bfloat16).float()).abs().max() <= 2 * ref64.abs().max() * 2 ** -8


def test_argmax_wide_two_stage():
    logits = rnd(3, 151936, seed=30, dtype=torch.float32)
    logits[1, 151935] = 99.0
    idx, val = K.argmax(logits, id_offset=5)
    ridx, rval = ref.argmax(logits.cpu(), 5)
    assert torch.equal(idx.cpu(), ridx) and torch.equal(val.cpu(), rval)


@pytest.mark.parametrize("gtype", [3, 6, 7, 10, 11, 13, 20, 23])
def test_gguf_read_only_formats_on_synthetic_blocks(gtype):
    """Q4_1, Q5_0/1, Q2_K, Q3_K, Q5_K, IQ4_NL/XS: random payload bytes with finite scales; fused mat-vec and the
    dequantise kernel against the PyTorch block decoder."""
    from volta_engine_b200.ops.linear_gguf import LinearGGUF
    from volta_engine_b200.quant import gguf as gq
    N, Kd = 520, 1024
    raw = gq.random_blocks(gtype, N, Kd, seed=gtype, amp=0.01)
    lin = LinearGGUF(raw.to(DEV), gtype, N, Kd)
    wd = gq.dequantize(raw, gtype, Kd)
    assert_close(lin.dequant().cpu(), wd, cos_min=0.9999, rel=0.004, name=f"gguf dequant type {gtype}")
    x = rnd(5, Kd, seed=43)
    assert_close(lin.forward(x).cpu(), x.cpu().float() @ wd.t(), name=f"gguf gemv type {gtype}")


@pytest.mark.parametrize("gtype", [8, 2, 12, 14])
def test_gguf_fused_gemv_and_dequant(gtype):
    from volta_engine_b200.ops.linear_gguf import LinearGGUF
    from volta_engine_b200.quant import gguf as gq
    N, Kd = 1000, 2048
    w = rnd(N, Kd, std=0.02, seed=40, dtype=torch.float32)
    lin = LinearGGUF.from_dense(w, gtype)
    wd = gq.dequantize(lin.raw.cpu(), gtype, Kd)
    assert_close(lin.dequant().cpu(), wd, cos_min=0.9999, rel=0.004, name="gguf dequant")
    x = rnd(16, Kd, seed=41)
    want = x.cpu().float() @ wd.t()
    full = lin.forward(x)
    assert_close(full.cpu(), want, name=f"gguf gemv type {gtype}")
    one = lin.forward(x[:1])
    assert torch.equal(one, full[:1]), "first row differs between M=1 and M=16"
    big = lin.forward(rnd(40, Kd, seed=42))
    assert_close(big.cpu(), rnd(40, Kd, seed=42).cpu().float() @ wd.t(), name="gguf prefill path")


def test_rope_store_multimodal_sections():
    nq, nkv, hd, rows = 8, 2, 128, 5
    kpool, vpool, table = _kv_setup(nkv, hd, 2, 256, 16)
    qkv = rnd(rows, (nq + 2 * nkv) * hd, seed=26)
    pos = torch.tensor([0, 1, 2, 3, 40], dtype=torch.int32, device=DEV)
    slot = torch.tensor([0, 0, 0, 0, 1], dtype=torch.int32, device=DEV)
    pos3 = torch.tensor([[0, 1, 1, 1, 9], [0, 0, 1, 1, 9], [0, 0, 0, 5, 9]], dtype=torch.int32, device=DEV)
    q_ref, k_ref, v_ref = qkv.cpu().clone(), kpool.cpu().clone(), vpool.cpu().clone()
    ref.rope_store(q_ref, pos.cpu(), slot.cpu(), table.cpu(), k_ref, v_ref, nq, nkv, hd, 128, 1e6, False, 1.0,
                   (pos3.cpu(), (16, 24)))
    K.rope_store(qkv, pos, slot, table, kpool, vpool, nq, nkv, hd, 128, 1e6, False, 1.0, (pos3, (16, 24)))
    assert_close(qkv.cpu(), q_ref, name="mrope q/k")
    assert_close(kpool.cpu(), k_ref, name="mrope k cache")
    # equal positions in the three rows reduce to the ordinary rotary embedding
    q2 = rnd(rows, (nq + 2 * nkv) * hd, seed=26)
    same = torch.stack([pos, pos, pos]).contiguous()
    a, b = q2.clone(), q2.clone()
    K.rope_store(a, pos, slot, table, kpool.clone(), vpool.clone(), nq, nkv, hd, 128, 1e6, False, 1.0, (same, (16, 24)))
    K.rope_store(b, pos, slot, table, kpool.clone(), vpool.clone(), nq, nkv, hd, 128, 1e6, False)
    assert torch.equal(a, b)


def test_bounded_wait_reports_through_the_status_word():
    """A wait on a flag that nothing sets runs out after its budget, records the peer-timeout code in the status word and
    returns; the context stays usable and a wait whose flag is already set finishes clean."""
    from volta_engine_b200._lib import call, ptr
    import time
    flag = torch.zeros(1, dtype=torch.int32, device=DEV)
    status = torch.zeros(1, dtype=torch.int32, device=DEV)
    t0 = time.time()
    call("wait_flag", "pilp", ptr(flag), 1, 50_000_000, ptr(status))          # 50 ms budget
    torch.cuda.synchronize()
    assert int(status.item()) == 2 and time.time() - t0 < 2.0                   # kErrPeerTimeout
    # the status word is sticky: a second wait on the same dead flag returns at once instead of spending its budget again
    t1 = time.time()
    call("wait_flag", "pilp", ptr(flag), 1, 2_000_000_000, ptr(status))        # 2 s budget that must not be used
    torch.cuda.synchronize()
    assert int(status.item()) == 2 and time.time() - t1 < 0.5
    status.zero_()
    flag.fill_(1)
    call("wait_flag", "pilp", ptr(flag), 1, 50_000_000, ptr(status))
    torch.cuda.synchronize()
    assert int(status.item()) == 0
    x = torch.ones(4, device=DEV)
    assert float((x + 1).sum()) == 8.0                                          # the context still works
