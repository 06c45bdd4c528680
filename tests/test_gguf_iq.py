"""Codebook GGUF formats (IQ1_S .. IQ3_S) and routed experts stored as GGUF blocks: the PyTorch decoders are the
statement (bit-equal to ggml's row dequantisers, see test_cpu_core); the CUDA decoders and mat-vecs are held to it."""
import pytest
import torch

from volta_engine_b200.quant import gguf as G
from volta_engine_b200.quant import gguf_iq as Q

IQ = sorted(Q.IQ_BLOCK)


def test_grid_file_layout_and_block_sizes():
    assert len(Q.grid_blob()) == Q.GRID_BYTES == 33920
    T = Q.tables()
    assert T["1s"].shape == (2048, 8) and set(T["1s"].unique().tolist()) == {-1.0, 0.0, 1.0}
    assert T["3s"].shape == (512, 4) and T["2s"].shape == (1024, 8)
    # the sign table: bit 7 makes the number of set bits even
    for i in (0, 1, 3, 77, 127):
        assert bin(int(T["signs"][i])).count("1") % 2 == 0 and int(T["signs"][i]) & 127 == i
    for t in IQ:
        n, bs = Q.IQ_BLOCK[t]
        assert G.row_bytes(t, 512) == 2 * bs and G.BLOCK[t] == (n, bs)
        y = G.dequantize(G.random_blocks(t, 3, 512, seed=t), t, 512)
        assert y.shape == (3, 512) and torch.isfinite(y).all() and float(y.abs().max()) > 0


def test_moe_model_with_gguf_experts_runs_on_cpu():
    from volta_engine_b200.models.moe import MoEConfig, MoEModel
    from volta_engine_b200.ops.moe_gguf import GGUFExpertBank, parse_expert_quant
    from volta_engine_b200.runtime.engine import Engine
    from volta_engine_b200.runtime.kv_cache import PagedKVCache
    assert parse_expert_quant("gguf_iq2_xxs+q4_k") == (G.GGML_IQ2_XXS, G.GGML_Q4_K)
    with pytest.raises(ValueError):
        parse_expert_quant("gguf_nope")
    cfg = MoEConfig.tiny_moe(expert_quant="gguf_iq2_xs+q4_k", hidden=256, expert_ffn=256)
    m = MoEModel(cfg, "cpu").init_random(seed=3)
    assert isinstance(m.layers[0].bank, GGUFExpertBank) and m.layers[0].bank.gu_type == G.GGML_IQ2_XS
    kv = PagedKVCache(2, m.nkv, 64, 16, 1, 512, "cpu")
    prompt = torch.randint(0, cfg.vocab, (40,), generator=torch.Generator().manual_seed(1)).tolist()
    out, _ = Engine(m, kv, use_graphs=False, prefill_chunk=16).generate(prompt, 5)
    assert len(out) == 5
    # a bank quantised from dense weights decodes back within the step of its type
    gu, dn = torch.randn(2, 512, 256) * 0.05, torch.randn(2, 256, 256) * 0.05
    bank = GGUFExpertBank.from_dense(gu, dn, G.GGML_Q8_0, G.GGML_Q4_K)
    assert float((bank.dequant("gu", 1) - gu[1]).abs().max()) < 2e-3
    assert float((bank.dequant("dn", 0) - dn[0]).abs().max()) < 3e-2


@pytest.mark.gpu
@pytest.mark.parametrize("t", IQ)
def test_gpu_iq_dequant_and_matvec_match_the_statement(t):
    from volta_engine_b200.ops.linear_gguf import LinearGGUF
    dev = "cuda"
    N, Kd = 264, 1024
    raw = G.random_blocks(t, N, Kd, seed=50 + t, amp=0.05)
    want = G.dequantize(raw, t, Kd)
    lin = LinearGGUF(raw.to(dev), t, N, Kd)
    got = lin.dequant().float().cpu()
    assert torch.equal(got, want.to(torch.bfloat16).float()), Q.IQ_NAMES[t]
    g = torch.Generator().manual_seed(t)
    for rows in (1, 5, 16):
        x = (torch.randn(rows, Kd, generator=g)).to(torch.bfloat16)
        y = lin.forward(x.to(dev), out_f32=True).cpu()
        ref = x.float() @ want.t()
        assert torch.allclose(y, ref, atol=2e-3 * float(ref.abs().max()) + 1e-4, rtol=2e-3), (Q.IQ_NAMES[t], rows)
        one = lin.forward(x[:1].to(dev), out_f32=True).cpu()
        assert torch.equal(one[0], y[0]), "row 0 of a block equals the one-row product bit for bit"
    big = (torch.randn(40, Kd, generator=g)).to(torch.bfloat16)
    yb = lin.forward(big.to(dev)).float().cpu()
    refb = big.float() @ want.to(torch.bfloat16).float().t()
    assert torch.allclose(yb, refb, atol=2e-2 * float(refb.abs().max()), rtol=2e-2)


@pytest.mark.gpu
@pytest.mark.parametrize("spec", ["gguf_iq2_xxs+q4_k", "gguf_iq1_m+iq3_s", "gguf_q4_k+q6_k"])
def test_gpu_routed_experts_in_gguf_blocks(spec):
    from volta_engine_b200.ops.moe_gguf import GGUFExpertBank, parse_expert_quant
    dev = "cuda"
    gt, dt = parse_expert_quant(spec)
    E, I, H, k = 8, 256, 512, 2
    bank_c = GGUFExpertBank.random(E, I, H, gt, dt, e0=4, seed=9, amp=0.05)
    bank_g = bank_c.to(dev)
    g = torch.Generator().manual_seed(2)
    for rows in (1, 7, 16, 150):
        x = torch.randn(rows, H, generator=g).to(torch.bfloat16)
        ids = torch.randint(0, 16, (rows, k), generator=g, dtype=torch.int32)     # experts 4..11 are local, the rest elsewhere
        want = bank_c.routes(x, ids, 0, 0.0).float()
        got = bank_g.routes(x.to(dev), ids.to(dev), 0, 0.0).float().cpu()
        scale = float(want.abs().max()) + 1e-6
        assert float((got - want).abs().max()) < 3e-2 * scale, (spec, rows, float((got - want).abs().max()), scale)
        away = ((ids < 4) | (ids >= 12)).reshape(-1)
        assert float(got[away].abs().max()) == 0.0 if away.any() else True
    from volta_engine_b200.ops import kernels as K
    assert K.check_status(dev) == 0


@pytest.mark.gpu
def test_gpu_moe_model_with_gguf_experts_matches_the_cpu_statement():
    from volta_engine_b200.models.moe import MoEConfig, MoEModel
    from volta_engine_b200.models.util import to_device
    from volta_engine_b200.runtime.batch import BatchRows
    from volta_engine_b200.runtime.kv_cache import PagedKVCache
    from util import cos
    cfg = MoEConfig.tiny_moe(expert_quant="gguf_iq3_xxs+q4_k", hidden=256, expert_ffn=256)
    mc = MoEModel(cfg, "cpu").init_random(seed=3)
    mg = to_device(mc, "cuda")
    mg.ensure_workspace(16, 8)
    prompt = torch.randint(0, cfg.vocab, (90,), generator=torch.Generator().manual_seed(1)).tolist()
    kvg, kvc = PagedKVCache(2, mg.nkv, 64, 16, 1, 512, "cuda"), PagedKVCache(2, mc.nkv, 64, 16, 1, 512, "cpu")
    kvg.reserve(0, 128)
    kvc.reserve(0, 128)
    G_ = mg.nq // mg.nkv
    lg = mg.forward(BatchRows.make(prompt, list(range(90)), [0] * 90, "cuda", "last", G_, prefill=True), kvg)
    lc = mc.forward(BatchRows.make(prompt, list(range(90)), [0] * 90, "cpu", "last", G_, prefill=True), kvc)
    assert cos(lg.cpu(), lc) > 0.99
    dg = mg.forward(BatchRows.make([5, 6], [90, 91], [0, 0], "cuda", "all", G_, nsplit=2), kvg)
    dc = mc.forward(BatchRows.make([5, 6], [90, 91], [0, 0], "cpu", "all", G_), kvc)
    assert cos(dg.cpu(), dc) > 0.99
