"""MoE kernels and model on the GPU against the fp32 CPU statement."""
import pytest
import torch

from volta_engine_b200._lib import call, ptr
from volta_engine_b200.models.moe import MoEConfig, MoEModel, route_reference
from volta_engine_b200.runtime.batch import BatchRows
from volta_engine_b200.runtime.engine import Engine
from volta_engine_b200.runtime.kv_cache import PagedKVCache
from util import assert_close, cos

pytestmark = pytest.mark.gpu
DEV = "cuda"


@pytest.mark.parametrize("router,n_group,topk_group,E,k", [("softmax", 1, 1, 512, 10), ("sigmoid", 1, 1, 128, 8),
                                                          ("sigmoid", 8, 4, 256, 8)])
def test_router_select(router, n_group, topk_group, E, k):
    cfg = MoEConfig(n_experts=E, top_k=k, router=router, router_scale=2.5 if router == "sigmoid" else 1.0,
                    n_group=n_group, topk_group=topk_group)
    g = torch.Generator(device=DEV).manual_seed(0)
    logits = torch.randn(7, E, generator=g, device=DEV)
    logits[3, 5] = logits[3, 9]                      # a tie: lowest index first
    bias = torch.randn(E, generator=g, device=DEV) * 0.1 if router == "sigmoid" else None
    ids = torch.empty(7, k, dtype=torch.int32, device=DEV)
    w = torch.empty(7, k, dtype=torch.float32, device=DEV)
    heat = torch.zeros(E, dtype=torch.float32, device=DEV)
    call("router_select", "pliiiipfiippp", ptr(logits), logits.stride(0), 7, E, k, 1 if router == "sigmoid" else 0,
         ptr(bias), float(cfg.router_scale), n_group, topk_group, ptr(ids), ptr(w), ptr(heat))
    assert torch.equal(heat.cpu(), torch.bincount(ids.cpu().flatten().long(), minlength=E).float())
    rid, rw = route_reference(logits.cpu(), cfg, bias.cpu() if bias is not None else None)
    assert torch.equal(ids.cpu(), rid)
    assert_close(w.cpu(), rw, rel=1e-4, abs_=1e-5, name="router weights")


@pytest.mark.parametrize("mode", [0, 1])
def test_router_select_keeps_ids_in_range_on_nan_and_inf_rows(mode):
    """A row of NaN or infinite logits (an overflowed hidden state) must give expert ids inside [0, E) and finite weights:
    the ids index shared and global memory in the kernels behind the router."""
    from volta_engine_b200._lib import NativeError
    E, k = 64, 6
    logits = torch.randn(4, E, device=DEV)
    logits[0] = float("nan")
    logits[1] = float("-inf")
    logits[2, ::2] = float("inf")
    ids = torch.full((4, k), -7, dtype=torch.int32, device=DEV)
    w = torch.empty(4, k, dtype=torch.float32, device=DEV)
    heat = torch.zeros(E, dtype=torch.float32, device=DEV)
    call("router_select", "pliiiipfiippp", ptr(logits), logits.stride(0), 4, E, k, mode, 0, 1.0, 1, 1, ptr(ids), ptr(w), ptr(heat))
    torch.cuda.synchronize()
    assert int(ids.min()) >= 0 and int(ids.max()) < E
    for r in range(4):
        assert len(set(ids[r].tolist())) == k                      # distinct experts
    assert bool(torch.isfinite(w).all())
    assert float(heat.sum()) == 4 * k
    for bad in [dict(topk=E + 1), dict(n_group=8, topk_group=9), dict(n_group=8, topk_group=0), dict(n_group=64, topk_group=1)]:
        a = dict(topk=k, n_group=1, topk_group=1)
        a.update(bad)
        ids2 = torch.empty(4, max(a["topk"], 1), dtype=torch.int32, device=DEV)
        w2 = torch.empty(4, max(a["topk"], 1), dtype=torch.float32, device=DEV)
        with pytest.raises(NativeError):
            call("router_select", "pliiiipfiippp", ptr(logits), logits.stride(0), 4, E, a["topk"], mode, 0, 1.0, a["n_group"],
                 a["topk_group"], ptr(ids2), ptr(w2), 0)


def _models(**kw):
    cfg = MoEConfig.tiny_moe(**kw)
    m_gpu = MoEModel(cfg, DEV).init_random(seed=4)
    m_cpu = MoEModel(MoEConfig.tiny_moe(**kw), "cpu")
    # same weights on the CPU: copy tensors instead of re-drawing (CPU and CUDA generators differ)
    m_cpu.embed, m_cpu.final_norm = m_gpu.embed.cpu(), m_gpu.final_norm.cpu()
    import copy
    for L in m_gpu.layers:
        Lc = copy.copy(L)
        for name in ("qkv", "o_proj", "shared_gu", "shared_dn", "gate_up", "down"):
            lin = getattr(L, name, None)
            if lin is not None:
                c = copy.copy(lin)
                c.packed, c.scales = lin.packed.cpu(), lin.scales.cpu()
                c._gv = c._sf_k128 = c._sf_atoms = None
                setattr(Lc, name, c)
        Lc.attn_norm, Lc.ffn_norm = L.attn_norm.cpu(), L.ffn_norm.cpu()
        if not L.dense_ffn:
            Lc.router = type(L.router)(L.router.weight.cpu())
            Lc.router_bias = L.router_bias.cpu() if L.router_bias is not None else None
            b = copy.copy(L.bank)
            for n in ("gu_p", "gu_s", "gu_g", "dn_p", "dn_s", "dn_g"):
                setattr(b, n, getattr(L.bank, n).cpu())
            b.gu_sf = b.dn_sf = None
            Lc.bank = b
        m_cpu.layers.append(Lc)
    m_cpu.lm_head = type(m_gpu.lm_head)(m_gpu.lm_head.weight.cpu())
    return m_gpu, m_cpu


@pytest.mark.parametrize("rows", [1, 5, 200])
def test_moe_ffn_block_matches_reference(rows):
    m_gpu, m_cpu = _models()
    g = torch.Generator(device=DEV).manual_seed(rows)
    x = torch.randn(rows, m_gpu.cfg.hidden, generator=g, device=DEV).to(torch.bfloat16)
    L, Lc = m_gpu.layers[0], m_cpu.layers[0]
    got = m_gpu.ffn_block(0, L, x, None, None)
    want = m_cpu.ffn_block(0, Lc, x.cpu(), None, None)
    assert_close(got.cpu(), want, rel=0.02, name=f"moe ffn rows={rows}")


def test_shared_expert_on_a_side_stream_gives_the_same_bits_eager_and_in_a_graph():
    m_gpu, _ = _models()
    prompt = torch.randint(0, m_gpu.cfg.vocab, (70,), generator=torch.Generator().manual_seed(3)).tolist()
    runs = []
    for side, graphs in ((False, True), (True, True), (True, False)):
        m_gpu.side_streams = side
        eng = Engine(m_gpu, PagedKVCache(2, m_gpu.nkv, 64, 16, 1, 512, DEV), prefill_chunk=64, use_graphs=graphs)
        out, _ = eng.generate(prompt, 12)
        runs.append(out)
    m_gpu.side_streams = False
    assert runs[0] == runs[1] == runs[2], runs


def test_kv_pools_and_workspaces_carved_from_one_arena():
    from volta_engine_b200.ops import kernels as K
    from volta_engine_b200.runtime.arena import Arena, ScratchRegistry
    m_gpu, _ = _models()
    pages = 16
    need = PagedKVCache.pool_bytes(2, m_gpu.nkv, 64, pages, "bf16")
    arena = Arena(need + (8 << 20), DEV)
    kv = PagedKVCache(2, m_gpu.nkv, 64, pages, 1, 512, DEV, arena=arena)
    lo, hi = arena.buf.data_ptr(), arena.buf.data_ptr() + arena.capacity
    assert lo <= kv.k.data_ptr() < hi and lo <= kv.v.data_ptr() < hi and kv.k.data_ptr() % 256 == 0
    assert arena.report()["by_name"]["kv"] >= need - 4 * 256
    reg = ScratchRegistry(arena, overflow=True)
    a = reg.typed("t/a", (1024,), torch.float32)
    assert lo <= a.data_ptr() < hi and reg.typed("t/a", (1024,), torch.float32).data_ptr() == a.data_ptr()
    big = reg.typed("t/big", (16 << 20,), torch.uint8)          # does not fit: allocated by itself, counted
    assert not (lo <= big.data_ptr() < hi) and reg.overflow_bytes == 16 << 20
    prompt = torch.randint(0, m_gpu.cfg.vocab, (70,), generator=torch.Generator().manual_seed(3)).tolist()
    out_a, _ = Engine(m_gpu, kv, prefill_chunk=64).generate(prompt, 8)
    out_b, _ = Engine(m_gpu, PagedKVCache(2, m_gpu.nkv, 64, pages, 1, 512, DEV), prefill_chunk=64).generate(prompt, 8)
    assert out_a == out_b


def test_moe_model_generates_like_reference_and_zipf_bias():
    m_gpu, m_cpu = _models(router_bias_zipf=1.2)
    prompt = torch.randint(0, m_gpu.cfg.vocab, (90,), generator=torch.Generator().manual_seed(1)).tolist()
    kv = PagedKVCache(2, m_gpu.nkv, 64, 16, 1, 512, DEV)
    kvc = PagedKVCache(2, m_cpu.nkv, 64, 16, 1, 512, "cpu")
    b = BatchRows.make(prompt, list(range(90)), [0] * 90, DEV, "last", m_gpu.nq // m_gpu.nkv, prefill=True)
    bc = BatchRows.make(prompt, list(range(90)), [0] * 90, "cpu", "last", m_cpu.nq // m_cpu.nkv, prefill=True)
    kv.reserve(0, 128)
    kvc.reserve(0, 128)
    lg, lc = m_gpu.forward(b, kv), m_cpu.forward(bc, kvc)
    assert cos(lg.cpu(), lc) > 0.995
    out, _ = Engine(m_gpu, PagedKVCache(2, m_gpu.nkv, 64, 16, 1, 512, DEV), prefill_chunk=64).generate(prompt, 6)
    assert len(out) == 6


def test_expert_tier_reads_cold_experts_in_place_and_rebalances():
    """Two of eight experts resident: the tiered layer (cold experts read from pinned host memory through the pointer
    table) gives the stacked bank's bits; the routing histogram moves the busiest experts into the device slots."""
    m_gpu, _ = _models()
    m_ref, _ = _models()
    E = m_gpu.cfg.n_experts
    tiers = m_gpu.enable_expert_tier(2)
    assert tiers and all(t.resident() == [0, 1] for _, t in tiers) and m_gpu.layers[0].bank.gu_p is None
    g = torch.Generator(device=DEV).manual_seed(5)
    for rows in (1, 6, 40):
        x = torch.randn(rows, m_gpu.cfg.hidden, generator=g, device=DEV).to(torch.bfloat16)
        got = m_gpu.ffn_block(0, m_gpu.layers[0], x, None, None)
        m_ref.layers[0].bank.gu_sf = None                      # same route-indexed kernel on the stacked bank
        want = m_ref.ffn_block(0, m_ref.layers[0], x, None, None)
        assert torch.equal(got, want), f"tiered != stacked at rows={rows}"
    assert float(m_gpu.heat[0].sum()) == (1 + 6 + 40) * m_gpu.cfg.top_k
    swaps = m_gpu.rebalance_experts(max_swaps=2)
    tier = tiers[0][1]
    top2 = sorted(torch.topk(m_gpu.heat[0].cpu(), 2).indices.tolist())
    assert swaps >= 1 and len(tier.resident()) == 2 and set(tier.resident()) & set(top2)
    x = torch.randn(3, m_gpu.cfg.hidden, generator=g, device=DEV).to(torch.bfloat16)
    assert torch.equal(m_gpu.ffn_block(0, m_gpu.layers[0], x, None, None), m_ref.ffn_block(0, m_ref.layers[0], x, None, None))
    torch.cuda.synchronize()
    assert tier.device_bytes() * (E // 2) == tier.host_bytes()


def test_cpu_expert_service_answers_through_the_mailbox_and_a_stopped_service_times_out():
    from volta_engine_b200.ops import kernels as K
    from volta_engine_b200.runtime.cpu_experts import attach_cpu_experts
    m_gpu, _ = _models()
    m_ref, _ = _models()
    svc = attach_cpu_experts(m_gpu, 0.5, budget_ms=5000.0)
    try:
        L = m_gpu.layers[0]
        assert L.cpu.owner.cpu().tolist() == [0, 0, 0, 0, 1, 1, 1, 1] and float(L.bank.gu_p[4:].float().abs().sum()) == 0
        g = torch.Generator(device=DEV).manual_seed(9)
        for rows in (1, 6, 40):
            x = torch.randn(rows, m_gpu.cfg.hidden, generator=g, device=DEV).to(torch.bfloat16)
            got = m_gpu.ffn_block(0, L, x, None, None)
            want = m_ref.ffn_block(0, m_ref.layers[0], x, None, None)
            torch.cuda.synchronize()
            assert_close(got.cpu(), want.cpu(), rel=0.03, name=f"host + device experts rows={rows}")
        assert svc.served >= 3 and K.check_status(x.device) == 0
        # a whole model generates through CUDA graphs with the host in the loop
        prompt = torch.randint(0, m_gpu.cfg.vocab, (40,), generator=torch.Generator().manual_seed(1)).tolist()
        out, _ = Engine(m_gpu, PagedKVCache(2, m_gpu.nkv, 64, 16, 1, 512, DEV), prefill_chunk=64).generate(prompt, 6)
        ref_out, _ = Engine(m_ref, PagedKVCache(2, m_ref.nkv, 64, 16, 1, 512, DEV), prefill_chunk=64).generate(prompt, 6)
        assert len(out) == 6 and out[0] == ref_out[0]
    finally:
        svc.stop()
    # nobody answers: the wait runs out after its budget, reports through the status word, and the context lives on
    for Lx in m_gpu.layers:
        if getattr(Lx, "cpu", None) is not None:
            Lx.cpu.budget_ns = 50_000_000
    x = torch.randn(8, m_gpu.cfg.hidden, device=DEV).to(torch.bfloat16)       # 16 routes: some go to host-owned experts
    m_gpu.ffn_block(0, m_gpu.layers[0], x, None, None)
    torch.cuda.synchronize()
    assert K.check_status(x.device) == 2
    K.status_word(x.device).zero_()
    assert float((x.float() + 1).sum()) != 0


def test_expert_staging_gives_the_in_place_bits_and_copies_a_layer_once_while_it_stays_staged():
    """Prefill rows of a tiered model with the cold experts staged a layer ahead: the same bits as reading them in place
    from pinned host memory; a layer's cold set is copied once for as long as its buffer keeps it; rows at or below 16 do
    not stage; a rebalance makes the next chunk copy the new cold set."""
    m, _ = _models()
    tiers = m.enable_expert_tier(2)
    g = torch.Generator(device=DEV).manual_seed(9)
    xs = {rows: torch.randn(rows, m.cfg.hidden, generator=g, device=DEV).to(torch.bfloat16) for rows in (6, 40, 200)}
    idx = [li for li, _ in tiers]
    want = {rows: [m.ffn_block(li, m.layers[li], x, None, None).clone() for li in idx] for rows, x in xs.items()}
    st = m.enable_expert_staging()
    assert st is not None and st.n_cold == m.e_local - 2
    for rep in range(2):
        for rows, x in xs.items():
            got = [m.ffn_block(li, m.layers[li], x, None, None) for li in idx]
            for a, b in zip(got, want[rows]):
                assert torch.equal(a, b), f"staged != in place at rows={rows}"
    torch.cuda.synchronize()
    # with at most two tiered layers nothing overwrites a buffer, so the first copy serves every later chunk; with more,
    # every chunk (two staged row counts, two repetitions) copies every layer once
    assert st.copies == (len(idx) if len(idx) <= 2 else 4 * len(idx)), (st.copies, len(idx))
    swaps = m.rebalance_experts(max_swaps=2)                     # residency moves: the next chunk stages the new cold set
    assert swaps >= 1
    m_ref, _ = _models()
    m_ref.layers[idx[0]].bank.gu_sf = None
    x = xs[40]
    assert torch.equal(m.ffn_block(idx[0], m.layers[idx[0]], x, None, None), m_ref.ffn_block(idx[0], m_ref.layers[idx[0]], x, None, None))


def test_expert_tier_from_launch_options_rebalances_while_decoding(tmp_path):
    """expert_cache = 0.5: half of every layer's experts resident, the rest read in place from pinned memory; the tokens
    equal the untiered model's; the generator rebalances every expert_adapt_every steps; the heat file round-trips."""
    from volta_engine_b200.runtime.generator import Generator, Request
    from volta_engine_b200.runtime.options import Options
    from volta_engine_b200.server.cli import configure_expert_tier, dump_calibration

    class Tok:
        eos_ids = [0]

        def decode_bytes(self, ids, skip_special=False):
            return bytes(i & 0xFF for i in ids)

        def encode(self, text, allow_special=True):
            return list(text.encode())

    prompt = torch.randint(1, 1000, (60,), generator=torch.Generator().manual_seed(5)).tolist()
    m_ref, _ = _models(router_bias_zipf=1.2)
    want, _ = Engine(m_ref, PagedKVCache(2, m_ref.nkv, 64, 16, 1, 512, DEV), prefill_chunk=64).generate(prompt, 20)
    heat_file = str(tmp_path / "heat.pt")
    o = Options.resolve({"expert_cache": 0.5, "expert_adapt_every": 4, "expert_swaps": 2, "expert_heat_file": heat_file,
                         "max_slots": 1, "prefix_cache_mib": 0}, env={})
    m, _ = _models(router_bias_zipf=1.2)
    configure_expert_tier(m, o)
    assert m.expert_adapt_every == 4 and m.expert_max_swaps == 2 and len(m.tiers) == 2
    assert all(len(t.resident()) == m.e_local // 2 for _, t in m.tiers)
    eng = Engine(m, PagedKVCache(2, m.nkv, 64, 16, 1, 512, DEV), prefill_chunk=64)
    gen = Generator(eng, Tok(), o, eos_ids=[])
    out = gen.generate(Request(prompt, max_tokens=20, cache_prefix=False))["tokens"]
    assert out == want
    assert sum(t.swaps for _, t in m.tiers) > 0, "the skewed router should have moved experts"
    assert heat_file in dump_calibration(m, o)
    m2, _ = _models(router_bias_zipf=1.2)
    configure_expert_tier(m2, o)                       # starts from the saved counts: the hottest experts are resident
    hot = torch.load(heat_file)[0].topk(m2.e_local // 2).indices.tolist()
    assert len(set(hot) & set(m2.tiers[0][1].resident())) >= m2.e_local // 2 - 1
