"""Host-side tests (no GPU): NVFP4 codec, paged KV bookkeeping, dense model on the CPU oracle path."""
import torch

from volta_engine_b200.models.dense import DenseConfig, DenseModel
from volta_engine_b200.quant import nvfp4 as qn
from volta_engine_b200.runtime.engine import Engine
from volta_engine_b200.runtime.kv_cache import OutOfPages, PagedKVCache


def test_e2m1_ties_and_saturation():
    x = torch.tensor([0.25, 0.75, 1.25, 1.75, 2.5, 3.5, 5.0, 7.0, -0.3, 0.0, -6.5])
    want = torch.tensor([0.0, 1.0, 1.0, 2.0, 2.0, 4.0, 4.0, 6.0, -0.5, 0.0, -6.0])
    assert torch.equal(qn.e2m1_decode(qn.e2m1_encode(x)), want)


def test_nvfp4_roundtrip_and_search_improves():
    g = torch.Generator().manual_seed(0)
    w = torch.randn(128, 256, generator=g) * 0.02
    p, s, gs = qn.quantize_nvfp4(w, search=True)
    p0, s0, gs0 = qn.quantize_nvfp4(w, search=False)
    e1 = (qn.dequantize_nvfp4(p, s, gs) - w).norm() / w.norm()
    e0 = (qn.dequantize_nvfp4(p0, s0, gs0) - w).norm() / w.norm()
    assert e1 <= e0 and e1 < 0.1
    assert p.shape == (128, 128) and s.shape == (128, 16)
    # largest block scale maps near the E4M3 maximum
    assert qn.e4m3_decode(s).max() >= 224


def test_scale_layouts():
    s = torch.arange(256 * 32, dtype=torch.int32).remainder(251).to(torch.uint8).reshape(256, 32)
    a = qn.scales_atoms_512(s)
    assert a.shape == (2, 8, 512)
    r, kb = 200, 13
    assert a[r // 128, kb // 4, ((r % 128) % 32) * 16 + ((r % 128) // 32) * 4 + kb % 4] == s[r, kb]
    b = qn.scales_blocked_k128(s)
    assert b[r // 128, kb // 8, r % 128, kb % 8] == s[r, kb]


def test_paged_kv_alloc_release():
    kv = PagedKVCache(2, 2, 64, num_pages=6, max_slots=2, max_seq=512, device="cpu")
    kv.reserve(0, 130)
    assert kv.slot_pages[0] == 3 and kv.free_pages() == 2
    assert len(set(kv.host_table[0, :3].tolist())) == 3 and 0 not in kv.host_table[0, :3].tolist()
    assert not kv.can_reserve(1, 64 * 3)
    try:
        kv.reserve(1, 64 * 3)
        assert False
    except OutOfPages:
        pass
    kv.release(0, keep_tokens=64)
    assert kv.slot_pages[0] == 1 and kv.free_pages() == 4


def test_dense_cpu_prefill_equals_decode():
    cfg = DenseConfig.tiny()
    m = DenseModel(cfg, "cpu").init_random(seed=0, search=True)
    g = torch.Generator().manual_seed(0)
    prompt = torch.randint(0, cfg.vocab, (70,), generator=g).tolist()
    kv = PagedKVCache(cfg.n_layers, m.nkv, cfg.head_dim, 16, 2, 512, "cpu")
    out, st = Engine(m, kv, use_graphs=False, prefill_chunk=32).generate(prompt, 6)
    kv2 = PagedKVCache(cfg.n_layers, m.nkv, cfg.head_dim, 16, 2, 512, "cpu")
    nxt = Engine(m, kv2, use_graphs=False, prefill_chunk=1000).prefill(0, prompt + out[:4])
    assert nxt == out[4]
    assert st.new_tokens == 6


def test_native_build_present():
    from volta_engine_b200 import _build
    libs = _build.build_all()
    assert libs["kernels"].exists()


def test_sandwich_norm_windowed_model_prefill_equals_decode():
    """Gemma-style block: pre / post norms around both sub-layers, (1 + w) norm weights, alternating sliding-window and
    full-attention layers with their own rotary base, GELU gate, scaled embedding, logit soft-cap."""
    cfg = DenseConfig.tiny(n_layers=4, sandwich_norm=True, window_pattern=2, sliding_window=24, rope_theta_local=1e4,
                           norm_bias=1.0, act="gelu_tanh", embed_scale=16.0, logit_softcap=30.0, qk_norm=True)
    m = DenseModel(cfg, "cpu").init_random(seed=3, search=False)
    assert [m.layer_window(i) for i in range(4)] == [24, 0, 24, 0]
    assert m.layer_theta(0) == 1e4 and m.layer_theta(1) == cfg.rope_theta
    g = torch.Generator().manual_seed(3)
    prompt = torch.randint(0, cfg.vocab, (90,), generator=g).tolist()
    kv = PagedKVCache(cfg.n_layers, m.nkv, cfg.head_dim, 16, 2, 512, "cpu")
    out, _ = Engine(m, kv, use_graphs=False, prefill_chunk=32).generate(prompt, 5)
    kv2 = PagedKVCache(cfg.n_layers, m.nkv, cfg.head_dim, 16, 2, 512, "cpu")
    nxt = Engine(m, kv2, use_graphs=False, prefill_chunk=1000).prefill(0, prompt + out[:3])
    assert nxt == out[3]
    # the window matters: the same weights without it give a different continuation state
    cfg2 = DenseConfig.tiny(**{**cfg.to_dict(), "window_pattern": 0, "sliding_window": 0})
    m2 = DenseModel(cfg2, "cpu").init_random(seed=3, search=False)
    kv3 = PagedKVCache(cfg.n_layers, m2.nkv, cfg.head_dim, 16, 2, 512, "cpu")
    Engine(m2, kv3, use_graphs=False, prefill_chunk=1000).prefill(0, prompt)
    Engine(m, PagedKVCache(cfg.n_layers, m.nkv, cfg.head_dim, 16, 2, 512, "cpu"), use_graphs=False, prefill_chunk=1000).prefill(0, prompt)
    assert not torch.allclose(m.last_hidden[-1].float(), m2.last_hidden[-1].float(), atol=1e-3)


def test_gguf_block_decoders_match_ggml_goldens():
    """(sum, one element, max |x|) of the decoded synthetic blocks; the numbers were produced by the ggml C row
    dequantisers on the same bytes (bit-equal to this decoder for every format when they were taken)."""
    from volta_engine_b200.quant import gguf as G
    golden = {
        3: (5.891298294067383, -0.13057708740234375, 0.30628204345703125),
        6: (-0.6080513000488281, 0.2533721923828125, 0.313232421875),
        7: (44.34039878845215, 0.1629791259765625, 0.627166748046875),
        10: (132.822509765625, -0.012451171875, 0.9476165771484375),
        11: (9.363227844238281, 0.231536865234375, 1.7039794921875),
        13: (-4511.329105377197, 0.2799797058105469, 24.929656982421875),
        20: (17.381572723388672, -0.029878616333007812, 2.507598876953125),
        23: (1052.876178741455, -0.05899810791015625, 44.815093994140625),
        # the codebook formats: IQ2_XXS, IQ2_XS, IQ3_XXS, IQ1_S, IQ3_S, IQ2_S, IQ1_M
        16: (-3.6108641624450684, -0.38962554931640625, 2.257613182067871),
        17: (-5.912283897399902, 0.3155059814453125, 3.1120147705078125),
        18: (34.321876525878906, 0.09368896484375, 7.841766357421875),
        19: (-0.5756797790527344, -0.14499664306640625, 0.30487060546875),
        21: (0.289398193359375, 0.39859771728515625, 4.753875732421875),
        22: (1.9254817962646484, 0.18060302734375, 3.0135135650634766),
        29: (-2.6709327697753906, 0.05484151840209961, 0.32469749450683594),
    }
    for t, (s, e, m) in golden.items():
        y = G.dequantize(G.random_blocks(t, 2, 512, seed=100 + t), t, 512).double()
        assert abs(float(y.sum()) - s) < 1e-6 and float(y[1, 300]) == e and float(y.abs().max()) == m, G.NAMES[t]
    # the formats with a quantiser round-trip within their step size
    x = torch.randn(4, 256, generator=torch.Generator().manual_seed(0)) * 0.1
    for t, tol in ((G.GGML_Q4_1, 0.03), (G.GGML_Q5_0, 0.03), (G.GGML_Q5_1, 0.015), (G.GGML_IQ4_NL, 0.05)):
        back = G.dequantize(G.quantize(x, t), t, 256)
        assert float((back - x).abs().max()) < tol, G.NAMES[t]


def test_kv_release_prefix_recycles_pages_below_a_window():
    from volta_engine_b200.runtime.kv_cache import PagedKVCache
    kv = PagedKVCache(1, 1, 8, 9, 2, 4096, "cpu")
    kv.reserve(0, 64 * 6)
    assert kv.free_pages() == 2
    assert kv.release_prefix(0, 64 * 4 + 10) == 4 and kv.free_pages() == 6
    assert kv.host_table[0, :4].tolist() == [0, 0, 0, 0] and int(kv.host_table[0, 4]) != 0
    kv.reserve(0, 64 * 10)                                  # positions keep growing over the same eight physical pages
    assert kv.free_pages() == 2 and kv.release_prefix(0, 64 * 4) == 0
    kv.release(0)
    assert kv.free_pages() == 8 and kv.slot_first[0] == 0 and kv.slot_pages[0] == 0


def test_expert_tier_policy_swaps_the_hottest_cold_expert_in():
    from types import SimpleNamespace
    from volta_engine_b200.runtime.expert_tier import ExpertTier
    E = 6
    bank = SimpleNamespace(e_local=E, gu_p=torch.arange(E * 4, dtype=torch.uint8).reshape(E, 2, 2),
                           gu_s=torch.zeros(E, 2, 1, dtype=torch.uint8), dn_p=torch.ones(E, 2, 2, dtype=torch.uint8),
                           dn_s=torch.zeros(E, 2, 1, dtype=torch.uint8), gu_sf=None, dn_sf=None)
    t = ExpertTier(bank, 2, decay=0.5, margin=1.25)
    assert t.resident() == [0, 1] and bank.gu_p is None
    assert int(t.tab_gu[0]) == t.slots["gu_p"][0].data_ptr() and int(t.tab_gu[2 * 4]) == t.cold["gu_p"][4].data_ptr()
    counts = torch.tensor([5.0, 1.0, 0.0, 9.0, 0.0, 4.0])
    assert t.rebalance(counts, max_swaps=1) == 1 and t.resident() == [0, 3]              # 3 replaces the coldest hot expert
    assert torch.equal(t.slots["gu_p"][t.slot_of[3]], t.cold["gu_p"][3])
    assert int(t.tab_gu[2 * 1]) == t.cold["gu_p"][1].data_ptr()                          # the evicted expert reads from the host copy
    assert t.rebalance(counts, max_swaps=4) == 0                                           # no new routing: heat only decays
    counts2 = counts + torch.tensor([0.0, 0.0, 30.0, 0.0, 0.0, 0.0])
    assert t.rebalance(counts2, max_swaps=4) == 1 and 2 in t.resident() and t.swaps == 2


def test_expert_stager_copies_cold_experts_into_alternating_scratch_buffers():
    """Staging a layer ahead: the scratch holds the layer's cold experts in ascending order, the staged tables point hot
    experts at their slots and cold ones into the scratch, consecutive layers alternate buffers, a changed residency is
    staged again."""
    from types import SimpleNamespace
    from volta_engine_b200.runtime.expert_tier import ExpertStager, ExpertTier
    E = 6

    def tier(seed):
        g = torch.Generator().manual_seed(seed)
        r = lambda *s: torch.randint(0, 255, s, generator=g, dtype=torch.uint8)
        bank = SimpleNamespace(e_local=E, gu_p=r(E, 4, 2), gu_s=r(E, 4, 1), dn_p=r(E, 2, 4), dn_s=r(E, 2, 1), gu_sf=None, dn_sf=None)
        return ExpertTier(bank, 2, decay=0.5, margin=1.0)
    tiers = [(3, tier(1)), (4, tier(2)), (7, tier(3))]
    st = ExpertStager(tiers)
    assert st.n_cold == 4 and ExpertStager.scratch_bytes(tiers) == 2 * 4 * (8 + 4 + 8 + 2)
    assert st.wants(tiers[0][1], 17) and not st.wants(tiers[0][1], 16)
    t0, t1, t2 = (t for _, t in tiers)
    gu, dn = st.acquire(t0)
    assert st.staged == [(0, 0), (1, 0)] and st.copies == 2              # this layer and the next one
    for j, e in enumerate([2, 3, 4, 5]):
        assert torch.equal(st.buf[0]["gu_p"][j], t0.cold["gu_p"][e]) and torch.equal(st.buf[1]["dn_s"][j], t1.cold["dn_s"][e])
        assert int(gu[2 * e]) == st.buf[0]["gu_p"][j].data_ptr() and int(dn[2 * e + 1]) == st.buf[0]["dn_s"][j].data_ptr()
    assert int(gu[0]) == t0.slots["gu_p"][0].data_ptr() and int(gu[3]) == t0.slots["gu_s"][1].data_ptr()
    st.release(t0)
    st.acquire(t1)
    assert st.staged == [(2, 0), (1, 0)] and st.copies == 3              # layer 2 went into the buffer layer 0 released
    st.release(t1)
    st.acquire(t2)
    st.release(t2)
    assert st.copies == 3
    # residency of layer 0 changes: expert 4 in, expert 1 out -> cold set 1 2 3 5, staged again with new tables
    assert t0.rebalance(torch.tensor([5.0, 0.0, 0.0, 0.0, 9.0, 0.0]), max_swaps=1) == 1 and t0.resident() == [0, 4]
    gu2, _ = st.acquire(t0)
    assert st.copies == 4 and st.staged[0] == (0, 1)                     # layer 1 was still staged
    for j, e in enumerate([1, 2, 3, 5]):
        assert torch.equal(st.buf[0]["gu_p"][j], t0.cold["gu_p"][e]) and int(gu2[2 * e]) == st.buf[0]["gu_p"][j].data_ptr()
    assert int(gu2[2 * 4]) == t0.slots["gu_p"][t0.slot_of[4]].data_ptr()


def test_sentencepiece_style_tokenizer(tmp_path):
    import json
    from volta_engine_b200.loader.tokenizer import Tokenizer
    sp = "▁"
    pieces = ["<unk>", "<bos>", "<eos>"] + [f"<0x{b:02X}>" for b in range(256)] + \
        [sp, "h", "e", "l", "o", "w", "r", "d", "he", "ll", "hell", "hello", sp + "w", "or", sp + "wor", "ld", sp + "world", sp + sp, "é"]
    vocab = {p: i for i, p in enumerate(pieces)}
    merges = [["h", "e"], ["l", "l"], ["he", "ll"], ["hell", "o"], [sp, "w"], ["o", "r"], [sp + "w", "or"], ["l", "d"],
              [sp + "wor", "ld"], [sp, sp]]
    tj = {"model": {"type": "BPE", "byte_fallback": True, "vocab": vocab, "merges": merges},
          "added_tokens": [{"id": 1, "content": "<bos>"}, {"id": 2, "content": "<eos>"}]}
    (tmp_path / "tokenizer.json").write_text(json.dumps(tj))
    (tmp_path / "config.json").write_text(json.dumps({"model_type": "gemma3"}))
    t = Tokenizer.load(str(tmp_path))
    assert t.mode == "spm"
    ids = t.encode("hello world")
    assert ids == [vocab["hello"], vocab[sp + "world"]]
    assert t.decode(ids) == "hello world"
    ids = t.encode("<bos>hello  wé中")
    # the lower-ranked merge (space + w) wins over the later (space + space) one
    want = [1, vocab["hello"], vocab[sp], vocab[sp + "w"], vocab["é"]] + [vocab[f"<0x{b:02X}>"] for b in "中".encode()]
    assert ids == want and t.decode(ids, skip_special=True) == "hello  wé中"
    long = ("hello world " * 3000).strip()                     # whole-text merging stays fast on long inputs
    assert len(t.encode(long)) == 8999 and t.decode(t.encode(long)) == long


def test_cpu_expert_service_handles_a_mailbox_request():
    import numpy as np
    from volta_engine_b200.runtime.cpu_experts import CpuExpertService, HostExpert
    g = torch.Generator().manual_seed(0)
    H, I = 32, 16
    svc = CpuExpertService()
    mb = svc.mailbox(H, "cpu")
    e5 = HostExpert(torch.randn(2 * I, H, generator=g) * 0.2, torch.randn(H, I, generator=g) * 0.2)
    e7 = HostExpert(torch.randn(2 * I, H, generator=g) * 0.2, torch.randn(H, I, generator=g) * 0.2)
    svc.add_expert(3, 5, e5)
    svc.add_expert(3, 7, e7)
    x = torch.randn(2, H, generator=g).to(torch.bfloat16)
    mb.x[:2] = x
    mb.hdr[2:6] = [3, 2, 3, H]
    for r, (row, e, w) in enumerate([(0, 5, 0.25), (1, 7, 0.5), (1, 5, 0.125)]):
        mb.routes[r, 0], mb.routes[r, 1] = row, e
        mb.route_w[r, 2] = w
    svc.start()
    try:
        mb.hdr[0] = 1                                        # what the post kernel publishes last
        for _ in range(200):
            if int(mb.hdr[1]) == 1:
                break
            import time
            time.sleep(0.01)
        assert int(mb.hdr[1]) == 1 and svc.served == 1
    finally:
        svc.stop()
    xf = x.float()
    want0 = 0.25 * e5.forward(xf[0:1])[0]
    want1 = 0.5 * e7.forward(xf[1:2])[0] + 0.125 * e5.forward(xf[1:2])[0]
    assert np.allclose(mb.out[0], want0.numpy(), atol=1e-6) and np.allclose(mb.out[1], want1.numpy(), atol=1e-6)


def test_native_host_nvfp4_kernels_match_the_torch_statement():
    """csrc/host/cpu_experts.cpp: the packed NVFP4 mat-vec against the dequantised matrix, one expert against the fp32
    host expert (same rounding points), with and without the pinned worker pool."""
    import ctypes
    from volta_engine_b200._lib import hcall
    from volta_engine_b200.quant import nvfp4 as qn
    from volta_engine_b200.runtime.cpu_experts import HostExpert, HostExpertNVFP4, numa_node_cpus, parse_cpu_list
    g = torch.Generator().manual_seed(2)
    H, I = 256, 128
    wgu, wdn = torch.randn(2 * I, H, generator=g) * 0.05, torch.randn(H, I, generator=g) * 0.05
    (gp, gs, gg), (dp, ds, dg) = qn.quantize_nvfp4(wgu, search=False), qn.quantize_nvfp4(wdn, search=False)
    x = torch.randn(3, H, generator=g)
    want = x @ qn.dequantize_nvfp4(gp, gs, gg).t()
    y = torch.empty(2 * I)
    for pool_threads in (0, 3):
        pool = hcall("cpu_pool_create", "ipii", pool_threads, 0, 0, 50, restype=ctypes.c_void_p) if pool_threads else None
        try:
            for r in range(3):
                assert hcall("cpu_nvfp4_gemv", "pppfppii", pool, gp.data_ptr(), gs.data_ptr(), float(gg), x[r].contiguous().data_ptr(),
                             y.data_ptr(), 2 * I, H) == 0
                assert torch.allclose(y, want[r], atol=1e-4, rtol=1e-4), pool_threads
            ref_e = HostExpert(qn.dequantize_nvfp4(gp, gs, gg), qn.dequantize_nvfp4(dp, ds, dg), 0, 0.0)
            nat = HostExpertNVFP4(gp, gs, gg, dp, ds, dg, 0, 0.0)
            out = torch.zeros(3, H)
            for r in range(3):
                nat.add_to(pool, x[r].contiguous(), out[r], 0.5)
            exp = 0.5 * ref_e.forward(x)
            # (an fp32 sum in another order can move a value across a bf16 rounding boundary: one bf16 step of slack)
            assert torch.allclose(out, exp, atol=2e-3, rtol=2e-2) and float((out - exp).abs().mean()) < 2e-4
        finally:
            if pool:
                hcall("cpu_pool_destroy", "p", pool, restype=None)
    assert hcall("cpu_nvfp4_gemv", "pppfppii", None, gp.data_ptr(), gs.data_ptr(), 1.0, x.data_ptr(), y.data_ptr(), 4, 24) == 1
    assert parse_cpu_list("0-3,8,10-11") == [0, 1, 2, 3, 8, 10, 11] and parse_cpu_list("") == [] and numa_node_cpus(9999) == []
    assert hcall("cpu_has_avx2", "") in (0, 1)


def test_cpu_expert_service_serves_native_experts_through_the_mailbox():
    import numpy as np
    from volta_engine_b200.quant import nvfp4 as qn
    from volta_engine_b200.runtime.cpu_experts import CpuExpertService, HostExpert, HostExpertNVFP4
    g = torch.Generator().manual_seed(4)
    H, I = 128, 64
    svc = CpuExpertService(threads=2, spin_us=50, cpus=[0])
    refs = {}
    for e in range(3):
        (gp, gs, gg), (dp, ds, dg) = (qn.quantize_nvfp4(torch.randn(2 * I, H, generator=g) * 0.05, search=False),
                                      qn.quantize_nvfp4(torch.randn(H, I, generator=g) * 0.05, search=False))
        svc.add_expert(0, e, HostExpertNVFP4(gp, gs, gg, dp, ds, dg))
        refs[e] = HostExpert(qn.dequantize_nvfp4(gp, gs, gg), qn.dequantize_nvfp4(dp, ds, dg))
    mb = svc.mailbox(H, "cpu")
    svc.start()
    try:
        assert svc.pool is not None
        x = torch.randn(2, H, generator=g).to(torch.bfloat16)
        mb.x[:2] = x
        routes = [(0, 1, 0.7), (0, 2, 0.3), (1, 0, 1.0)]
        for i, (row, e, w) in enumerate(routes):
            mb.routes[i, 0], mb.routes[i, 1] = row, e
            mb.route_w[i, 2] = w
        mb.hdr[2:6] = [0, 2, len(routes), H]
        mb.hdr[0] = 1
        import time
        t0 = time.time()
        while int(mb.hdr[1]) != 1 and time.time() - t0 < 20:
            time.sleep(0.005)
        assert int(mb.hdr[1]) == 1
        want = np.zeros((2, H), dtype=np.float32)
        for row, e, w in routes:
            want[row] += w * refs[e].forward(x[row:row + 1].float())[0].numpy()
        assert np.allclose(mb.out[:2], want, atol=2e-3, rtol=2e-2)
    finally:
        svc.stop()
    assert svc.pool is None


def test_expert_tier_history_share_and_resident_route_bias():
    from volta_engine_b200.models.moe import MoEConfig, MoEModel
    cfg = MoEConfig.tiny() if hasattr(MoEConfig, "tiny") else None
    if cfg is None:
        pytest.skip("no tiny MoE configuration")
    m = MoEModel(cfg, "cpu").init_random(seed=1)
    tiers = m.enable_expert_tier(2, decay=0.5, margin=1.0, margin_add=0.0, history_pct=75, resident_bias=0.25)
    li, tier = tiers[0]
    L = m.layers[li]
    E = tier.E
    assert tier.resident() == [0, 1] and tier.history_pct == 75
    # the router's selection bias carries the value on the resident experts only, and follows a swap
    assert L.router_bias[m.e0:m.e0 + E].tolist() == [0.25, 0.25] + [0.0] * (E - 2)
    counts = torch.zeros(E)
    counts[E - 1] = 50.0                                   # one window in which the last expert is hot
    assert tier.rebalance(counts, max_swaps=1) == 1 and (E - 1) in tier.resident()
    bias = L.router_bias[m.e0:m.e0 + E].tolist()
    assert bias[E - 1] == 0.25 and sum(1 for b in bias if b == 0.25) == 2
    # long-run counts pull the decision: expert 2 has a long history, the last window favours expert 3 only slightly
    def scenario(pct):
        m2 = MoEModel(cfg, "cpu").init_random(seed=1)
        t = m2.enable_expert_tier(1, decay=0.0, margin=1.0, history_pct=pct)[0][1]
        hist = torch.zeros(t.E)
        hist[2] = 10000.0
        t.rebalance(hist.clone(), max_swaps=0)             # what earlier runs left (a heat file)
        win = hist.clone()
        win[3] += 30.0
        win[2] += 20.0
        t.rebalance(win, max_swaps=1)
        return t.resident()
    assert scenario(0) == [3]                              # windows only: the window's leader comes in
    assert scenario(75) == [2]                             # with the long-run share the expert with the history wins
