"""Block drafter speculation: tap ring contents, drafting rounds that leave greedy output unchanged, the candidate walk,
the dynamic convolution and the sparse draft head (CPU statements; the CUDA kernels against them on a GPU)."""
import pytest
import torch

from volta_engine_b200.models.dense import DenseConfig, DenseModel
from volta_engine_b200.ops.linear import LinearBF16
from volta_engine_b200.runtime import dflash_runner as D
from volta_engine_b200.runtime.engine import Engine
from volta_engine_b200.runtime.generator import Generator, Request
from volta_engine_b200.runtime.kv_cache import PagedKVCache
from volta_engine_b200.runtime.options import Options


class ByteTok:
    eos_ids = [0]

    def decode_bytes(self, ids, skip_special=False):
        return bytes(i & 0xFF for i in ids)

    def encode(self, text, allow_special=True):
        return list(text.encode())


def _setup(device="cpu", block=4, use_graphs=False):
    cfg = DenseConfig.tiny(vocab=256)
    m = DenseModel(cfg, device).init_random(seed=0)
    kv = PagedKVCache(cfg.n_layers, m.nkv, cfg.head_dim, 40, 2, 512, device)
    eng = Engine(m, kv, use_graphs=use_graphs, prefill_chunk=32)
    dc = D.DFlashConfig(block_size=block, n_layers=2, hidden=cfg.hidden, n_q=cfg.n_q, n_kv=cfg.n_kv, head_dim=cfg.head_dim,
                        ffn=cfg.ffn, target_layer_ids=(0, cfg.n_layers - 1), sliding_window=64, rope_theta=1e4, mask_token_id=255,
                        tap_cap=64, quant="bf16")
    return cfg, m, eng, dc


def _prompt(n, seed=0):
    return torch.randint(1, 255, (n,), generator=torch.Generator().manual_seed(seed)).tolist()


def test_drafter_rounds_leave_greedy_output_unchanged_and_taps_follow_the_target():
    cfg, m, eng, dc = _setup()
    p = _prompt(45, 5)
    o = Options.resolve({"max_slots": 2, "prefix_interval": 0}, env={})
    plain = Generator(eng, ByteTok(), o, eos_ids=[]).generate(Request(p, max_tokens=12, cache_prefix=False))
    cfg2, m2, eng2, _ = _setup()
    o2 = Options.resolve({"max_slots": 2, "prefix_interval": 0, "speculator": "draft", "spec_ctrl": False, "spec_depth": 3}, env={})
    g = Generator(eng2, ByteTok(), o2, eos_ids=[])
    g.drafter = D.DFlashRunner(eng2, dc)
    spec = g.generate(Request(p, max_tokens=12, cache_prefix=False))
    assert spec["tokens"] == plain["tokens"]
    assert g.metrics.spec["rounds"] > 0 and g.metrics.spec["proposed"] == 3 * g.metrics.spec["rounds"]
    # the ring holds the tapped layers' outputs of the prompt positions: replay the prompt on a fresh model and compare
    cfg3, m3, eng3, _ = _setup()
    ring = D.TapRing(2, 64, (0, cfg.n_layers - 1), cfg.hidden, "cpu")
    m3.tap_ring = ring
    eng3.prefill(0, p)
    assert torch.equal(ring.rows(0, 0, len(p)), g.drafter.ring.rows(0, 0, len(p)))
    last = m3.last_residual[-1].to(torch.bfloat16)                       # last layer's output of the last prompt row
    H = cfg.hidden
    assert torch.equal(ring.taps[0, (len(p) - 1) % 64, H:2 * H], last)


def test_ingest_window_and_release():
    cfg, m, eng, dc = _setup()
    r = D.DFlashRunner(eng, dc)
    p = _prompt(100, 6)
    eng.prefill(0, p)
    assert r.ingest(0, 100) == 64 and r.ctx_len[0] == 100                # only the ring's span is still available
    assert r.ingest(0, 100) == 0
    d = r.draft(0, 7, 100)
    assert len(d) == dc.block_size - 1 and all(0 <= t < 256 for t in d)
    assert len(r.draft(0, 7, 100, depth=2)) == 2
    r.release(0)
    assert r.ctx_len[0] == 0 and r.kv.slot_pages[0] == 0


def _v2_config(dc):
    import dataclasses
    return dataclasses.replace(dc, version=2, conv_group_size=16, selector_rank=32, selector_top_k=8)


def test_version2_drafter_rounds_leave_greedy_output_unchanged():
    """The version-2 drafter (dynamic convolutions around every sub-layer, candidate walk) proposes other tokens than
    version 1 but the verified output is the target's greedy output all the same."""
    cfg, m, eng, dc = _setup()
    p = _prompt(45, 5)
    o = Options.resolve({"max_slots": 2, "prefix_interval": 0}, env={})
    plain = Generator(eng, ByteTok(), o, eos_ids=[]).generate(Request(p, max_tokens=12, cache_prefix=False))
    cfg2, m2, eng2, _ = _setup()
    o2 = Options.resolve({"max_slots": 2, "prefix_interval": 0, "speculator": "draft", "spec_ctrl": False, "spec_depth": 3}, env={})
    g = Generator(eng2, ByteTok(), o2, eos_ids=[])
    g.drafter = D.DFlashRunner(eng2, _v2_config(dc))
    spec = g.generate(Request(p, max_tokens=12, cache_prefix=False))
    assert spec["tokens"] == plain["tokens"] and g.metrics.spec["rounds"] > 0
    assert g.drafter.last_conf is not None and g.drafter.last_conf.numel() == dc.block_size - 1


def test_version2_with_identity_convolutions_and_no_pairwise_term_is_version1():
    """Static kernels = identity on tap 0, dynamic coefficients zero, pairwise codebooks zero: the version-2 stream is the
    version-1 stream (up to the fp32 residual) and the walk picks every row's best candidate, the version-1 argmax."""
    cfg, m, eng, dc = _setup()
    p = _prompt(60, 7)
    r1 = D.DFlashRunner(eng, dc, seed=11)
    eng.prefill(0, p)                                      # the runner's ring is attached: the prompt's taps land in it
    assert float(r1.ring.rows(0, 0, len(p)).abs().sum()) > 0
    want = r1.draft(0, 9, len(p))
    cfg_b, m_b, eng_b, _ = _setup()                        # the same target again (same seed) for the second drafter
    r2 = D.DFlashRunner(eng_b, _v2_config(dc), seed=11)
    eng_b.prefill(0, p)
    r2.model.layers = r1.model.layers
    r2.model.final_norm, r2.fc, r2.hidden_norm = r1.model.final_norm, r1.fc, r1.hidden_norm
    taps = dc.conv_kernel_size
    for V in r2.v2["layers"]:
        for k in ("attn", "mlp"):
            V[k + "_proj"].weight.zero_()
            V[k + "_base"].zero_()
            V[k + "_base"][0] = 1.0
            V[k + "_base"][taps] = 1.0
    r2.v2["pred"].zero_()
    got = r2.draft(0, 9, len(p))
    assert got == want, (got, want)
    assert float(r2.last_conf.min()) > 0 and float(r2.last_conf.max()) <= 1


def _walk_inputs(dev="cpu"):
    g = torch.Generator().manual_seed(3)
    bsz, rows, k, rank, vocab = 2, 5, 6, 32, 100
    unary = torch.randn(bsz, rows, k, generator=g)
    cands = torch.randint(0, vocab, (bsz, rows, k), generator=g, dtype=torch.int32)
    gate = torch.randn(bsz, rows, rank, generator=g).to(torch.bfloat16)
    pred = torch.randn(vocab, rank, generator=g).to(torch.bfloat16)
    succ = torch.randn(vocab, rank, generator=g).to(torch.bfloat16)
    anchor = torch.tensor([3, 77], dtype=torch.int32)
    return [t.to(dev) for t in (unary, cands, gate, pred, succ, anchor)]


def test_candidate_walk_without_pairwise_term_picks_the_best_unary():
    cfg, m, eng, dc = _setup()
    r = D.DFlashRunner(eng, dc)
    unary, cands, gate, pred, succ, anchor = _walk_inputs()
    out, conf = r.walk_candidates(unary, cands, torch.zeros_like(gate), pred, succ, anchor)
    want = cands.gather(2, unary.argmax(-1, keepdim=True)).squeeze(-1)
    assert torch.equal(out[:, 1:], want) and torch.equal(out[:, 0], anchor)
    assert torch.all((conf > 0) & (conf <= 1))


def test_dynconv_and_sparse_head_cpu():
    g = torch.Generator().manual_seed(4)
    T, C, gs, taps = 6, 32, 8, 2
    x = torch.randn(T, C, generator=g)
    dyn = torch.randn(T, taps, C // gs, generator=g).to(torch.bfloat16)
    base = torch.randn(taps, C, generator=g).to(torch.bfloat16)
    out = D.dynconv(x, dyn, base, gs)
    t, c = 3, 17
    want = sum((float(base[k, c]) + float(dyn[t, k, c // gs])) * float(x[t - k, c]) for k in range(taps))
    assert abs(float(out[t, c]) - want) < 1e-5
    assert abs(float(out[0, c]) - (float(base[0, c]) + float(dyn[0, 0, c // gs])) * float(x[0, c])) < 1e-5
    W = (torch.randn(300, 64, generator=g) * 0.1).to(torch.bfloat16)
    cols = torch.tensor(D.SparseHead.choose_columns({5: 10, 9: 7, 200: 7, 3: 1}, 3, always=[299]), dtype=torch.int32)
    assert cols.tolist() == [5, 9, 299]
    sh = D.SparseHead.extract(LinearBF16(W), 64, 300, cols, ident_rows=48)
    assert torch.equal(sh.w_sub, W[cols.long()])
    xq = torch.randn(2, 64, generator=g).to(torch.bfloat16)
    lg = sh.logits(xq)
    assert lg.shape == (2, 300) and int(lg[0].float().argmax()) in cols.tolist()
    assert torch.allclose(lg[:, cols.long()].float(), (xq.float() @ W[cols.long()].float().t()), atol=0.02, rtol=0.02)


# ------------------------------------------------------------------------------------------------ GPU
@pytest.mark.gpu
def test_spec_kernels_match_cpu():
    dev = torch.device("cuda:0")
    cfg, m, eng, dc = _setup()
    r = D.DFlashRunner(eng, dc)
    ins = _walk_inputs()
    want, wconf = r.walk_candidates(*ins)
    got, gconf = r.walk_candidates(*[t.to(dev) for t in ins])
    assert torch.equal(got.cpu(), want) and torch.allclose(gconf.cpu(), wconf, atol=1e-3)
    g = torch.Generator().manual_seed(8)
    T, C, gs, taps = 8, 5120, 16, 2
    x = torch.randn(T, C, generator=g)
    dyn = torch.randn(T, taps, C // gs, generator=g).to(torch.bfloat16)
    base = torch.randn(taps, C, generator=g).to(torch.bfloat16)
    acc0 = torch.randn(T, C, generator=g)
    assert torch.allclose(D.dynconv(x.to(dev), dyn.to(dev), base.to(dev), gs).cpu(), D.dynconv(x, dyn, base, gs), atol=1e-5)
    a, b = acc0.clone(), acc0.to(dev)
    D.dynconv(x, dyn, base, gs, out=a, accumulate=True)
    D.dynconv(x.to(dev), dyn.to(dev), base.to(dev), gs, out=b, accumulate=True)
    assert torch.allclose(b.cpu(), a, atol=1e-5)
    xs = torch.randn(3, 4, 640, generator=g)
    for mode in (0, 1, 4):
        assert torch.equal(D.reduce_streams(xs.to(dev), mode).cpu(), D.reduce_streams(xs, mode))
    # tap ring: bf16 and fp32 sources, rows of idle slots skipped
    ring = D.TapRing(2, 16, (3, 7), 640, dev)
    h = torch.randn(4, 640, generator=g)
    pos = torch.tensor([5, 21, 2, 9], dtype=torch.int32, device=dev)
    slot = torch.tensor([0, 1, -1, 1], dtype=torch.int32, device=dev)
    ring.publish(7, h.to(dev), pos, slot, 4)
    ring.publish(3, h.to(dev).to(torch.bfloat16), pos, slot, 4)
    ring.publish(5, h.to(dev), pos, slot, 4)                              # not a tapped layer: ignored
    t = ring.taps.cpu()
    hb = h.to(torch.bfloat16)
    assert torch.equal(t[0, 5, 640:], hb[0]) and torch.equal(t[1, 21 % 16, :640], hb[1]) and torch.equal(t[1, 9, 640:], hb[3])
    assert float(t[0, 2].abs().sum()) == 0 and float(t[1, 2].abs().sum()) == 0
    # sparse head on the device
    W = (torch.randn(1024, 256, generator=g) * 0.1).to(torch.bfloat16)
    cols = torch.tensor([1, 17, 500, 1023], dtype=torch.int32)
    sh = D.SparseHead.extract(LinearBF16(W.to(dev)), 256, 1024, cols.to(dev), ident_rows=100)
    assert torch.equal(sh.w_sub.cpu(), W[cols.long()])
    xq = torch.randn(3, 256, generator=g).to(torch.bfloat16)
    lg = sh.logits(xq.to(dev)).cpu()
    ref = D.SparseHead(cols, W[cols.long()], 1024).logits(xq)
    assert torch.allclose(lg.float()[:, cols.long()], ref.float()[:, cols.long()], atol=0.03, rtol=0.02)
    assert torch.equal(lg.float().argmax(-1), ref.float().argmax(-1))


@pytest.mark.gpu
def test_drafter_rounds_on_gpu_equal_plain_greedy():
    dev = torch.device("cuda:0")
    p = _prompt(45, 5)
    cfg, m, eng, dc = _setup(dev)
    o = Options.resolve({"max_slots": 2, "prefix_interval": 0}, env={})
    plain = Generator(eng, ByteTok(), o, eos_ids=[]).generate(Request(p, max_tokens=16, cache_prefix=False))
    cfg2, m2, eng2, _ = _setup(dev)
    o2 = Options.resolve({"max_slots": 2, "prefix_interval": 0, "speculator": "draft", "spec_ctrl": False, "spec_depth": 3}, env={})
    g = Generator(eng2, ByteTok(), o2, eos_ids=[])
    g.drafter = D.DFlashRunner(eng2, dc)
    spec = g.generate(Request(p, max_tokens=16, cache_prefix=False))
    assert spec["tokens"] == plain["tokens"] and g.metrics.spec["rounds"] > 0


@pytest.mark.gpu
def test_version2_drafter_on_gpu_matches_cpu_statement_and_plain_greedy():
    dev = torch.device("cuda:0")
    p = _prompt(45, 5)
    cfg, m, eng, dc = _setup(dev)
    o = Options.resolve({"max_slots": 2, "prefix_interval": 0}, env={})
    plain = Generator(eng, ByteTok(), o, eos_ids=[]).generate(Request(p, max_tokens=16, cache_prefix=False))
    cfg2, m2, eng2, _ = _setup(dev)
    o2 = Options.resolve({"max_slots": 2, "prefix_interval": 0, "speculator": "draft", "spec_ctrl": False, "spec_depth": 3}, env={})
    g = Generator(eng2, ByteTok(), o2, eos_ids=[])
    g.drafter = D.DFlashRunner(eng2, _v2_config(dc))
    spec = g.generate(Request(p, max_tokens=16, cache_prefix=False))
    assert spec["tokens"] == plain["tokens"] and g.metrics.spec["rounds"] > 0
    # the block's hidden rows on the device against the CPU statement of the same weights
    from volta_engine_b200.models.util import to_device
    from volta_engine_b200.runtime.batch import BatchRows, LOGITS_ALL
    cfg3, m3, eng3, _ = _setup(dev)
    r = D.DFlashRunner(eng3, _v2_config(dc))
    eng3.prefill(0, p)
    r.ingest(0, len(p))
    r._reserve(0, len(p) + dc.block_size + 1)
    B = dc.block_size
    b = BatchRows.make([9] + [dc.mask_token_id] * (B - 1), [len(p) + i for i in range(B)], [0] * B, dev, LOGITS_ALL, 1, nsplit=1)
    b.key_end = torch.full((B,), len(p) + B - 1, dtype=torch.int32, device=dev)
    h_gpu = r._forward_v2(b).float().cpu()
    mc = to_device(m3, "cpu")                         # the same target weights on the CPU
    engc = Engine(mc, PagedKVCache(cfg3.n_layers, mc.nkv, cfg3.head_dim, 40, 2, 512, "cpu"), use_graphs=False, prefill_chunk=32)
    rc = D.DFlashRunner(engc, _v2_config(dc))
    engc.prefill(0, p)
    rc.model.layers = to_device(r.model, "cpu").layers
    rc.fc = LinearBF16(r.fc.weight.cpu())
    rc.hidden_norm, rc.model.final_norm = r.hidden_norm.cpu(), r.model.final_norm.cpu()
    rc.v2 = {"layers": [{k: (LinearBF16(v.weight.cpu()) if isinstance(v, LinearBF16) else v.cpu()) for k, v in V.items()} for V in r.v2["layers"]],
             "gate": LinearBF16(r.v2["gate"].weight.cpu()), "pred": r.v2["pred"].cpu(), "succ": r.v2["succ"].cpu()}
    rc.ingest(0, len(p))
    rc._reserve(0, len(p) + B + 1)
    bc = BatchRows.make([9] + [dc.mask_token_id] * (B - 1), [len(p) + i for i in range(B)], [0] * B, "cpu", LOGITS_ALL, 1, nsplit=1)
    bc.key_end = torch.full((B,), len(p) + B - 1, dtype=torch.int32)
    h_cpu = rc._forward_v2(bc).float()
    cos = torch.nn.functional.cosine_similarity(h_gpu.flatten(), h_cpu.flatten(), dim=0)
    assert cos > 0.995, float(cos)


def test_sparse_head_policy_subset_hysteresis_and_persistence(tmp_path):
    from volta_engine_b200.runtime.sparse_head_policy import SparseHeadParams, SparseHeadPolicy
    p = SparseHeadPolicy(1000, SparseHeadParams(capacity=8, interval=16, decay_tokens=64, min_evidence=10.0, min_change=0.25,
                                                full_probe_rounds=5))
    assert not p.rebuild_due() and not p.use_sparse()
    p.observe_prompt([1, 2, 3, 1, 2000, -1])                   # out-of-range ids are ignored, prompt tokens weigh 0.2
    assert abs(float(p.counts[1]) - 0.4) < 1e-6 and abs(p.evidence - 1.2) < 1e-6
    for t in [5] * 6 + [6] * 4 + [7] * 3 + list(range(20, 30)):
        p.observe_generated(t)
    assert p.rebuild_due()
    first = p.ranked()
    assert first[:3] == [5, 6, 7] and len(first) == 8 and first[3:] == [20, 21, 22, 23, 24]     # ties to the lower id
    p.set_subset(first)
    assert p.built and p.subset_n == 8
    # an incumbent keeps its place until a challenger beats its count by the margin
    p.observe_generated(25)                                     # 25: 2.0, incumbent 24: 1.0 -> replaced (2.0 > 1.25)
    assert 25 in p.ranked() and 24 not in p.ranked()
    for t in (26, 24):                                          # 26: 2.0 against incumbents 23 / 24 ...
        p.observe_generated(t)
    assert 24 in p.ranked()                                     # 24: 2.0 * 1.25 stays ahead of the challengers at 2.0
    # miss rate: plain mean at first (3 tokens scored: 25 miss, 26 miss, 24 hit)
    assert abs(p.miss - 2 / 3) < 1e-9 and p.scored == 3
    # use: needs timings and MIN_SCORED tokens; below the break-even miss rate the sparse head is on, with hysteresis
    for _ in range(70):
        p.observe_generated(5)
    assert not p.use_sparse()                                   # no full-head timing yet
    p.draft_step_time(False, 2.0)
    assert p.use_sparse() and p.on                              # measures the sparse steps once
    p.draft_step_time(True, 0.5)
    p.round_time(10.0, 4)
    assert abs(p.breakeven() - 2 * 1.5 * 4 / 10.0) < 1e-9
    p.miss = 0.5
    assert p.use_sparse()
    p.miss = 1.5                                                # above 1.2 x break-even (1.44): off
    assert not p.use_sparse() and not p.on
    p.miss = 1.0                                                # between 0.8x and 1.2x: stays off
    assert not p.use_sparse()
    p.miss = 0.9
    assert p.use_sparse()
    seen = [p.use_sparse() for _ in range(6)]                   # every fifth sparse round is a full probe, the mode stays on
    assert seen.count(False) == 1 and p.on
    # rebuild again only after the interval and when enough of the subset would change
    p.since_rebuild = 0
    assert not p.rebuild_due()
    for t in range(100, 116):
        for _ in range(4):
            p.observe_generated(t)
    assert p.rebuild_due()
    # decay halves the counts
    c5 = float(p.counts[5])
    p.since_decay = p.p.decay_tokens - 1
    p.observe_generated(999)
    assert abs(float(p.counts[5]) - c5 / 2) < 1e-4
    # persistence: counts survive, another vocabulary is refused
    path = tmp_path / "sparse.bin"
    assert p.save(path)
    q = SparseHeadPolicy(1000)
    assert q.load(path) and abs(q.evidence - p.evidence) < 1e-9 and (q.counts == p.counts).all()
    assert not SparseHeadPolicy(999).load(path) and not q.load(tmp_path / "absent.bin")


def test_candidate_log_and_target_spool_round_trip(tmp_path):
    from volta_engine_b200.runtime.spec_logs import CandLog, TargetSpool, read_cand_log
    log = CandLog()
    log.round(0, 1, 2, 3, [])                                    # closed: nothing happens
    assert not log.on() and log.open(tmp_path / "cand.bin") and log.on()
    log.round(1, 40, 7, 7, [(11, 11, [0.5, 0.25], [11, 12]), (13, 14, list(range(20)), list(range(100, 120)))])
    log.request(1, [1, 2, 3, 11, 14])
    log.flush()
    log.close()
    recs = read_cand_log(tmp_path / "cand.bin")
    assert [r["kind"] for r in recs] == ["round", "request"] and recs[1]["tokens"] == [1, 2, 3, 11, 14]
    r0 = recs[0]
    assert (r0["slot"], r0["pos"], r0["anchor"], r0["active"]) == (1, 40, 7, 7) and len(r0["rows"]) == 2
    assert r0["rows"][0]["ids"][:3] == [11, 12, -1] and r0["rows"][0]["vals"][1] == 0.25 and r0["rows"][0]["vals"][2] == float("-inf")
    assert r0["rows"][1]["ids"] == list(range(100, 116)) and (r0["rows"][1]["chosen"], r0["rows"][1]["target"]) == (13, 14)
    sp = TargetSpool()
    sp.add(0, 5, [1.0], [3])
    assert sp.take(0) == []                                       # off by default
    sp.enable()
    sp.add(0, 5, [1.0, 0.5], [3, 4])
    sp.add(1, 9, [2.0], [8])
    sp.add(0, 6, [0.1], [2])
    assert [r[0] for r in sp.take(0)] == [5, 6] and sp.take(0) == [] and sp.take(1) == [(9, [2.0], [8])]


def test_version2_drafter_loads_from_a_checkpoint_directory(tmp_path):
    """A drafter directory whose config says version 2 brings the convolution pairs and the selector in under the
    reference's tensor names; the loaded runner drafts what a runner holding the same tensors drafts."""
    import json
    from volta_engine_b200.loader.safetensors import write_safetensors
    from volta_engine_b200.models.factory import save_dense_checkpoint
    from volta_engine_b200.server.cli import load_drafter
    cfg, m, eng, dc = _setup()
    dcfg = DenseConfig(n_layers=dc.n_layers, hidden=dc.hidden, n_q=dc.n_q, n_kv=dc.n_kv, head_dim=dc.head_dim, ffn=dc.ffn,
                       vocab=cfg.vocab, rope_theta=dc.rope_theta, rms_eps=dc.rms_eps, qk_norm=True)
    save_dense_checkpoint(tmp_path, dcfg, seed=3, fmt="bf16", shards=1)
    hf = json.loads((tmp_path / "config.json").read_text())
    hf.update(sliding_window=64, dflash_config={"block_size": 4, "target_layer_ids": [0, cfg.n_layers - 1], "mask_token_id": 255,
                                                "version": 2, "conv_group_size": 16, "selector_rank": 32, "selector_top_k": 8})
    (tmp_path / "config.json").write_text(json.dumps(hf))
    g = torch.Generator().manual_seed(9)
    bf, H, taps, G = torch.bfloat16, dc.hidden, 2, dc.hidden // 16
    extra = {"fc.weight": (torch.randn(H, 2 * H, generator=g) * 0.02).to(bf), "hidden_norm.weight": torch.ones(H, dtype=bf),
             "candidate_selector.hidden_projection.weight": (torch.randn(32, H, generator=g) * 0.05).to(bf),
             "candidate_selector.predecessor_codebook": (torch.randn(cfg.vocab, 32, generator=g) * 0.3).to(bf),
             "candidate_selector.successor_codebook": (torch.randn(cfg.vocab, 32, generator=g) * 0.3).to(bf)}
    for i in range(dc.n_layers):
        for name in ("attention_conv", "mlp_conv"):
            base = (torch.randn(2 * taps, H, generator=g) * 0.02)
            base[0] += 1
            base[taps] += 1
            extra[f"layers.{i}.{name}.base_kernel"] = base.to(bf)
            extra[f"layers.{i}.{name}.kernel_projection.weight"] = (torch.randn(2 * taps * G, H, generator=g) * 0.02).to(bf)
    write_safetensors(tmp_path / "drafter_extra.safetensors", extra)
    r = load_drafter(eng, str(tmp_path))
    assert r.cfg.version == 2 and r.v2 is not None and r.cfg.selector_rank == 32
    assert torch.equal(r.v2["pred"], extra["candidate_selector.predecessor_codebook"])
    assert torch.equal(r.v2["layers"][1]["mlp_proj"].weight, extra["layers.1.mlp_conv.kernel_projection.weight"])
    p = _prompt(50, 2)
    eng.prefill(0, p)
    d = r.draft(0, 9, len(p))
    assert len(d) == 3 and all(0 <= t < cfg.vocab for t in d)


def test_drafter_round_profile_reports_stage_times():
    cfg, m, eng, dc = _setup()
    r = D.DFlashRunner(eng, _v2_config(dc))
    r.enable_profile()
    p = _prompt(40, 1)
    eng.prefill(0, p)
    r.draft(0, 5, len(p))
    r.draft(0, 6, len(p))
    rep = r.profile_report()
    assert rep["rounds"] == 2 and rep["backbone_ms"] > 0 and rep["select_ms"] > 0 and rep["ingest_ms"] >= 0


def test_tap_spool_records_tokens_taps_and_target_candidates(tmp_path):
    from volta_engine_b200.runtime.spec_logs import TapSpool, TargetSpool, read_tap_spool
    cfg, m, eng, dc = _setup()
    p = _prompt(45, 5)
    o = Options.resolve({"max_slots": 2, "prefix_interval": 0, "speculator": "draft", "spec_ctrl": False, "spec_depth": 3}, env={})
    g = Generator(eng, ByteTok(), o, eos_ids=[])
    g.drafter = D.DFlashRunner(eng, dc)
    g.tap_spool = TapSpool(str(tmp_path / "taps.bin"), window=32)
    g.target_spool = TargetSpool()
    g.target_spool.enable()
    out = g.generate(Request(p, max_tokens=10, cache_prefix=False))
    recs = read_tap_spool(str(tmp_path / "taps.bin"))
    assert len(recs) == 1 and recs[0]["tokens"] == p + out["tokens"]
    r = recs[0]
    n_all = len(p) + len(out["tokens"])
    assert r["taps"].shape == (32, 2 * cfg.hidden) and r["first_pos"] + 32 <= n_all
    assert float(abs(r["taps"]).sum()) > 0
    # every recorded target row predicts the token the request really produced at that position
    assert r["targets"] and all(t["ids"][max(range(16), key=lambda i: t["vals"][i])] == (p + out["tokens"])[t["pos"]] for t in r["targets"])
    # and the spooling step decodes the same tokens as the plain one
    cfg2, m2, eng2, _ = _setup()
    plain = Generator(eng2, ByteTok(), Options.resolve({"max_slots": 2, "prefix_interval": 0}, env={}), eos_ids=[]).generate(
        Request(p, max_tokens=10, cache_prefix=False))
    assert plain["tokens"] == out["tokens"]


def test_drafter_hessian_capture_accumulates_block_rows(tmp_path):
    cfg, m, eng, dc = _setup()
    r = D.DFlashRunner(eng, dc)
    hs = r.model.enable_hessians(None, min_rows=1)
    p = _prompt(40, 1)
    eng.prefill(0, p)
    r.draft(0, 5, len(p))
    files = hs.dump(str(tmp_path), 0)
    assert files and all(f.endswith(".f32") for f in files)
    import numpy as np
    h = np.fromfile(str(tmp_path / files[0]), dtype=np.float32)
    assert h.size > 0 and float(np.abs(h).sum()) > 0
