"""Steering: control-vector files, layer / scope specs, residual edits (CPU oracle and CUDA kernel), marker penalty,
probe axes, and the effect on a model's output."""
import pytest
import torch

from volta_engine_b200.runtime import steering as st


def _file(H=64, layers=6):
    g = torch.Generator().manual_seed(0)
    v = torch.randn(H, generator=g)
    v = v / v.norm()
    return st.SteerFile(H, layers, st.SCOPE_GENERATED, 2.0, [
        st.SteerEntry(2, st.STEER_ADD, 0.5, v), st.SteerEntry(3, st.STEER_CLAMP, 0.1, v),
        st.SteerEntry(3, st.STEER_CLAMP_KEEP, -0.2, torch.roll(v, 1)), st.SteerEntry(1, st.STEER_ROUTE, 1.5, None, expert=7)])


def test_file_round_trip_and_specs(tmp_path):
    sf = _file()
    st.save_steer_file(tmp_path / "a.steer", sf)
    back = st.load_steer_file(tmp_path / "a.steer")
    assert (back.hidden, back.layers, back.scope, back.scale, len(back.entries)) == (64, 6, st.SCOPE_GENERATED, 2.0, 4)
    assert torch.equal(back.entries[0].vec, sf.entries[0].vec) and back.entries[3].expert == 7 and back.entries[3].vec is None
    (tmp_path / "bad.steer").write_bytes(b"NOPE" + b"\0" * 40)
    with pytest.raises(ValueError):
        st.load_steer_file(tmp_path / "bad.steer")
    raw = (tmp_path / "a.steer").read_bytes()
    (tmp_path / "cut.steer").write_bytes(raw[:-10])
    with pytest.raises(ValueError):
        st.load_steer_file(tmp_path / "cut.steer")
    assert st.parse_steer_scope("prompt,think") == 3 and st.parse_steer_scope("generated") == 6 and st.parse_steer_scope("all") == 7
    with pytest.raises(ValueError):
        st.parse_steer_scope("everything")
    assert st.parse_steer_layers("", 48) == (16, 32)
    assert st.parse_steer_layers("4-last", 48) == (4, 47)
    assert st.parse_steer_layers("0.25-1/2", 48) == (12, 24)
    for bad in ("7", "9-3", "0-48", "x-y"):
        with pytest.raises(ValueError):
            st.parse_steer_layers(bad, 48)


def _tables(dev):
    sf = _file()
    t = st.SteerTables(64, 1, 4, 3, dev)
    t.set_slot(1, sf, prompt_len=5, scale=1.5, think_end=9, penalty_ids=[3, 10, 70], penalty=2.5)
    return sf, t


def test_residual_edit_semantics_cpu():
    sf, t = _tables("cpu")
    g = torch.Generator().manual_seed(1)
    h = torch.randn(4, 64, generator=g).to(torch.bfloat16)
    pos = torch.tensor([2, 6, 6, 12], dtype=torch.int32)
    slot = torch.tensor([1, 1, 0, 1], dtype=torch.int32)
    v = sf.entries[0].vec
    out = t.apply(h.clone(), pos, slot, 2)
    assert torch.equal(out[0], h[0]) and torch.equal(out[2], h[2])            # prompt row / unsteered slot untouched
    want = (h[1].float() + 0.5 * 2.0 * 1.5 * v).to(torch.bfloat16)
    assert torch.equal(out[1], want) and not torch.equal(out[3], h[3])
    big = (v * 3.0).to(torch.bfloat16)[None].repeat(2, 1)
    out3 = t.apply(big.clone(), torch.tensor([6, 6], dtype=torch.int32), torch.tensor([1, 1], dtype=torch.int32), 3)
    assert abs(float(out3[0].float() @ v) - 0.1) < 0.35                        # clamped towards the reference level
    assert torch.equal(t.apply(h.clone(), pos, slot, 0), h)                    # layer outside the steered range
    logits = torch.zeros(4, 100)
    t.penalize(logits, pos, slot, id0=0)
    assert float(logits[1, 3]) == -2.5 and float(logits[1, 70]) == -2.5 and float(logits[1].sum()) == -7.5
    assert float(logits[0].abs().sum()) == 0 and float(logits[3].abs().sum()) == 0     # prompt row, answer row


def test_probe_axes():
    g = torch.Generator().manual_seed(2)
    d = torch.zeros(32); d[3] = 1.0
    a = torch.randn(20, 32, generator=g) * 0.1
    b = a + 2.0 * d
    ax = st.probe_axis(a, b)
    assert float(ax.dir @ d) > 0.99 and abs(ax.pb - ax.pa - 2.0) < 0.1
    assert abs(st.probe_fraction(ax, a.mean(0))) < 1e-3 and abs(st.probe_fraction(ax, b.mean(0)) - 1.0) < 1e-3
    axo = st.probe_axis(a, b, orthogonalize=True)
    assert abs(float(axo.dir.norm()) - 1.0) < 1e-5


def test_steering_changes_a_model_output_only_for_steered_slots():
    from volta_engine_b200.models.dense import DenseConfig, DenseModel
    from volta_engine_b200.runtime.engine import Engine
    from volta_engine_b200.runtime.kv_cache import PagedKVCache
    cfg = DenseConfig.tiny(vocab=256)
    m = DenseModel(cfg, "cpu").init_random(seed=0)
    prompt = [(5 * i + 1) % 256 for i in range(20)]

    def run(slot):
        kv = PagedKVCache(cfg.n_layers, m.nkv, cfg.head_dim, 16, 2, 256, "cpu")
        return Engine(m, kv, use_graphs=False, prefill_chunk=64).generate(prompt, 6, slot=slot)[0]
    base = run(0)
    g = torch.Generator().manual_seed(3)
    v = torch.randn(cfg.hidden, generator=g)
    sf = st.SteerFile(cfg.hidden, cfg.n_layers, st.SCOPE_ALL, 1.0, [st.SteerEntry(0, st.STEER_ADD, 40.0, v / v.norm())])
    m.steer = st.SteerTables(cfg.hidden, 0, 1, 2, "cpu")
    m.steer.set_slot(1, sf, prompt_len=len(prompt))
    assert run(0) == base                      # slot 0 carries no steering
    assert run(1) != base
    m.steer = None


@pytest.mark.gpu
def test_gpu_kernels_match_cpu_semantics():
    dev = torch.device("cuda:0")
    _, tc = _tables("cpu")
    _, tg = _tables(dev)
    g = torch.Generator().manual_seed(4)
    h = (torch.randn(6, 64, generator=g) * 2).to(torch.bfloat16)
    pos = torch.tensor([2, 6, 6, 12, 7, 8], dtype=torch.int32)
    slot = torch.tensor([1, 1, 0, 1, 1, -1], dtype=torch.int32)
    for layer in (1, 2, 3, 4):
        want = tc.apply(h.clone(), pos, slot, layer).float()
        got = tg.apply(h.clone().to(dev), pos.to(dev), slot.to(dev), layer).float().cpu()
        assert torch.allclose(got, want, atol=3e-2, rtol=2e-2), layer
    lw = tc.penalize(torch.zeros(6, 100), pos, slot, id0=5)
    lg = tg.penalize(torch.zeros(6, 100, device=dev), pos.to(dev), slot.to(dev), id0=5).cpu()
    assert torch.equal(lg, lw)


def test_request_time_probe_builds_directions_gates_and_steers(tmp_path):
    """runtime.steer_probe on a tiny dense model: states are read at the band layers for every opening, the gate places
    the prompt between the two groups, a fired gate installs clamps (count per layer = directions, hedge adds one, push adds
    one), a shut gate installs nothing; through the scheduler a probed request reports its scores and still decodes."""
    from volta_engine_b200.models.dense import DenseConfig, DenseModel
    from volta_engine_b200.runtime import steer_probe as sp
    from volta_engine_b200.runtime.engine import Engine
    from volta_engine_b200.runtime.generator import Generator, Request
    from volta_engine_b200.runtime.kv_cache import PagedKVCache
    from volta_engine_b200.runtime.options import Options

    class Tok:
        eos_ids = [0]

        def decode_bytes(self, ids, skip_special=False):
            return bytes(i & 0xFF for i in ids)

        def encode(self, text, allow_special=True):
            return [1 + (b % 250) for b in text.encode()]
    cfg = DenseConfig.tiny(vocab=256)
    m = DenseModel(cfg, "cpu").init_random(seed=0)
    eng = Engine(m, PagedKVCache(cfg.n_layers, m.nkv, cfg.head_dim, 40, 2, 512, "cpu"), use_graphs=False, prefill_chunk=32)
    o = Options.resolve({"max_slots": 2, "prefix_interval": 0, "steer": "on", "steer_layers": "0-last", "steer_band": "0-last",
                         "steer_directions": 2, "steer_hedge_strength": 0.5, "steer_gate_threshold": "-100"}, env={})
    scfg = st.SteerConfig(o, cfg.n_layers, Tok())
    m.steer = scfg.tables(cfg.hidden, 2, "cpu")
    ps = sp.ProbeSettings.from_options(o, cfg.n_layers, scfg.first, scfg.last)
    assert ps.directions == 2 and ps.band == (0, cfg.n_layers - 1) and ps.gate_threshold == -100.0 and ps.edit_strength == sp.AUTO_STRENGTH
    prompt = [5 + (3 * i) % 200 for i in range(30)]
    eng.prefill(0, prompt)
    states = sp.collect_states(eng, m.steer, 0, len(prompt), prompt[-1], ps.openings, Tok(), ps.band)
    assert set(states) == {"prompt", "accept", "decline", "plain", "hedged"}
    assert set(states["accept"]) == set(range(cfg.n_layers)) and states["accept"][0].shape == (4, cfg.hidden)
    edits, scores = sp.build_edits(states, ps, cfg.hidden, cfg.n_layers)
    assert scores["fired"] and edits is not None
    per = {}
    for e in edits.entries:
        per[e.layer] = per.get(e.layer, 0) + 1
        assert abs(float(e.vec.norm()) - 1.0) < 1e-4 and e.kind in (st.STEER_CLAMP, st.STEER_CLAMP_KEEP)
    assert all(v == 3 for v in per.values())                    # first direction + one extra + the hedge clamp
    ps.gate_threshold = 100.0
    assert sp.build_edits(states, ps, cfg.hidden, cfg.n_layers)[0] is None
    ps.push = -0.5                                              # a push does not wait for the gate
    pushed, _ = sp.build_edits(states, ps, cfg.hidden, cfg.n_layers)
    assert pushed is not None and all(e.kind == st.STEER_ADD and e.par < 0 for e in pushed.entries)
    # the extra directions are orthogonal to the first one
    ex = sp.extra_directions(states["accept"][1], states["decline"][1], st.probe_axis(states["accept"][1], states["decline"][1]).dir, 2)
    assert ex and all(abs(float(d @ st.probe_axis(states["accept"][1], states["decline"][1]).dir)) < 1e-4 for d in ex)
    # openings file
    f = tmp_path / "open.txt"
    f.write_text("accept: Absolutely\naccept: Gladly\ndecline: No.\nnoise line\n")
    op = sp.load_openings(str(f))
    assert op["accept"] == ["Absolutely", "Gladly"] and op["decline"] == ["No."] and op["plain"] == sp.DEFAULT_OPENINGS["plain"]
    # through the scheduler
    eng2 = Engine(m, PagedKVCache(cfg.n_layers, m.nkv, cfg.head_dim, 40, 2, 512, "cpu"), use_graphs=False, prefill_chunk=32)
    g = Generator(eng2, Tok(), o, eos_ids=[])
    g.steer_cfg = scfg
    g.probe_cfg = sp.ProbeSettings.from_options(o, cfg.n_layers, scfg.first, scfg.last)
    plain = g.generate(Request(prompt, max_tokens=6, cache_prefix=False))
    assert "steer_probe" not in plain["usage"]
    probed = g.generate(Request(prompt, max_tokens=6, cache_prefix=False, **scfg.for_request({"steer_probe": True})))
    sc = probed["usage"]["steer_probe"]
    assert sc["fired"] and sc["edits"] > 0 and len(probed["tokens"]) == 6
    again = g.generate(Request(prompt, max_tokens=6, cache_prefix=False))
    assert again["tokens"] == plain["tokens"]                   # the slot's edits are gone with the request


def test_probe_files_are_scored_at_the_last_prompt_token(tmp_path):
    from volta_engine_b200.models.dense import DenseConfig, DenseModel
    from volta_engine_b200.runtime import steer_probe as sp
    from volta_engine_b200.runtime.engine import Engine
    from volta_engine_b200.runtime.generator import Generator, Request
    from volta_engine_b200.runtime.kv_cache import PagedKVCache
    from volta_engine_b200.runtime.options import Options

    class Tok:
        eos_ids = [0]

        def decode_bytes(self, ids, skip_special=False):
            return bytes(i & 0xFF for i in ids)

        def encode(self, text, allow_special=True):
            return [1 + (b % 250) for b in text.encode()]
    cfg = DenseConfig.tiny(vocab=256)
    m = DenseModel(cfg, "cpu").init_random(seed=0)
    g = torch.Generator().manual_seed(5)
    v = torch.randn(cfg.hidden, generator=g)
    v = v / v.norm()
    st.save_steer_file(tmp_path / "mood.steer", st.SteerFile(cfg.hidden, cfg.n_layers, st.SCOPE_ALL, 1.0,
                                                             [st.SteerEntry(1, st.STEER_PROBE, 0.25, v)]))
    st.save_steer_file(tmp_path / "empty.steer", st.SteerFile(cfg.hidden, cfg.n_layers, st.SCOPE_ALL, 1.0,
                                                              [st.SteerEntry(1, st.STEER_ADD, 0.25, v)]))
    probes = sp.load_probe_files("mood", str(tmp_path))
    assert list(probes) == ["mood"] and len(probes["mood"]) == 1
    with pytest.raises(ValueError):
        sp.load_probe_files("empty", str(tmp_path))
    with pytest.raises(ValueError):
        sp.load_probe_files("../mood", str(tmp_path))
    o = Options.resolve({"max_slots": 2, "prefix_interval": 0, "steer": "on", "steer_layers": "0-last"}, env={})
    scfg = st.SteerConfig(o, cfg.n_layers, Tok())
    m.steer = scfg.tables(cfg.hidden, 2, "cpu")
    eng = Engine(m, PagedKVCache(cfg.n_layers, m.nkv, cfg.head_dim, 40, 2, 512, "cpu"), use_graphs=False, prefill_chunk=32)
    gen = Generator(eng, Tok(), o, eos_ids=[])
    gen.steer_cfg, gen.probe_files = scfg, probes
    prompt = [5 + (3 * i) % 200 for i in range(30)]
    out = gen.generate(Request(prompt, max_tokens=4, cache_prefix=False))
    score = out["usage"]["probes"]["mood"]
    # the same number from a capture by hand
    eng2 = Engine(m, PagedKVCache(cfg.n_layers, m.nkv, cfg.head_dim, 40, 2, 512, "cpu"), use_graphs=False, prefill_chunk=32)
    eng2.prefill(0, prompt)
    with sp.StateCapture(m.steer, (1, 1)) as cap:
        cap.row = 0
        sp._run_rows(eng2, 0, [prompt[-1]], len(prompt) - 1)
    assert abs(score - (float(cap.states[1] @ v) - 0.25)) < 1e-3
    m.steer = None
