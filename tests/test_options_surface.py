"""Launch options: every key of the reference's option table parses; unknown keys are fatal; aliases map; the keys
that name subsystems this build does not wire say so. Reference: inc/engine/runtime/options.def, docs/CONFIG.md."""
import os

import pytest
import torch

from volta_engine_b200.runtime import options as O

KEYS_FILE = os.path.join(os.path.dirname(__file__), "data", "reference_option_keys.txt")


def _reference_keys():
    """Option names of the reference's table (inc/engine/runtime/options.def), one per line."""
    with open(KEYS_FILE) as f:
        return [ln.strip() for ln in f if ln.strip()]


def test_every_reference_key_is_accepted():
    keys = _reference_keys()
    assert len(keys) > 100
    known = O.known_keys()
    missing = [k for k in keys if k not in known]
    assert not missing, missing
    for k in keys:
        assert O.disposition(k)


def test_unknown_key_is_fatal():
    with pytest.raises(KeyError):
        O.Options.resolve({"no_such_option": 1}, env={})


def test_aliases_and_wide_values():
    o = O.Options.resolve({"prefix_cache_gib": 3, "loop_detect": "stop", "speculator": "dflash", "mtp_graph": False,
                           "expert_shard": 0, "sparse_head_file": "/tmp/x.bin", "spec_suffix": 2, "kv_format": ""}, env={})
    assert o.prefix_cache_mib == 3072 and o.loop_detect is True and o.speculator == "draft" and o.no_graphs is True
    assert o.expert_parallel is True and o.sparse_head_state == "/tmp/x.bin" and o.kv_format == "bf16"
    o = O.Options.resolve({"spec_suffix": 2}, env={})
    assert o.speculator == "suffix"
    o = O.Options.resolve({"speculator": "mtp", "mtp_depth": 5}, env={})
    assert o.spec_depth == 5


def test_ignored_lists_the_keys_without_effect():
    o = O.Options.resolve({"gemv_int8": False, "steer_push": 2.0, "prefill_cooldown": 2, "vision_mmproj": "x",
                           "expert_stage": 0}, env={})
    names = [k for k, _ in o.ignored()]
    assert "gemv_int8" in names and "prefill_cooldown" not in names and "steer_push" not in names
    assert "vision_mmproj" not in names and "expert_stage" not in names          # wired: they name subsystems that exist


def test_env_and_docs():
    o = O.Options.resolve({}, env={"ENGINE_PREFILL_COOLDOWN": "3", "ENGINE_AR_LL": "0"})
    assert o.prefill_cooldown == 3 and o.ar_ll is False
    doc = O.config_docs()
    for k in ("arena_gib", "prefill_cooldown", "gemv_int8", "steer_push", "trace_layers"):
        assert f"`{k}`" in doc


def test_layer_trace_wraps_sub_layers():
    from volta_engine_b200.models.dense import DenseConfig, DenseModel
    from volta_engine_b200.runtime.batch import BatchRows
    from volta_engine_b200.runtime.kv_cache import PagedKVCache
    from volta_engine_b200.utils.trace import enable_layer_trace
    cfg = DenseConfig(n_layers=2, hidden=256, n_q=2, n_kv=1, head_dim=128, ffn=256, vocab=512)
    model = DenseModel(cfg, torch.device("cpu")).init_random(seed=0)
    kv = PagedKVCache(2, model.nkv, 128, 4, 1, 128, torch.device("cpu"))
    seen, depth = [], [0]

    def push(name):
        seen.append(name)
        depth[0] += 1

    def pop():
        depth[0] -= 1

    assert enable_layer_trace(model, push, pop) == ["attn_block", "ffn_block"]
    assert enable_layer_trace(model, push, pop) == []            # wrapping twice would nest the ranges
    kv.reserve(0, 8)
    model.forward(BatchRows.make([1, 2, 3], [0, 1, 2], [0, 0, 0], torch.device("cpu")), kv)
    assert seen == ["L0.attn", "L0.ffn", "L1.attn", "L1.ffn"] and depth[0] == 0


def test_disk_tier_budget_trims_oldest(tmp_path):
    from volta_engine_b200.runtime.prefix_cache import PrefixCache
    pc = PrefixCache(1 << 30, str(tmp_path), fingerprint="m", disk_budget_bytes=200_000)

    def snap(a, b):
        return {"k": torch.zeros(b - a, 2000, dtype=torch.bfloat16)}

    for i in range(6):
        toks = [i] * 40
        pc.insert(toks, 16, snap)
        pc.flush()
    files = [f for f in os.listdir(os.path.join(str(tmp_path), "m")) if f.endswith(".pt")]
    total = sum(os.path.getsize(os.path.join(str(tmp_path), "m", f)) for f in files)
    assert total <= 200_000 and 1 <= len(files) < 6
    assert pc.stats["disk_bytes"] == total


def test_steering_from_launch_options_and_request_fields(tmp_path):
    """steer = file applies the file to every request; a request may switch it off, name another file of steer_dir,
    rescale it; the reasoning-marker penalty lowers the first tokens of the marker words inside the reasoning block."""
    from volta_engine_b200.models.dense import DenseConfig, DenseModel
    from volta_engine_b200.runtime.engine import Engine
    from volta_engine_b200.runtime.generator import Generator, Request
    from volta_engine_b200.runtime.kv_cache import PagedKVCache
    from volta_engine_b200.runtime.steering import SteerConfig, SteerEntry, SteerFile, STEER_ADD, save_steer_file
    from volta_engine_b200.server.protocol import ProtocolError, steer_fields

    class Tok:
        eos_ids = [0]

        def decode_bytes(self, ids, skip_special=False):
            return bytes(i & 0xFF for i in ids)

        def encode(self, text, allow_special=True):
            return list(text.encode())

    cfg = DenseConfig.tiny(vocab=256)
    model = DenseModel(cfg, "cpu").init_random(seed=0, search=False)
    g = torch.Generator().manual_seed(1)
    sf = SteerFile(hidden=cfg.hidden, layers=cfg.n_layers, entries=[
        SteerEntry(layer=li, kind=STEER_ADD, par=4.0, vec=torch.randn(cfg.hidden, generator=g)) for li in range(cfg.n_layers)])
    save_steer_file(str(tmp_path / "push.steer"), sf)
    o = O.Options.resolve({"steer": "file", "steer_file": str(tmp_path / "push.steer"), "steer_dir": str(tmp_path),
                           "steer_layers": f"0-{cfg.n_layers - 1}", "think_penalty": 0.0, "max_slots": 1}, env={})
    sc = SteerConfig(o, cfg.n_layers, Tok())
    assert sc.enabled and sc.default is not None and sc.penalty_ids

    def run(fields):
        kv = PagedKVCache(cfg.n_layers, model.nkv, cfg.head_dim, 24, 1, 512, "cpu")
        eng = Engine(model, kv, use_graphs=False, prefill_chunk=32)
        gen = Generator(eng, Tok(), o, eos_ids=[])
        gen.steer_cfg = sc
        model.steer = sc.tables(cfg.hidden, 1, "cpu")
        prompt = [(7 * i + 3) % 250 + 1 for i in range(40)]
        out = gen.generate(Request(prompt, max_tokens=8, cache_prefix=False, **sc.for_request(fields)))["tokens"]
        model.steer = None
        return out

    steered, plain = run({}), run({"steer_vector": "off"})
    assert steered != plain                                   # the file edits every request unless it says otherwise
    assert run({"steer_vector": "push"}) == steered           # the same file by name from steer_dir
    assert run({"steer_scale": 0.0}) == plain                 # scale 0 leaves the residual alone
    with pytest.raises(ValueError):
        sc.for_request({"steer_vector": "../etc/passwd"})
    assert steer_fields({"steer_scale": "2", "think_penalty": 1}) == {"steer_scale": 2.0, "think_penalty": 1.0}
    with pytest.raises(ProtocolError):
        steer_fields({"steer_scale": "x"})
    off = SteerConfig(O.Options.resolve({}, env={}), cfg.n_layers, Tok())
    assert not off.enabled and off.for_request({"steer_vector": "push"})["steer"] is None


def test_model_switches_drop_indexers_and_the_routing_histogram():
    from volta_engine_b200.models.mla import MLAConfig, MLAModel
    from volta_engine_b200.runtime.options import Options
    from volta_engine_b200.server.cli import apply_model_switches
    m = MLAModel(MLAConfig.tiny_mla(dsa=True, mtp_layers=0), "cpu").init_random(seed=1)
    assert all(L.dsa is not None for L in m.layers) and m.prefix_resume is None and m.heat is not None
    apply_model_switches(m, Options.resolve({}, env={}))
    assert all(L.dsa is not None for L in m.layers) and m.heat is not None          # defaults change nothing
    apply_model_switches(m, Options.resolve({"dsa": False, "expert_stats": False}, env={}))
    assert all(L.dsa is None for L in m.layers) and m.cfg.dsa is False and m.prefix_resume == "kv" and m.heat is None


def test_small_runtime_switches():
    import logging
    from volta_engine_b200.runtime.route_dump import RouteRecorder
    from volta_engine_b200.runtime.sparse_head_policy import SparseHeadParams, SparseHeadPolicy
    from volta_engine_b200.runtime.spec_controller import SpecController
    import torch
    p = SparseHeadPolicy(100, SparseHeadParams(capacity=4, interval=7))
    assert p.p.interval == 7 and not p.use_sparse()
    p.set_subset([1, 2, 3])
    p.force = True
    assert p.use_sparse()                      # forced: whatever the measured miss rate
    rec = RouteRecorder(layers=range(3, 5), min_rows=1)
    x, ids, w = torch.zeros(2, 8), torch.tensor([[0, 1], [1, 2]]), torch.ones(2, 2)
    rec.record(1, x, ids, w)
    rec.record(4, x, ids, w)
    assert list(rec.data) == [4]
    c = SpecController()
    c.log_decisions = True
    records = []
    h = logging.Handler()
    h.emit = lambda r: records.append(r.getMessage())
    lg = logging.getLogger("volta.spec")
    lg.addHandler(h)
    lg.setLevel(logging.INFO)
    try:
        c.use_speculation()
        c.record_round(3, 3, 2, 1.0)
        c.record_plain(1.0)
        for _ in range(40):
            c.use_speculation()
    finally:
        lg.removeHandler(h)
    assert any("probe" in r for r in records) and any("speculative round" in r for r in records)


def test_depth_by_rate_prefers_the_depth_with_the_best_expected_rate():
    from volta_engine_b200.runtime.spec_controller import DepthByRate
    d = DepthByRate(4)
    assert d.choose(3) in (2, 3) and d.time_model() is None
    # rounds cost 2 ms + 1 ms per row; the first draft is nearly always right, the later ones nearly never
    for i in range(60):
        drafted = 2 + (i % 3)
        d.record(drafted, 1, 2.0 + 1.0 * (drafted + 1))
    a, b = d.time_model()
    assert abs(a - 2.0) < 1e-6 and abs(b - 1.0) < 1e-6 and d.p[0] > 0.9 and d.p[1] < 0.1
    assert d.choose(4) == 1
    # every draft right and rows nearly free: go deep
    e = DepthByRate(4)
    for i in range(60):
        drafted = 3 + (i % 2)
        e.record(drafted, drafted, 5.0 + 0.01 * (drafted + 1))
    assert e.choose(3) == 4
