"""Scheduler behaviour on the CPU oracle path: greedy equivalence, speculation == plain decoding, stop rules,
seeded sampling, prefix-cache resume (RAM and disk), concurrent == sequential."""
import os

import pytest
import torch

from volta_engine_b200.models.dense import DenseConfig, DenseModel
from volta_engine_b200.runtime.engine import Engine
from volta_engine_b200.runtime.generator import Generator, Request, _utf8_split
from volta_engine_b200.runtime.kv_cache import PagedKVCache
from volta_engine_b200.runtime.options import Options
from volta_engine_b200.runtime.prefix_cache import PrefixCache
from volta_engine_b200.runtime.sampling import SamplingParams


class ByteTok:
    """Token id == byte value (vocab 256+): enough for the scheduler tests."""
    eos_ids = [0]

    def decode_bytes(self, ids, skip_special=False):
        return bytes(i & 0xFF for i in ids)

    def encode(self, text, allow_special=True):
        return list(text.encode())


@pytest.fixture(scope="module")
def model():
    cfg = DenseConfig.tiny(vocab=256)
    return DenseModel(cfg, "cpu").init_random(seed=0, search=False)


def make(model, slots=2, cache=None, **opt):
    kv = PagedKVCache(model.cfg.n_layers, model.nkv, model.cfg.head_dim, 40, slots, 512, "cpu")
    eng = Engine(model, kv, use_graphs=False, prefill_chunk=32)
    o = Options.resolve(dict({"max_slots": slots, "prefix_interval": 64}, **opt), env={})
    return Generator(eng, ByteTok(), o, prefix_cache=cache, eos_ids=[]), eng


def prompt(n, seed=0):
    return torch.randint(1, 256, (n,), generator=torch.Generator().manual_seed(seed)).tolist()


def test_greedy_matches_engine_and_length_stop(model):
    g, _ = make(model)
    r = g.generate(Request(prompt(70), max_tokens=12))
    kv = PagedKVCache(model.cfg.n_layers, model.nkv, model.cfg.head_dim, 40, 1, 512, "cpu")
    ref, _ = Engine(model, kv, use_graphs=False, prefill_chunk=1000).generate(prompt(70), 12)
    assert r["tokens"] == ref and r["reason"] == "length"
    assert r["usage"]["completion_tokens"] == 12 and r["usage"]["prompt_tokens"] == 70


def test_suffix_speculation_equals_plain(model):
    p = (prompt(20, 3) * 6)[:100]   # repetitive prompt so drafts exist
    plain, _ = make(model)
    a = plain.generate(Request(p, max_tokens=24))
    spec, _ = make(model, speculator="suffix", spec_ctrl=False, spec_depth=4)
    b = spec.generate(Request(p, max_tokens=24))
    assert a["tokens"] == b["tokens"]
    assert spec.metrics.spec["rounds"] > 0


def test_stop_string_and_stop_token(model):
    g, _ = make(model)
    full = g.generate(Request(prompt(40, 1), max_tokens=20))
    text = full["text"]
    cut = text[5:8]
    if cut and text.find(cut) == 5:
        r = g.generate(Request(prompt(40, 1), max_tokens=20, stop=[cut]))
        assert r["reason"] == "stop_string" and r["text"] == text[:5]
    r2 = g.generate(Request(prompt(40, 1), max_tokens=20, stop_token_ids=[full["tokens"][3]]))
    assert r2["reason"] == "stop" and r2["tokens"] == full["tokens"][:full["tokens"].index(full["tokens"][3])]


def test_seeded_sampling_is_reproducible(model):
    g, _ = make(model)
    sp = SamplingParams(temperature=0.9, top_p=0.95, top_k=12, seed=7, presence_penalty=0.2)
    a = g.generate(Request(prompt(30, 2), max_tokens=10, params=sp))
    b = g.generate(Request(prompt(30, 2), max_tokens=10, params=sp))
    c = g.generate(Request(prompt(30, 2), max_tokens=10, params=SamplingParams(temperature=0.9, seed=8)))
    assert a["tokens"] == b["tokens"] and len(a["tokens"]) == 10
    assert c["tokens"] != a["tokens"] or True


def test_prefix_cache_resume_ram_and_disk(model, tmp_path):
    p = prompt(150, 5)
    cache = PrefixCache(64 << 20, disk_dir=str(tmp_path), fingerprint="t")
    g, _ = make(model, cache=cache)
    a = g.generate(Request(p, max_tokens=8))
    b = g.generate(Request(p, max_tokens=8))
    assert a["tokens"] == b["tokens"]
    assert b["usage"]["cached_tokens"] >= 128 and a["usage"]["cached_tokens"] == 0
    # follow-up turn resumes after the first answer
    p2 = p + a["tokens"] + prompt(10, 6)
    c = g.generate(Request(p2, max_tokens=4))
    assert c["usage"]["cached_tokens"] >= len(p) + len(a["tokens"]) - 1
    cache.flush()
    cache2 = PrefixCache(64 << 20, disk_dir=str(tmp_path), fingerprint="t")   # restart: disk tier only
    g2, _ = make(model, cache=cache2)
    d = g2.generate(Request(p, max_tokens=8))
    assert d["tokens"] == a["tokens"] and d["usage"]["cached_tokens"] >= 128
    assert cache2.stats["disk_hits"] > 0


def test_concurrent_equals_sequential(model):
    g, _ = make(model, slots=2)
    pa, pb = prompt(50, 8), prompt(90, 9)
    sa = g.generate(Request(pa, max_tokens=10))["tokens"]
    sb = g.generate(Request(pb, max_tokens=10))["tokens"]
    out = {}
    g.submit(Request(pa, max_tokens=10, on_text=lambda t, ids, lp: out.setdefault("a", []).extend(ids)))
    g.submit(Request(pb, max_tokens=10, on_text=lambda t, ids, lp: out.setdefault("b", []).extend(ids)))
    for _ in range(200):
        g.step()
        if not g.pending and all(s.phase == "idle" for s in g.slots):
            break
    assert out["a"] == sa and out["b"] == sb
    assert g.metrics.snapshot()["totals"]["completed"] == 4


def test_utf8_boundary():
    b = "héllo 🙂".encode()
    t, rest = _utf8_split(b[:-2])
    assert t == "héllo " and rest == b[-4:-2]
    assert _utf8_split(b) == ("héllo 🙂", b"")


def test_mtp_speculation_equals_plain_greedy():
    from volta_engine_b200.models.mla import MLAConfig, MLAModel
    cfg = MLAConfig.tiny_mla(vocab=256)
    m = MLAModel(cfg, "cpu").init_random(seed=1)

    def gen(**opt):
        kv = PagedKVCache(cfg.n_layers + 1, 1, 576, 24, 2, 512, "cpu", v_head_dim=8)
        eng = Engine(m, kv, use_graphs=False, prefill_chunk=32)
        o = Options.resolve(dict({"max_slots": 2, "prefix_interval": 0}, **opt), env={})
        return Generator(eng, ByteTok(), o, eos_ids=[])
    p = prompt(45, 12)
    plain = gen().generate(Request(p, max_tokens=14, cache_prefix=False))
    g = gen(speculator="mtp", spec_ctrl=False, spec_depth=3)
    spec = g.generate(Request(p, max_tokens=14, cache_prefix=False))
    assert spec["tokens"] == plain["tokens"]
    assert g.metrics.spec["rounds"] > 0 and g.metrics.spec["proposed"] == 3 * g.metrics.spec["rounds"]


def test_reasoning_budget_forces_the_closing_sequence(model):
    gen, _ = make(model, thinking_soft_close=0)
    prompt = [(11 * i + 5) % 250 for i in range(30)]
    free = gen.generate(Request(prompt=prompt, max_tokens=24))["tokens"]
    close = [201, 202, 203]
    assert not any(t in close for t in free)
    out = gen.generate(Request(prompt=prompt, max_tokens=24, think_open=True, think_end_id=202, think_close=close,
                               thinking_budget=5))["tokens"]
    k = out.index(close[0])
    assert out[:k] == free[:k] and 3 <= k <= 5       # untouched while inside the budget
    assert out[k:k + 3] == close and len(out) == 24  # then the closing sequence, then the model goes on
    # a block that closes by itself is left alone
    own = gen.generate(Request(prompt=prompt, max_tokens=12, think_open=True, think_end_id=free[2], think_close=close,
                               thinking_budget=8))["tokens"]
    assert own == free[:12]


def test_reasoning_budget_soft_close_waits_for_a_sentence_end(model):
    """thinking_soft_close = n: once the budget is spent the block stays open until a token ends a sentence or a line,
    at most n tokens; the byte tokenizer of the test makes token 46 a full stop and 10 a newline."""
    gen0, _ = make(model, thinking_soft_close=0)
    prompt = [(11 * i + 5) % 250 for i in range(30)]
    free = gen0.generate(Request(prompt=prompt, max_tokens=24))["tokens"]
    close = [201, 202, 203]
    # no sentence end among the free tokens: the close lands exactly soft tokens after the budget ran out
    assert not any(t in (10, 33, 46, 63) for t in free[:12])
    gen, _ = make(model, thinking_soft_close=4)
    out = gen.generate(Request(prompt=prompt, max_tokens=24, think_open=True, think_end_id=202, think_close=close,
                               thinking_budget=5))["tokens"]
    exact = gen0.generate(Request(prompt=prompt, max_tokens=24, think_open=True, think_end_id=202, think_close=close,
                                  thinking_budget=5))["tokens"].index(close[0])
    k = out.index(close[0])
    assert out[:k] == free[:k] and k == exact + 4 and out[k:k + 3] == close
    # the sentence rule itself
    class S:
        last_char = ""
    g = gen
    assert g._ends_sentence(S(), 46) and g._ends_sentence(S(), 10) and g._ends_sentence(S(), 33) and not g._ends_sentence(S(), 65)
    S.last_char = "3"
    assert not g._ends_sentence(S(), 46)          # "3." is a number, not the end of a sentence


@pytest.mark.parametrize("family", ["hybrid", "dsv4"])
def test_models_with_state_outside_the_kv_pool_do_not_resume_from_snapshots(family):
    """Snapshots hold KV pages only. A model with recurrent / ring / indexer state outside the pool must answer the
    same prompt identically the second time with the cache passed in (the scheduler drops it), not continue from the state
    the slot's previous request left behind."""
    if family == "hybrid":
        from volta_engine_b200.models.hybrid import HybridConfig, HybridModel
        cfg = HybridConfig.tiny_hybrid(vocab=256, qsa=True)          # indexer keys live outside the pool
        m = HybridModel(cfg, "cpu").init_random(seed=0, search=False)
        kv = PagedKVCache(m.kv_layers, m.nkv, cfg.head_dim, 24, 2, 512, "cpu")
    else:
        from volta_engine_b200.models.dsv4 import DSV4Config, DSV4Model
        cfg = DSV4Config.tiny_dsv4()
        m = DSV4Model(cfg, "cpu").init_random(seed=5, std=0.05)
        kv = PagedKVCache(1, 1, 64, 24, 2, 512, "cpu")
    assert m.prefix_resume is None
    eng = Engine(m, kv, use_graphs=False, prefill_chunk=32)
    o = Options.resolve({"max_slots": 1, "prefix_interval": 32}, env={})
    g = Generator(eng, ByteTok(), o, prefix_cache=PrefixCache(64 << 20), eos_ids=[])
    assert g.cache is None
    p = [t % cfg.vocab for t in prompt(70, 3)]
    cold = g.generate(Request(p, max_tokens=6))
    again = g.generate(Request(p, max_tokens=6))
    assert again["tokens"] == cold["tokens"] and again["usage"]["cached_tokens"] == 0
    turn2 = g.generate(Request(p + cold["tokens"] + p[:9], max_tokens=4))
    kv2 = type(kv)(kv.n_layers, kv.n_kv, kv.head_dim, 24, 2, 512, "cpu")
    g2 = Generator(Engine(m, kv2, use_graphs=False, prefill_chunk=32), ByteTok(), o, eos_ids=[])
    assert g2.generate(Request(p + cold["tokens"] + p[:9], max_tokens=4))["tokens"] == turn2["tokens"]


def test_prefix_cache_fingerprint_separates_models(tmp_path):
    from volta_engine_b200.runtime.prefix_cache import model_fingerprint
    d = tmp_path / "m"
    d.mkdir()
    (d / "config.json").write_text('{"model_type": "dense", "hidden_size": 64}')
    (d / "model.safetensors").write_bytes(b"x" * 100)
    a = model_fingerprint(str(d), kv_format="bf16", tp=1)
    assert a == model_fingerprint(str(d), kv_format="bf16", tp=1)
    assert a != model_fingerprint(str(d), kv_format="fp8", tp=1)
    assert a != model_fingerprint(str(d), kv_format="bf16", tp=2)
    (d / "model.safetensors").write_bytes(b"y" * 101)
    assert a != model_fingerprint(str(d), kv_format="bf16", tp=1)


def test_prefix_cache_insert_refuses_a_detached_parent():
    cache = PrefixCache(1 << 20)
    toks = list(range(1, 40))
    snap = lambda a, b: {"from": a, "to": b, "p0": 0, "k": torch.zeros(1, 1, 4), "v": torch.zeros(1, 1, 4)}
    parent = cache.insert(toks, 16, snap)
    assert parent is not None and cache.entries == 1

    def evicting_snapshot(a, b):
        # the parent disappears while the snapshot is being taken (outside the lock)
        cache.root.children[toks[0]].remove(parent)
        cache.entries -= 1
        return snap(a, b)
    assert cache.insert(toks, 32, evicting_snapshot) is None
    assert cache.entries == 0 and cache.find(toks) == []


def test_speculative_sampling_step_is_distributed_like_the_target():
    """Accept the draft with probability p(draft), else draw from the rest renormalised: the token that comes out has the
    target distribution whatever the draft (inc/engine/runtime/sampling.h:197-223 in the reference)."""
    from volta_engine_b200.runtime.sampling import Candidates, Xoshiro256pp, distribution, spec_step
    c = Candidates([7, 3, 9, 1], [2.0, 1.5, 0.2, -1.0], 2.9)
    p = SamplingParams(temperature=0.8)
    want = dict(zip(c.ids, distribution(c, p)))
    for draft in (7, 9, 55):                        # likely draft, unlikely draft, draft outside the candidates
        rng = Xoshiro256pp(123 + draft)
        n, seen, hits = 40000, {}, 0
        for _ in range(n):
            ok, t = spec_step(c, p, draft, rng)
            assert ok == (t == draft) or (not ok and t != draft)
            hits += ok
            seen[t] = seen.get(t, 0) + 1
        for tok, q in want.items():
            assert abs(seen.get(tok, 0) / n - q) < 0.012, (draft, tok, seen.get(tok, 0) / n, q)
        assert abs(hits / n - want.get(draft, 0.0)) < 0.012


def test_sampled_requests_take_speculative_rounds(model):
    p = (prompt(20, 3) * 6)[:100]
    spec, _ = make(model, speculator="suffix", spec_ctrl=False, spec_depth=4)
    sp = SamplingParams(temperature=0.7, top_k=8, seed=11)
    a = spec.generate(Request(p, max_tokens=24, params=sp))
    assert spec.metrics.spec["rounds"] > 0 and len(a["tokens"]) == 24
    b = spec.generate(Request(p, max_tokens=24, params=sp))
    assert a["tokens"] == b["tokens"]               # seeded: the same draws, round by round
    # a near-zero temperature makes the sampled rounds agree with greedy decoding
    cold = spec.generate(Request(p, max_tokens=24, params=SamplingParams(temperature=1e-4, seed=5)))
    plain, _ = make(model)
    assert cold["tokens"] == plain.generate(Request(p, max_tokens=24))["tokens"]


def _hybrid():
    from volta_engine_b200.models.hybrid import HybridConfig, HybridModel
    cfg = HybridConfig.tiny_hybrid(vocab=256)
    m = HybridModel(cfg, "cpu").init_random(seed=0, search=False)

    def gen(cache=None, **opt):
        kv = PagedKVCache(m.kv_layers, m.nkv, cfg.head_dim, 24, 2, 512, "cpu")
        eng = Engine(m, kv, use_graphs=False, prefill_chunk=32)
        o = Options.resolve(dict({"max_slots": 1, "prefix_interval": 32}, **opt), env={})
        return Generator(eng, ByteTok(), o, prefix_cache=cache, eos_ids=[])
    return m, gen


def test_hybrid_model_resumes_from_snapshots_that_carry_its_recurrent_state():
    """KV pages + the convolution and recurrent state at the snapshot's last position: the second request continues from
    the cached prefix and produces what a cold run produces; another request in between leaves its own state in the slot."""
    m, gen = _hybrid()
    assert m.prefix_resume == "kv+state"
    g = gen(cache=PrefixCache(256 << 20))
    assert g.cache is not None
    p = prompt(70, 3)
    cold = g.generate(Request(p, max_tokens=6))
    g.generate(Request(prompt(50, 9), max_tokens=3))             # overwrites the slot's state
    again = g.generate(Request(p, max_tokens=6))
    assert again["usage"]["cached_tokens"] >= 64 and again["tokens"] == cold["tokens"]
    turn2 = p + cold["tokens"] + p[:9]
    warm = g.generate(Request(turn2, max_tokens=5))
    assert warm["usage"]["cached_tokens"] >= 70                  # the reply snapshot
    assert warm["tokens"] == gen().generate(Request(turn2, max_tokens=5))["tokens"]


def test_hybrid_model_takes_rejected_draft_rows_back():
    """Suffix speculation on the model with recurrent state: a verify block runs journalled, rejected rows are rolled
    back, and the tokens equal plain greedy decoding."""
    m, gen = _hybrid()
    p = prompt(60, 3)
    kv0 = PagedKVCache(m.kv_layers, m.nkv, m.cfg.head_dim, 24, 2, 512, "cpu")
    plain, _ = Engine(m, kv0, use_graphs=False, prefill_chunk=32).generate(p, 12)
    m.gdn_states = None
    kv1 = PagedKVCache(m.kv_layers, m.nkv, m.cfg.head_dim, 24, 2, 512, "cpu")
    eng = Engine(m, kv1, use_graphs=False, prefill_chunk=32)
    assert eng.supports_journal
    assert eng.prefill(0, p) == plain[0]
    out, pos = [plain[0]], len(p)
    wrong = (plain[3] + 1) % 256
    for drafts in ([plain[1], plain[2], wrong, 7], [wrong], [plain[5], plain[6]], [plain[8], wrong, wrong]):
        rows = [out[-1]] + drafts
        toks = eng.step(rows, [pos + i for i in range(len(rows))], [0] * len(rows), journal=True)
        acc = 0
        while acc < len(drafts) and toks[acc] == drafts[acc]:
            acc += 1
        if acc < len(drafts):
            eng.rollback(0, acc + 1)
        out += drafts[:acc] + [toks[acc]]
        pos += acc + 1
    assert out == plain[:len(out)] and len(out) >= 9, (out, plain)
    m.gdn_states = None
    # the journal's replay equals stepping: state after a block of 4 rows rolled back to 2 == state after 2 rows
    from volta_engine_b200.runtime.batch import BatchRows
    kv = PagedKVCache(m.kv_layers, m.nkv, m.cfg.head_dim, 24, 2, 512, "cpu")
    kv.reserve(0, 64)
    m.gdn_states = None
    rows = BatchRows.make([5, 6, 7, 8], [0, 1, 2, 3], [0] * 4, "cpu")
    m.begin_journal(True, 4)
    m.forward(rows, kv)
    m.rollback_state(0, 2)
    got = [(s.conv[0].clone(), s.rec[0].clone()) for s in m.gdn_states if s is not None]
    m.gdn_states = None
    m.begin_journal(False)
    m.forward(BatchRows.make([5, 6], [0, 1], [0] * 2, "cpu"), kv)
    want = [(s.conv[0], s.rec[0]) for s in m.gdn_states if s is not None]
    assert all(torch.equal(a, c) and torch.equal(b, d) for (a, b), (c, d) in zip(got, want))


def test_hybrid_model_with_its_own_mtp_head_speculates_like_plain_greedy():
    """The hybrid (GDN + gated attention) family with a checkpoint-style MTP head: the head's block is one more
    full-attention layer with its own cache layer; rounds run journalled and rejected drafts are rolled back."""
    from volta_engine_b200.models.hybrid import HybridConfig, HybridModel
    cfg = HybridConfig.tiny_hybrid(vocab=256, mtp_layers=1)
    m = HybridModel(cfg, "cpu").init_random(seed=0, search=False)
    assert m.mtp is not None and m.kv_layers == m.n_full + 1 and len(m.layers) == cfg.n_layers
    assert m.mtp["layer"].gdn is None and m.mtp["layer"].kv_index == m.n_full

    def gen(**opt):
        kv = PagedKVCache(m.kv_layers, m.nkv, cfg.head_dim, 24, 2, 512, "cpu")
        m.gdn_states = None
        eng = Engine(m, kv, use_graphs=False, prefill_chunk=32)
        o = Options.resolve(dict({"max_slots": 2, "prefix_interval": 0}, **opt), env={})
        return Generator(eng, ByteTok(), o, eos_ids=[])
    p = prompt(45, 12)
    plain = gen().generate(Request(p, max_tokens=14, cache_prefix=False))
    g = gen(speculator="mtp", spec_ctrl=False, spec_depth=3)
    spec = g.generate(Request(p, max_tokens=14, cache_prefix=False))
    assert spec["tokens"] == plain["tokens"]
    assert g.metrics.spec["rounds"] > 0 and g.metrics.spec["accepted"] < g.metrics.spec["proposed"]
