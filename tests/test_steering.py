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
