"""Gated DeltaNet mixer and the hybrid model: oracle properties on CPU, CUDA kernels against the oracle."""
import pytest
import torch

from volta_engine_b200.models.hybrid import HybridConfig, HybridModel
from volta_engine_b200.ops.gdn import GDNDims, GDNState, gdn_forward, gdn_reference
from volta_engine_b200.runtime.engine import Engine
from volta_engine_b200.runtime.kv_cache import PagedKVCache


def _params(d, g):
    return dict(conv_w=torch.randn(d.conv_dim, d.conv_k, generator=g) * 0.5,
                A_log=torch.log(torch.linspace(1.0, 4.0, d.n_v)), dt_bias=torch.linspace(-1, 1, d.n_v),
                norm_w=torch.rand(d.dv, generator=g) + 0.5)


def test_oracle_chunking_and_slot_independence():
    d = GDNDims(n_k=2, n_v=4, dk=64, dv=64, conv_k=4)
    g = torch.Generator().manual_seed(0)
    P = _params(d, g)
    T = 9
    proj = (torch.randn(T, d.proj_out, generator=g)).to(torch.bfloat16)
    pos = torch.arange(T, dtype=torch.int32)
    whole = gdn_reference(proj, pos, torch.zeros(T, dtype=torch.int32), GDNState(d, 2, "cpu"), d, eps=1e-6, **P)
    st = GDNState(d, 2, "cpu")
    parts = [gdn_reference(proj[a:b], pos[a:b], torch.ones(b - a, dtype=torch.int32), st, d, eps=1e-6, **P)
             for a, b in ((0, 4), (4, 5), (5, 9))]
    assert torch.allclose(torch.cat(parts), whole, atol=1e-5)
    # two slots interleaved in one batch behave like two separate sequences
    st2 = GDNState(d, 2, "cpu")
    both = gdn_reference(torch.cat([proj[:3], proj[:3]]), torch.tensor([0, 1, 2, 0, 1, 2], dtype=torch.int32),
                         torch.tensor([0, 0, 0, 1, 1, 1], dtype=torch.int32), st2, d, eps=1e-6, **P)
    assert torch.allclose(both[:3], whole[:3], atol=1e-5) and torch.allclose(both[3:], whole[:3], atol=1e-5)
    # a new sequence in a used slot starts from zero state
    again = gdn_reference(proj[:3], pos[:3], torch.zeros(3, dtype=torch.int32), st2, d, eps=1e-6, **P)
    assert torch.allclose(again, whole[:3], atol=1e-5)


def test_hybrid_model_prefill_equals_decode_on_cpu():
    cfg = HybridConfig.tiny_hybrid()
    m = HybridModel(cfg, "cpu").init_random(seed=0, search=False)
    assert m.kv_layers == 2 and [L.gdn is not None for L in m.layers] == [True, False, True, False]
    g = torch.Generator().manual_seed(0)
    prompt = torch.randint(0, cfg.vocab, (40,), generator=g).tolist()
    kv = PagedKVCache(m.kv_layers, m.nkv, cfg.head_dim, 16, 2, 512, "cpu")
    out, _ = Engine(m, kv, use_graphs=False, prefill_chunk=16).generate(prompt, 5)
    m.gdn_states = None
    kv2 = PagedKVCache(m.kv_layers, m.nkv, cfg.head_dim, 16, 2, 512, "cpu")
    nxt = Engine(m, kv2, use_graphs=False, prefill_chunk=1000).prefill(0, prompt + out[:3])
    assert nxt == out[3]


@pytest.mark.gpu
def test_gpu_gdn_matches_oracle():
    dev = torch.device("cuda:0")
    for d in (GDNDims(2, 4, 64, 64, 4), GDNDims(2, 4, 128, 128, 4)):
        g = torch.Generator().manual_seed(1)
        P = _params(d, g)
        Pg = {k: v.float().to(dev).contiguous() for k, v in P.items()}
        # batch 1: slot 1 rows 0..5 and slot 0 rows 0..2; batch 2 continues both (state carried), batch 3 restarts slot 1
        batches = [([0, 1, 2, 3, 4, 5, 0, 1, 2], [1] * 6 + [0] * 3), ([6, 3], [1, 0]), ([0, 1, 4], [1, 1, 0])]
        st_c, st_g = GDNState(d, 3, "cpu"), GDNState(d, 3, dev)
        for pos, slot in batches:
            n = len(pos)
            proj = torch.randn(n, d.proj_out, generator=g).to(torch.bfloat16)
            pt, sl = torch.tensor(pos, dtype=torch.int32), torch.tensor(slot, dtype=torch.int32)
            ref = gdn_reference(proj, pt, sl, st_c, d, eps=1e-6, **P)
            out = gdn_forward(proj.to(dev), pt.to(dev), sl.to(dev), st_g, d, eps=1e-6, **Pg).float().cpu()
            assert torch.allclose(out, ref, atol=2e-2, rtol=2e-2), float((out - ref).abs().max())
            assert torch.allclose(st_g.rec.cpu(), st_c.rec, atol=1e-3, rtol=1e-3)
            assert torch.allclose(st_g.conv.cpu(), st_c.conv, atol=1e-6)


@pytest.mark.gpu
def test_gpu_hybrid_model_generates_and_matches_whole_prefill():
    dev = torch.device("cuda:0")
    cfg = HybridConfig.tiny_hybrid()
    m = HybridModel(cfg, dev).init_random(seed=0, search=False)
    g = torch.Generator().manual_seed(0)
    prompt = torch.randint(0, cfg.vocab, (150,), generator=g).tolist()
    kv = PagedKVCache(m.kv_layers, m.nkv, cfg.head_dim, 16, 2, 512, dev)
    eng = Engine(m, kv, use_graphs=True, prefill_chunk=64)
    t1 = eng.prefill(0, prompt)
    h1 = m.last_hidden[-1].float().cpu()
    out, _ = eng.generate(prompt, 8, slot=1)
    m.gdn_states = None
    kv2 = PagedKVCache(m.kv_layers, m.nkv, cfg.head_dim, 16, 2, 512, dev)
    t2 = Engine(m, kv2, use_graphs=False, prefill_chunk=1000).prefill(0, prompt)
    h2 = m.last_hidden[-1].float().cpu()
    cos = torch.nn.functional.cosine_similarity(h1, h2, dim=0)
    assert cos > 0.995, float(cos)            # chunked and whole prefill agree up to attention tile rounding
    assert len(out) == 8 and out[0] == t1
    # the CPU oracle sees the same last hidden state
    from volta_engine_b200.models.util import to_device
    mc = to_device(m, "cpu")
    mc.gdn_states = None
    kvc = PagedKVCache(mc.kv_layers, mc.nkv, cfg.head_dim, 16, 2, 512, "cpu")
    Engine(mc, kvc, use_graphs=False, prefill_chunk=1000).prefill(0, prompt)
    cosc = torch.nn.functional.cosine_similarity(mc.last_hidden[-1].float(), h2, dim=0)
    assert cosc > 0.98, float(cosc)


def _kda_weights(d, hidden, rank, g, device="cpu"):
    from volta_engine_b200.ops.gdn import KDAWeights
    from volta_engine_b200.ops.linear import LinearBF16
    bf = torch.bfloat16

    def lin(n, k, s):
        return LinearBF16((torch.randn(n, k, generator=g) * s).to(bf).to(device))
    return KDAWeights(f_a=lin(rank, hidden, 0.1), f_b=lin(d.n_v * d.dk, rank, 0.3), g_a=lin(rank, hidden, 0.1),
                      g_b=lin(d.n_v * d.dv, rank, 0.3), A_log=torch.log(torch.linspace(0.5, 2.0, d.n_v)).to(device),
                      dt_bias=torch.linspace(-1, 1, d.n_v * d.dk).to(device), norm_w=(torch.rand(d.dv, generator=g) + 0.5).to(device))


def test_kda_statement_per_channel_decay_and_chunking():
    from volta_engine_b200.ops.gdn import kda_forward, kda_reference
    d = GDNDims(2, 2, 64, 64, 4)
    g = torch.Generator().manual_seed(3)
    W = _kda_weights(d, 96, 32, g)
    conv_w = torch.randn(d.conv_dim, d.conv_k, generator=g) * 0.5
    x = torch.randn(7, 96, generator=g).to(torch.bfloat16)
    proj = torch.randn(7, d.proj_out, generator=g).to(torch.bfloat16)
    pos, slot = torch.arange(7, dtype=torch.int32), torch.zeros(7, dtype=torch.int32)
    st = GDNState(d, 1, "cpu")
    whole = kda_forward(proj, x, W, pos, slot, st, d, conv_w, 1e-6).float()
    st2 = GDNState(d, 1, "cpu")
    parts = torch.cat([kda_forward(proj[a:b], x[a:b], W, pos[a:b], slot[a:b], st2, d, conv_w, 1e-6).float() for a, b in ((0, 3), (3, 4), (4, 7))])
    assert torch.allclose(whole, parts, atol=1e-5) and torch.allclose(st.rec, st2.rec, atol=1e-6)
    # one step by hand: a fresh state after the first row is k (x) beta v, and the decay of the second row acts per key channel
    st3 = GDNState(d, 1, "cpu")
    f = W.f_b.forward(W.f_a.forward(x)).float()
    z = W.g_b.forward(W.g_a.forward(x)).float()
    kda_reference(proj[:1], f[:1], z[:1], pos[:1], slot[:1], st3, d, conv_w, W.A_log, W.dt_bias, W.norm_w, 1e-6)
    S1 = st3.rec[0].clone()
    kda_reference(proj[1:2], f[1:2], z[1:2], pos[1:2], slot[1:2], st3, d, conv_w, W.A_log, W.dt_bias, W.norm_w, 1e-6)
    gdec = torch.exp(-5.0 * torch.sigmoid(torch.exp(W.A_log)[:, None] * (f[1].reshape(2, 64) + W.dt_bias.reshape(2, 64))))
    assert float(gdec.min()) > 0.0066 and float(gdec.max()) < 1.0 and float(gdec.std()) > 0.01      # in (e^-5, 1), not one value per head
    assert st3.rec[0].shape == S1.shape and not torch.allclose(st3.rec[0], S1)


@pytest.mark.gpu
def test_gpu_kda_matches_statement():
    from volta_engine_b200.ops.gdn import kda_forward
    dev = torch.device("cuda:0")
    for d in (GDNDims(2, 2, 64, 64, 4), GDNDims(4, 4, 128, 128, 4)):
        g = torch.Generator().manual_seed(5)
        Wc = _kda_weights(d, 256, 64, g)
        g = torch.Generator().manual_seed(5)
        Wg = _kda_weights(d, 256, 64, g, dev)
        conv_w = torch.randn(d.conv_dim, d.conv_k, generator=g) * 0.5
        batches = [([0, 1, 2, 3, 4, 5, 0, 1, 2], [1] * 6 + [0] * 3), ([6, 3], [1, 0]), ([0, 1, 4], [1, 1, 0])]
        st_c, st_g = GDNState(d, 3, "cpu"), GDNState(d, 3, dev)
        for pos, slot in batches:
            n = len(pos)
            proj = torch.randn(n, d.proj_out, generator=g).to(torch.bfloat16)
            x = torch.randn(n, 256, generator=g).to(torch.bfloat16)
            pt, sl = torch.tensor(pos, dtype=torch.int32), torch.tensor(slot, dtype=torch.int32)
            ref = kda_forward(proj, x, Wc, pt, sl, st_c, d, conv_w, 1e-6).float()
            out = kda_forward(proj.to(dev), x.to(dev), Wg, pt.to(dev), sl.to(dev), st_g, d, conv_w.to(dev), 1e-6).float().cpu()
            assert torch.allclose(out, ref, atol=3e-2, rtol=3e-2), float((out - ref).abs().max())
            assert torch.allclose(st_g.rec.cpu(), st_c.rec, atol=2e-3, rtol=2e-3)


def test_hybrid_model_with_kda_mixer_prefill_equals_decode_on_cpu():
    cfg = HybridConfig.tiny_hybrid(linear_mixer="kda", gdn_k_heads=2, gdn_v_heads=2, kda_rank=32)
    m = HybridModel(cfg, "cpu").init_random(seed=2, std=0.05)
    assert "kda" in m.layers[0].gdn and m.layers[1].gdn is None
    kv = PagedKVCache(m.kv_layers, m.nkv, cfg.head_dim, 16, 1, 256, "cpu")
    eng = Engine(m, kv, use_graphs=False, prefill_chunk=16)
    toks = [(5 * i + 1) % 1000 for i in range(40)]
    a, _ = eng.generate(toks, 5)
    m2 = HybridModel(cfg, "cpu").init_random(seed=2, std=0.05)
    kv2 = PagedKVCache(m2.kv_layers, m2.nkv, cfg.head_dim, 16, 1, 256, "cpu")
    b, _ = Engine(m2, kv2, use_graphs=False, prefill_chunk=64).generate(toks, 5)
    assert a == b and len(a) == 5


@pytest.mark.gpu
def test_gpu_hybrid_verify_blocks_roll_back_bit_exactly():
    """A journalled block of 4 rows rolled back to k rows leaves the state that stepping only k rows leaves (same kernel,
    same operands), eager and as a CUDA graph replay; decoding after a rollback equals plain greedy decoding."""
    dev = torch.device("cuda:0")
    cfg = HybridConfig.tiny_hybrid()
    m = HybridModel(cfg, dev).init_random(seed=0, search=False)
    prompt = torch.randint(0, cfg.vocab, (90,), generator=torch.Generator().manual_seed(1)).tolist()

    def fresh(graphs):
        m.gdn_states = None
        kv = PagedKVCache(m.kv_layers, m.nkv, cfg.head_dim, 16, 2, 512, dev)
        return Engine(m, kv, use_graphs=graphs, prefill_chunk=64)

    plain, _ = fresh(True).generate(prompt, 14)
    for graphs in (False, True):
        eng = fresh(graphs)
        assert eng.prefill(0, prompt) == plain[0]
        out, pos = [plain[0]], len(prompt)
        wrong = (plain[3] + 1) % cfg.vocab
        # the same block shape three times so that the third is a graph replay
        for drafts in ([plain[1], wrong, 7], [plain[2], plain[3], wrong], [plain[4], wrong, wrong], [wrong, 1, 2]):
            rows = [out[-1]] + drafts
            toks = eng.step(rows, [pos + i for i in range(len(rows))], [0] * len(rows), journal=True)
            acc = 0
            while acc < len(drafts) and toks[acc] == drafts[acc]:
                acc += 1
            if acc < len(drafts):
                eng.rollback(0, acc + 1)
            out += drafts[:acc] + [toks[acc]]
            pos += acc + 1
        while len(out) < 12:
            out.append(eng.step([out[-1]], [pos], [0])[0])
            pos += 1
        assert out == plain[:len(out)], (graphs, out, plain)
    from volta_engine_b200.ops import kernels as K
    assert K.check_status(dev) == 0


@pytest.mark.parametrize("mixer", ["gdn", "kda", "glm5"])
def test_hybrid_model_tensor_parallel_matches_one_rank(tmp_path, mixer):
    """Linear-attention heads split over two CPU ranks (gloo): the gathered logits equal the single-rank model's to
    rounding (the shards are quantised against the whole matrices' tensor scales)."""
    import os
    import socket
    import subprocess
    import sys
    from volta_engine_b200.runtime.batch import BatchRows, LOGITS_ALL
    here = os.path.dirname(os.path.abspath(__file__))
    s = socket.socket()
    s.bind(("127.0.0.1", 0))
    port = s.getsockname()[1]
    s.close()
    out = str(tmp_path / "tp")
    procs = []
    for r in range(2):
        env = dict(os.environ, RANK=str(r), WORLD_SIZE="2", MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port), OMP_NUM_THREADS="2")
        procs.append(subprocess.Popen([sys.executable, os.path.join(here, "hybrid_tp_worker.py"), out, mixer], env=env,
                                      stdout=subprocess.PIPE, stderr=subprocess.STDOUT))
    for p in procs:
        text, _ = p.communicate(timeout=300)
        assert p.returncode == 0, text.decode()[-3000:]
    parts = [torch.load(f"{out}.{r}", weights_only=True) for r in range(2)]
    if mixer == "glm5":
        from volta_engine_b200.models.glm5 import Glm5NextConfig, Glm5NextModel
        cfg = Glm5NextConfig.tiny_glm5(vocab=256, gdn_k_heads=4, gdn_v_heads=4)
        m = Glm5NextModel(cfg, "cpu").init_random(seed=0, search=False)
        kv = m.make_cache(16, 2, 512)
    else:
        kw = {"linear_mixer": "kda", "gdn_k_heads": 4} if mixer == "kda" else {}
        cfg = HybridConfig.tiny_hybrid(vocab=256, **kw)
        m = HybridModel(cfg, "cpu").init_random(seed=0, search=False)
        kv = PagedKVCache(m.kv_layers, m.nkv, cfg.head_dim, 16, 2, 512, "cpu")
    assert parts[0]["heads"] == (m.dims.n_k // 2, m.dims.n_v // 2)
    toks = torch.randint(0, 256, (40,), generator=torch.Generator().manual_seed(11)).tolist()
    kv.reserve(0, 64)
    outs = []
    for lo, hi in ((0, 30), (30, 34), (34, 35), (35, 40)):
        b = BatchRows.make(toks[lo:hi], list(range(lo, hi)), [0] * (hi - lo), "cpu", LOGITS_ALL, m.nq // m.nkv, prefill=hi - lo > 16)
        outs.append(m.forward(b, kv).float())
    want = torch.cat(outs)
    got = torch.cat([p["logits"] for p in parts], 1)[:, :256]
    cos = torch.nn.functional.cosine_similarity(got, want[:, :256], dim=-1)
    # (a row whose router scores nearly tie may pick another expert under the other summation order: most rows agree
    # to rounding, none is far off)
    assert float(cos.median()) > 0.9995 and float((cos > 0.999).float().mean()) > 0.8 and float(cos.min()) > 0.95, cos
    assert float((got.argmax(-1) == want[:, :256].argmax(-1)).float().mean()) > 0.9


@pytest.mark.gpu
def test_gpu_hybrid_mtp_rounds_on_the_device_roll_back_and_match_plain_greedy():
    from volta_engine_b200.runtime.mtp_runner import MtpRunner
    dev = torch.device("cuda:0")
    cfg = HybridConfig.tiny_hybrid(mtp_layers=1)
    m = HybridModel(cfg, dev).init_random(seed=0, search=False)
    prompt = torch.randint(0, cfg.vocab, (77,), generator=torch.Generator().manual_seed(4)).tolist()

    def fresh():
        m.gdn_states = None
        return Engine(m, PagedKVCache(m.kv_layers, m.nkv, cfg.head_dim, 16, 2, 512, dev), prefill_chunk=64)
    plain, _ = fresh().generate(prompt, 20)
    eng = fresh()
    run = MtpRunner(eng, depth=3)
    assert run._device_round_ok() and not run._device_round_ok(2)
    eng.kv.reserve(0, len(prompt) + 40)
    out, pos = [run.prefill_rows(0, prompt, 0, len(prompt), True)], len(prompt)
    while len(out) < 20:
        new = run.round(0, out[-1], pos)
        out += new
        pos += len(new)
    assert out[:20] == plain[:20], (out, plain)
    assert run._sts[(1, 3)]["graph"] is not None and run.stats["accepted"] < run.stats["proposed"]


def test_hybrid_checkpoint_directory_loads_under_the_checkpoint_names(tmp_path):
    """A directory written under the hybrid checkpoint's tensor names (linear_attn.in_proj_qkv / z / b / a, conv1d, A_log,
    dt_bias, gated norm, out_proj; self_attn.q_proj carrying the output gate per head; dense or routed FFN; mtp.*) loads,
    chunked prefill + decode agree with a whole prefill, and a rank of a two-rank layout holds its heads' slices."""
    from volta_engine_b200.models.factory import TensorSource, load_model
    from volta_engine_b200.models.hybrid import HybridConfig, HybridModel
    from volta_engine_b200.models.hybrid_loader import load_hybrid, save_hybrid_checkpoint
    from volta_engine_b200.parallel.comm import LocalComm
    from volta_engine_b200.runtime.engine import Engine
    from volta_engine_b200.runtime.kv_cache import PagedKVCache
    from util import cos
    for moe in (False, True):
        d = tmp_path / ("moe" if moe else "dense")
        cfg = HybridConfig.tiny_hybrid(mtp_layers=1, norm_bias=1.0, quant="bf16", shared_gate=moe, first_dense_layers=0 if moe else 4,
                                      shared_ffn=256)                    # (a two-rank slice of the shared expert keeps 128 rows)
        t = save_hybrid_checkpoint(d, cfg, seed=3)
        m, hf = load_model(d, device="cpu")
        c = m.cfg
        assert isinstance(m, HybridModel) and ["gdn" if L.gdn is not None else "att" for L in m.layers] == ["gdn", "att", "gdn", "att"]
        assert (c.gdn_k_heads, c.gdn_v_heads, c.rot_dim, c.norm_bias, c.mtp_layers, c.attn_gate) == (2, 4, 32, 1.0, 1, True)
        assert all(L.dense_ffn != moe for L in m.layers) and m.mtp is not None and m.mtp["layer"].kv_index == 2 and m.kv_layers == 3
        P = "model.language_model."
        L0, L1, dm = m.layers[0], m.layers[1], m.dims
        w = L0.gdn["in_proj"].weight.float()
        qkv, z = t[P + "layers.0.linear_attn.in_proj_qkv.weight"].float(), t[P + "layers.0.linear_attn.in_proj_z.weight"].float()
        C = dm.conv_dim
        assert torch.equal(w[:C], qkv) and torch.equal(w[C:C + dm.n_v * dm.dv], z)
        assert torch.equal(w[C + dm.n_v * dm.dv:C + dm.n_v * dm.dv + dm.n_v], t[P + "layers.0.linear_attn.in_proj_b.weight"].float())
        assert torch.equal(L0.gdn["conv_w"], t[P + "layers.0.linear_attn.conv1d.weight"].float().reshape(C, -1))
        hd, nq = c.head_dim, c.n_q
        wq = t[P + "layers.1.self_attn.q_proj.weight"].float().reshape(nq, 2, hd, c.hidden)
        assert torch.equal(L1.qkv.weight.float()[: nq * hd], wq[:, 0].reshape(nq * hd, -1))
        assert torch.equal(L1.gate_proj.weight.float(), wq[:, 1].reshape(nq * hd, -1))
        kv = PagedKVCache(m.kv_layers, m.nkv, hd, 16, 2, 512, "cpu")
        prompt = list(range(5, 45))
        out, _ = Engine(m, kv, use_graphs=False, prefill_chunk=16).generate(prompt, 5)
        m.gdn_states = None
        kv2 = PagedKVCache(m.kv_layers, m.nkv, hd, 16, 2, 512, "cpu")
        assert Engine(m, kv2, use_graphs=False, prefill_chunk=1000).prefill(0, prompt + out[:3]) == out[3]

        class Rank1(LocalComm):
            rank, size = 1, 2
        m1 = load_hybrid(hf, TensorSource(d), "cpu", Rank1())
        d1 = m1.dims
        w1 = m1.layers[0].gdn["in_proj"].weight.float()
        kq, vv = d1.n_k * d1.dk, d1.n_v * d1.dv
        Kf, Vf = dm.n_k * dm.dk, dm.n_v * dm.dv
        assert (d1.n_k, d1.n_v) == (1, 2)
        assert torch.equal(w1[:kq], qkv[kq:2 * kq]) and torch.equal(w1[kq:2 * kq], qkv[Kf + kq:Kf + 2 * kq])
        assert torch.equal(w1[2 * kq:2 * kq + vv], qkv[2 * Kf + vv:2 * Kf + 2 * vv]) and torch.equal(w1[2 * kq + vv:2 * kq + 2 * vv], z[vv:2 * vv])
        assert torch.equal(m1.layers[0].gdn["A_log"], t[P + "layers.0.linear_attn.A_log"][2:4])
        assert torch.equal(m1.layers[1].gate_proj.weight.float(), wq[2:4, 1].reshape(2 * hd, -1))
        assert m1.layers[1].o_proj.weight.shape == (c.hidden, 2 * hd)


def test_flash_next_checkpoint_with_stream_mixers_and_indexer_loads(tmp_path):
    """qwen4_exp directories: the gated residual-stream mixers of every sublayer, the final mixer and the block-sparse
    indexer of the full-attention layers come from the checkpoint; n-gram embedding tensors are refused."""
    from volta_engine_b200.loader.safetensors import write_safetensors
    from volta_engine_b200.models.factory import load_model
    from volta_engine_b200.models.hybrid import HybridConfig
    from volta_engine_b200.models.hybrid_loader import save_hybrid_checkpoint
    from volta_engine_b200.runtime.engine import Engine
    from volta_engine_b200.runtime.kv_cache import PagedKVCache
    cfg = HybridConfig.tiny_hybrid(norm_bias=1.0, quant="bf16", shared_gate=True, first_dense_layers=0, residual="gated", hc_mult=4,
                                   hc_rank=16, qsa=True, shared_ffn=256)
    t = save_hybrid_checkpoint(tmp_path, cfg, seed=4)
    m, hf = load_model(tmp_path, device="cpu")
    c = m.cfg
    assert hf["model_type"] == "qwen4_exp" and (c.residual, c.hc_mult, c.hc_rank, c.qsa) == ("gated", 4, 16, True)
    P = "model.language_model."
    L1 = m.layers[1]
    assert torch.equal(L1.attn_hc.down, t[P + "layers.1.attn_hyper_connection.input_mix_weight_down.weight"])
    assert torch.equal(L1.mlp_hc.inject, t[P + "layers.1.mlp_hyper_connection.block_inject_weight.weight"])
    assert m.final_hc.inject is None and torch.equal(m.final_hc.up, t["model.language_model.hyper_connection_mixer.input_mix_weight_up.weight"])
    assert L1.qsa is not None and m.layers[0].qsa is None
    assert torch.equal(L1.qsa.proj.weight, t[P + "layers.1.self_attn.indexer.index_qk_proj.weight"])
    kv = PagedKVCache(m.kv_layers, m.nkv, c.head_dim, 16, 2, 512, "cpu")
    out, _ = Engine(m, kv, use_graphs=False, prefill_chunk=16).generate(list(range(5, 45)), 4)
    assert len(out) == 4
    write_safetensors(tmp_path / "ple.safetensors", {P + "layers.0.ple.key_proj.weight": torch.zeros(4, 4)})
    with pytest.raises(NotImplementedError):
        load_model(tmp_path, device="cpu")
