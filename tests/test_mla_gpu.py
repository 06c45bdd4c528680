"""MLA attention (absorbed decode kernel, expanded prefill) and the MTP head against the fp32 CPU statement."""
import pytest
import torch

from volta_engine_b200.models.mla import MLAConfig, MLAModel
from volta_engine_b200.models.util import to_device
from volta_engine_b200.runtime.batch import BatchRows
from volta_engine_b200.runtime.kv_cache import PagedKVCache
from util import cos

pytestmark = pytest.mark.gpu
DEV = "cuda"


def _kv(m, dev):
    return PagedKVCache(m.cfg.n_layers + m.cfg.mtp_layers, 1, 576, 24, 2, 1024, dev, v_head_dim=8)


@pytest.mark.parametrize("heads", [4, 20])
def test_mla_prefill_then_decode_matches_reference(heads):
    cfg = MLAConfig.tiny_mla(n_q=heads)
    mg = MLAModel(cfg, DEV).init_random(seed=5)
    mc = to_device(mg, "cpu")
    mg.ensure_workspace(16, 8)
    kvg, kvc = _kv(mg, DEV), _kv(mc, "cpu")
    prompt = torch.randint(0, cfg.vocab, (150,), generator=torch.Generator().manual_seed(2)).tolist()
    kvg.reserve(0, 256)
    kvc.reserve(0, 256)
    G = 1
    bg = BatchRows.make(prompt, list(range(150)), [0] * 150, DEV, "last", G, prefill=True)
    bc = BatchRows.make(prompt, list(range(150)), [0] * 150, "cpu", "last", G, prefill=True)
    lg, lc = mg.forward(bg, kvg), mc.forward(bc, kvc)
    assert cos(lg.cpu(), lc) > 0.995, "prefill logits"
    # latent cache rows written by both paths agree
    pg = kvg.k[0][kvg.host_table[0, 0].item(), 0, :64].float().cpu()
    pc = kvc.k[0][kvc.host_table[0, 0].item(), 0, :64].float()
    assert cos(pg, pc) > 0.999
    # decode / verify rows through the absorbed kernel, several split factors
    for nsplit in (1, 3):
        ids = [5, 9, 11]
        pos = [150, 151, 152]
        bg2 = BatchRows.make(ids, pos, [0] * 3, DEV, "all", G, nsplit=nsplit)
        bc2 = BatchRows.make(ids, pos, [0] * 3, "cpu", "all", G)
        lg2, lc2 = mg.forward(bg2, kvg), mc.forward(bc2, kvc)
        assert cos(lg2.cpu(), lc2) > 0.995, f"decode logits nsplit={nsplit}"
    from volta_engine_b200.ops import kernels as K
    assert K.check_status(DEV) == 0


def test_mtp_head_matches_reference():
    cfg = MLAConfig.tiny_mla()
    mg = MLAModel(cfg, DEV).init_random(seed=6)
    mc = to_device(mg, "cpu")
    mg.ensure_workspace(16, 8)
    kvg, kvc = _kv(mg, DEV), _kv(mc, "cpu")
    kvg.reserve(0, 64)
    kvc.reserve(0, 64)
    ids, pos = [3, 4, 5, 6], [0, 1, 2, 3]
    g = torch.Generator().manual_seed(0)
    hid = torch.randn(4, cfg.hidden, generator=g).to(torch.bfloat16)
    nxt = torch.tensor([4, 5, 6, 7], dtype=torch.int32)
    bg = BatchRows.make(ids, pos, [0] * 4, DEV, "all", 1, nsplit=2)
    bc = BatchRows.make(ids, pos, [0] * 4, "cpu", "all", 1)
    lg, hg = mg.mtp_forward(nxt.to(DEV), hid.to(DEV), bg, kvg)
    lc, hc = mc.mtp_forward(nxt, hid, bc, kvc)
    assert cos(lg.cpu(), lc) > 0.995 and cos(hg.cpu(), hc) > 0.999


def test_mtp_rounds_run_on_the_device_and_reproduce_plain_greedy():
    """Draft chain + verify step + acceptance count as one graph replay; the host reads one result vector per round."""
    from volta_engine_b200.runtime.engine import Engine
    from volta_engine_b200.runtime.mtp_runner import MtpRunner
    cfg = MLAConfig.tiny_mla(vocab=512)
    m = MLAModel(cfg, DEV).init_random(seed=1)
    prompt = torch.randint(0, cfg.vocab, (77,), generator=torch.Generator().manual_seed(4)).tolist()
    plain, _ = Engine(m, _kv(m, DEV), prefill_chunk=64).generate(prompt, 24)
    eng = Engine(m, _kv(m, DEV), prefill_chunk=64)
    run = MtpRunner(eng, depth=3)
    assert run._device_round_ok()
    eng.kv.reserve(0, len(prompt) + 40)
    tok = run.prefill_rows(0, prompt, 0, len(prompt), True)
    out, pos = [tok], len(prompt)
    while len(out) < 24:
        new = run.round(0, out[-1], pos)
        assert 1 <= len(new) <= 4
        out += new
        pos += len(new)
    assert out[:24] == plain[:24], (out, plain)
    assert run._sts[(1, 3)]["graph"] is not None and run.stats["rounds"] >= 6
    assert run.stats["proposed"] == 3 * run.stats["rounds"]
    # two slots in one joint round: one draft chain and one verify block of 8 rows; each slot continues its own greedy run
    other = torch.randint(0, cfg.vocab, (50,), generator=torch.Generator().manual_seed(9)).tolist()
    plain2, _ = Engine(m, _kv(m, DEV), prefill_chunk=64).generate(other, 16)
    eng2 = Engine(m, _kv(m, DEV), prefill_chunk=64)
    run2 = MtpRunner(eng2, depth=3)
    eng2.kv.reserve(0, len(prompt) + 40)
    eng2.kv.reserve(1, len(other) + 40)
    outs = [[run2.prefill_rows(0, prompt, 0, len(prompt), True)], [run2.prefill_rows(1, other, 0, len(other), True)]]
    poss = [len(prompt), len(other)]
    for _ in range(6):
        news = run2.round_joint([0, 1], [outs[0][-1], outs[1][-1]], poss)
        for j in range(2):
            outs[j] += news[j]
            poss[j] += len(news[j])
    n0, n1 = min(len(outs[0]), len(plain)), min(len(outs[1]), len(plain2))
    assert outs[0][:n0] == plain[:n0] and outs[1][:n1] == plain2[:n1] and n0 >= 7 and n1 >= 7, (outs, plain, plain2)
    assert run2._sts[(2, 3)]["graph"] is not None
    # the survival estimate shortens rounds whose later drafts are never accepted
    run2.adaptive = True
    run2.cond = [0.2, 0.2, 0.2]
    assert run2.round_depth() == 1
    run2.cond = [0.9, 0.9, 0.9]
    assert run2.round_depth() == 3
    from volta_engine_b200.ops import kernels as K
    assert K.check_status(DEV) == 0
