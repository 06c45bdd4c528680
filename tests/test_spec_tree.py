"""Tree verification: the tree structure, the attention mask against the fp32 oracle, per-node logits equal to linear
runs, branch commit (cache rows moved) and the suffix speculator's tree rounds leaving greedy output unchanged."""
import math

import pytest
import torch

from volta_engine_b200.models.dense import DenseConfig, DenseModel
from volta_engine_b200.ops import kernels as K
from volta_engine_b200.ops import reference as ref
from volta_engine_b200.runtime.engine import Engine
from volta_engine_b200.runtime.generator import Generator, Request
from volta_engine_b200.runtime.kv_cache import PagedKVCache
from volta_engine_b200.runtime.options import Options
from volta_engine_b200.runtime.spec_tree import TokenTree
from volta_engine_b200.runtime.suffix_index import SuffixIndex


class ByteTok:
    eos_ids = [0]

    def decode_bytes(self, ids, skip_special=False):
        return bytes(i & 0xFF for i in ids)

    def encode(self, text, allow_special=True):
        return list(text.encode())


def _engine(m, cfg, dev="cpu", graphs=False):
    return Engine(m, PagedKVCache(cfg.n_layers, m.nkv, cfg.head_dim, 40, 2, 512, dev), use_graphs=graphs, prefill_chunk=32)


def test_tree_structure_masks_and_acceptance():
    t = TokenTree.from_paths(5, [[7, 8], [9, 10, 11], [9, 12], [9, 10, 13, 14]])
    assert t.tokens == [5, 7, 8, 9, 10, 11, 12, 13, 14] and t.parents == [-1, 0, 1, 0, 3, 4, 3, 4, 7]
    assert t.depths == [0, 1, 2, 1, 2, 3, 2, 3, 4]
    assert t.masks[8] == 0b110011001 and t.masks[2] == 0b111 and t.children(3) == [4, 6]
    path, emit = t.accept([9, 0, 0, 10, 13, 0, 0, 99, 0])
    assert path == [0, 3, 4, 7] and emit == [9, 10, 13, 99]
    path, emit = t.accept([1] * 9)
    assert path == [0] and emit == [1]
    c = TokenTree.comb(5, [7, 8, 9], [[7, 20], [21], [9, 22, 23]])
    assert c.tokens[:4] == [5, 7, 8, 9] and sorted(c.tokens[4:]) == [20, 21, 22, 23]
    assert len(TokenTree.from_paths(1, [[i, i + 1, i + 2] for i in range(40)], max_nodes=16)) == 16
    s = SuffixIndex(min_k=1)
    s.extend([1, 2, 3, 1, 2, 4, 1, 2, 5, 9, 1, 2])
    assert s.draft_paths(2, 3) == [[5, 9], [4, 1], [3, 1]] and s.draft(2) == [5, 9]


def _attention_case(dev):
    hd, nq, nkv, pos0, n = 128, 8, 2, 70, 9
    g = torch.Generator().manual_seed(3)
    kpool = torch.randn(6, nkv, 64, hd, generator=g).to(torch.bfloat16).to(dev)
    vpool = torch.randn(6, nkv, 64, hd, generator=g).to(torch.bfloat16).to(dev)
    table = torch.tensor([[3, 1, 4, 0]], dtype=torch.int32, device=dev)
    t = TokenTree.from_paths(5, [[7, 8], [9, 10, 11], [9, 12], [9, 10, 13, 14]])
    q = torch.randn(n, (nq + 2 * nkv) * hd, generator=g).to(torch.bfloat16).to(dev)
    pos = torch.arange(pos0, pos0 + n, dtype=torch.int32, device=dev)
    slot = torch.zeros(n, dtype=torch.int32, device=dev)
    tree = (torch.full((n,), pos0, dtype=torch.int32, device=dev), torch.tensor(t.masks, dtype=torch.int64, device=dev))
    return t, q, pos, slot, table, kpool, vpool, nq, nkv, hd, tree


def test_tree_mask_in_the_oracle_equals_attention_over_the_ancestor_rows_only():
    t, q, pos, slot, table, kpool, vpool, nq, nkv, hd, tree = _attention_case("cpu")
    got = ref.attention(q, pos, slot, table, kpool, vpool, nq, nkv, hd, 0.1, 0, None, None, tree).float()
    pos0 = int(pos[0])
    for i in range(len(t)):
        # a linear sequence holding the prefix and the node's ancestors at consecutive positions gives the same row
        anc = [j for j in range(len(t)) if (t.masks[i] >> j) & 1]
        k2, v2 = kpool.clone(), vpool.clone()
        for d, j in enumerate(anc):
            src, dst = pos0 + j, pos0 + d
            k2[int(table[0, dst // 64]), :, dst % 64] = kpool[int(table[0, src // 64]), :, src % 64]
            v2[int(table[0, dst // 64]), :, dst % 64] = vpool[int(table[0, src // 64]), :, src % 64]
        want = ref.attention(q[i:i + 1], torch.tensor([pos0 + len(anc) - 1], dtype=torch.int32), slot[:1], table, k2, v2, nq, nkv,
                             hd, 0.1).float()
        assert torch.allclose(got[i], want[0], atol=2e-2), i


def test_tree_step_equals_linear_runs_and_commit_continues_like_plain_decoding():
    cfg = DenseConfig.tiny(vocab=256)
    m = DenseModel(cfg, "cpu").init_random(seed=0)
    p = torch.randint(1, 255, (45,), generator=torch.Generator().manual_seed(5)).tolist()
    plain, _ = _engine(m, cfg).generate(p, 10)
    e = _engine(m, cfg)
    assert e.supports_tree and e.prefill(0, p) == plain[0]
    tree = TokenTree.from_paths(plain[0], [[7, 8], [plain[1], plain[2], 9], [plain[1], 11], [plain[1], plain[2], plain[3], 3]])
    tg = e.step_tree(0, len(p), tree)
    for i in range(1, len(tree)):
        anc, j = [], i
        while j > 0:
            anc.append(tree.tokens[j])
            j = tree.parents[j]
        e3 = _engine(m, cfg)
        e3.prefill(0, p)
        rows = [plain[0]] + anc[::-1]
        assert e3.step(rows, [len(p) + k for k in range(len(rows))], [0] * len(rows))[-1] == tg[i]
    path, emit = tree.accept(tg)
    assert emit == plain[1:5] and len(path) == 4
    e.commit_tree(0, len(p), path)
    out, pos = [plain[0]] + emit, len(p) + len(path)
    while len(out) < 10:
        out.append(e.step([out[-1]], [pos], [0])[0])
        pos += 1
    assert out == plain


@pytest.mark.parametrize("dev", ["cpu", pytest.param("cuda", marks=pytest.mark.gpu)])
def test_suffix_tree_rounds_leave_greedy_output_unchanged(dev, monkeypatch):
    """The scheduler's tree rounds: the index proposes three continuations per round (a wrong one first, the right one, one
    that is right for one token), so every round must accept the right branch and the output is the plain greedy output."""
    if dev == "cpu":
        cfg, seed, p = DenseConfig.tiny(vocab=256), 0, torch.randint(1, 255, (45,), generator=torch.Generator().manual_seed(5)).tolist()
    else:       # a model whose greedy tokens have clear margins (block rows and single rows take different kernels)
        cfg, seed, p = DenseConfig(n_layers=3, hidden=512, n_q=4, n_kv=2, head_dim=128, ffn=1024, vocab=2048), 5, list(range(100, 180))
    m = DenseModel(cfg, dev).init_random(seed=seed)
    o = Options.resolve({"max_slots": 2, "prefix_interval": 0}, env={})
    n_out = 24 if dev == "cpu" else 12
    plain = Generator(_engine(m, cfg, dev, graphs=dev != "cpu"), ByteTok(), o, eos_ids=[]).generate(Request(p, max_tokens=n_out, cache_prefix=False))
    want = plain["tokens"]

    def paths(self, depth, width):
        done = len(self.toks) - len(p)                     # tokens generated so far (the next token to feed included)
        right = want[done:done + depth]
        if not right:
            return []
        return [[(right[0] + 1) % 256, 3], right, [right[0], 250]][:width]
    monkeypatch.setattr(SuffixIndex, "draft_paths", paths)
    o2 = Options.resolve({"max_slots": 2, "prefix_interval": 0, "speculator": "suffix", "spec_ctrl": False, "spec_depth": 4,
                          "spec_tree": 3}, env={})
    g = Generator(_engine(m, cfg, dev, graphs=dev != "cpu"), ByteTok(), o2, eos_ids=[])
    spec = g.generate(Request(p, max_tokens=n_out, cache_prefix=False))
    assert spec["tokens"] == want
    ms = g.metrics.spec
    assert ms.get("tree_rounds", 0) >= 2 and ms["tree_nodes"] >= 5 * ms["tree_rounds"] and ms["accepted"] >= 3 * (ms["tree_rounds"] - 1)
    if dev != "cpu":
        assert K.check_status(torch.device(dev)) == 0


@pytest.mark.gpu
def test_gpu_tree_attention_matches_oracle_for_every_kernel_form():
    dev = "cuda"
    t, q, pos, slot, table, kpool, vpool, nq, nkv, hd, tree = _attention_case(dev)
    want = ref.attention(q.cpu(), pos.cpu(), slot.cpu(), table.cpu(), kpool.cpu(), vpool.cpu(), nq, nkv, hd, 1 / math.sqrt(hd), 0,
                         None, None, (tree[0].cpu(), tree[1].cpu())).float()
    ws = K.AttnWorkspace(16, nq, hd, 4, torch.device(dev))
    for nsplit in (1, 2):
        got = K.attention(q, pos, slot, table, kpool, vpool, nq, nkv, hd, 1 / math.sqrt(hd), nsplit=nsplit, ws=ws, tree=tree)
        assert torch.allclose(got.float().cpu(), want, atol=2e-2, rtol=2e-2), nsplit
    plain = K.attention(q, pos, slot, table, kpool, vpool, nq, nkv, hd, 1 / math.sqrt(hd), nsplit=1, ws=ws)
    assert not torch.allclose(plain.float().cpu(), want, atol=2e-2)          # the mask does change the result
    assert K.check_status(torch.device(dev)) == 0


@pytest.mark.gpu
def test_gpu_tree_step_matches_the_cpu_statement_and_plain_decoding():
    from volta_engine_b200.models.util import to_device
    dev = torch.device("cuda:0")
    cfg = DenseConfig(n_layers=3, hidden=512, n_q=4, n_kv=2, head_dim=128, ffn=1024, vocab=2048)
    m = DenseModel(cfg, dev).init_random(seed=5)
    p = list(range(100, 180))
    plain, _ = _engine(m, cfg, dev, True).generate(p, 12)
    e = _engine(m, cfg, dev, True)
    assert e.prefill(0, p) == plain[0]
    tree = TokenTree.from_paths(plain[0], [[7, 8], [plain[1], plain[2], 9], [plain[1], 11], [plain[1], plain[2], plain[3], 3]])
    tg = e.step_tree(0, len(p), tree)
    path, emit = tree.accept(tg)
    assert emit == plain[1:5]
    e.commit_tree(0, len(p), path)
    out, pos = [plain[0]] + emit, len(p) + len(path)
    while len(out) < 12:
        out.append(e.step([out[-1]], [pos], [0])[0])
        pos += 1
    assert out == plain
    mc = to_device(m, "cpu")
    ec = _engine(mc, cfg)
    ec.prefill(0, p)
    tc = ec.step_tree(0, len(p), tree)
    assert sum(int(a == b) for a, b in zip(tc, tg)) >= len(tg) - 1          # (a near tie may flip one node)
