"""E5M2 KV cache: store rounding, attention over the byte cache (decode with one warp and with key-split warps,
split-KV, prefill tiles) against the CPU oracle reading the same bytes, and closeness to the bf16 cache."""
import math

import pytest
import torch

from volta_engine_b200.ops import kernels as K
from volta_engine_b200.ops import reference as ref

pytestmark = pytest.mark.gpu
DEV = torch.device("cuda:0") if torch.cuda.is_available() else None
F8 = torch.float8_e5m2


def _setup(nkv, hd, slots, max_seq, pages, seed=0):
    maxp = (max_seq + 63) // 64
    table = torch.zeros(slots, maxp, dtype=torch.int32)
    perm = torch.randperm(pages - 1, generator=torch.Generator().manual_seed(seed)) + 1
    table.view(-1)[: min(slots * maxp, pages - 1)] = perm[: slots * maxp].int()
    g = torch.Generator().manual_seed(seed + 1)
    kb = (torch.randn(pages, nkv, 64, hd, generator=g) * 0.7).to(torch.bfloat16)
    vb = (torch.randn(pages, nkv, 64, hd, generator=g) * 0.7).to(torch.bfloat16)
    return kb, vb, table


def test_store_rounds_like_the_oracle():
    nq, nkv, hd, rows = 8, 2, 128, 6
    _, _, table = _setup(nkv, hd, 2, 256, 16)
    g = torch.Generator().manual_seed(3)
    qkv = torch.randn(rows, (nq + 2 * nkv) * hd, generator=g).to(torch.bfloat16)
    pos = torch.tensor([0, 1, 63, 64, 130, 7], dtype=torch.int32)
    slot = torch.tensor([0, 0, 0, 0, 1, 1], dtype=torch.int32)
    kc = torch.zeros(16, nkv, 64, hd, dtype=F8)
    vc = torch.zeros_like(kc)
    qc = qkv.clone()
    ref.rope_store(qc, pos, slot, table, kc, vc, nq, nkv, hd, hd, 1e6, False)
    kg, vg = torch.zeros(16, nkv, 64, hd, dtype=F8, device=DEV), torch.zeros(16, nkv, 64, hd, dtype=F8, device=DEV)
    qg = qkv.clone().to(DEV)
    K.rope_store(qg, pos.to(DEV), slot.to(DEV), table.to(DEV), kg, vg, nq, nkv, hd, hd, 1e6, False)
    assert torch.equal(vg.cpu().view(torch.uint8), vc.view(torch.uint8))
    dk = (kg.cpu().float() - kc.float()).abs()
    assert float(dk.max()) <= 0.26 * float(kc.float().abs().max())       # rotation rounding may flip an E5M2 step
    assert float((dk > 0).float().mean()) < 0.02


@pytest.mark.parametrize("hd,nq,nkv", [(128, 40, 8), (256, 16, 2), (64, 8, 2)])
def test_attention_over_the_byte_cache(hd, nq, nkv, monkeypatch):
    kb, vb, table = _setup(nkv, hd, 3, 1024, 64)
    k8, v8 = kb.to(F8), vb.to(F8)
    pos = torch.tensor([0, 63, 64, 500, 1000, 129], dtype=torch.int32)
    slot = torch.tensor([0, 1, 2, 0, 1, -1], dtype=torch.int32)
    rows = pos.numel()
    g = torch.Generator().manual_seed(5)
    q = torch.randn(rows, (nq + 2 * nkv) * hd, generator=g).to(torch.bfloat16)
    scale = 1 / math.sqrt(hd)
    want = ref.attention(q, pos, slot, table, k8, v8, nq, nkv, hd, scale)
    bf = ref.attention(q, pos, slot, table, kb, vb, nq, nkv, hd, scale)
    ws = K.AttnWorkspace(rows, nq, hd, 8, DEV)
    args = (q.to(DEV), pos.to(DEV), slot.to(DEV), table.to(DEV), k8.to(DEV), v8.to(DEV), nq, nkv, hd, scale)
    for warps in (104, 1):
        monkeypatch.setattr(K, "ATTN_DECODE_WARPS", warps)
        for nsplit in (1, 4):
            got = K.attention(*args, nsplit=nsplit, ws=ws).float().cpu()
            assert torch.allclose(got[:5], want[:5].float(), atol=2e-2, rtol=2e-2), (warps, nsplit)
    # the byte cache stays close to the bf16 cache
    cos = torch.nn.functional.cosine_similarity(want[:5].float().flatten(), bf[:5].float().flatten(), dim=0)
    assert cos > 0.99
    # prefill tiles
    n = 100
    ppos = torch.arange(37, 37 + n, dtype=torch.int32)
    pslot = torch.ones(n, dtype=torch.int32)
    pq = torch.randn(n, (nq + 2 * nkv) * hd, generator=g).to(torch.bfloat16)
    tiles = K.make_prefill_tiles([1] * n, nq // nkv, DEV)
    got = K.attention(pq.to(DEV), ppos.to(DEV), pslot.to(DEV), table.to(DEV), k8.to(DEV), v8.to(DEV), nq, nkv, hd, scale,
                      tiles=tiles).float().cpu()
    wantp = ref.attention(pq, ppos, pslot, table, k8, v8, nq, nkv, hd, scale).float()
    assert torch.allclose(got, wantp, atol=3e-2, rtol=3e-2)
    assert K.check_status(DEV) == 0
