"""DSpark: the block drafter of the DeepSeek-V4.1-style model.

Three small decoder stages (window-only attention, their own routed experts, the four hyper-connection streams) entered
through the trunk: the stream means at the entry of the target layers are kept for the last positions of every slot
(tap ring), projected and normalised into one row per committed position, and every stage derives its window KV from
that row. A round for the anchor token at ``pos`` (not yet forwarded by the trunk) runs the block
[anchor, noise, noise, ...] at positions pos .. pos + B - 1; its rows are not causal among themselves: each sees the last
128 committed positions and the whole block. The head is the trunk's, biased token by token by a low-rank bigram
("Markov") head of the previously chosen token, so the B drafts come from one forward plus a short sequential argmax
chain; a confidence head over [hidden, bigram embedding] gives a logit per draft and the round keeps the drafts up to the
first whose sigmoid falls below the threshold.

Reference: src/runtime/dspark_runner.cpp (round, confidence cut at :94), inc/engine/models/model.h:335-346 (dspark_forward /
dspark_chain contract), inc/engine/modules/dsv4.h:78-92 (taps, block attention); the arithmetic is DeepSeek's public model.
Single rank (the trunk's vocabulary shards would have to be gathered for the chain on more).
"""
from __future__ import annotations

import copy
import math
from dataclasses import dataclass

import torch

from ..models.dsv4 import DSV4Model
from ..ops import dsv4 as V
from ..ops import kernels as K
from ..ops import streams as S
from ..ops.linear import LinearBF16
from .batch import BatchRows, LOGITS_ALL
from .dflash_runner import TapRing


@dataclass
class DSparkConfig:
    block_size: int = 5
    noise_token_id: int = 0
    target_layer_ids: tuple = ()
    stages: int = 3
    markov_rank: int = 256
    n_experts: int = 128
    top_k: int = 3
    conf_threshold: float = 0.5
    tap_cap: int = 256

    @classmethod
    def from_hf(cls, c: dict, conf_threshold: float = 0.5):
        return cls(block_size=int(c.get("dspark_block_size", 5)), noise_token_id=int(c.get("dspark_noise_token_id", 0)),
                   target_layer_ids=tuple(c.get("dspark_target_layer_ids", ())), stages=int(c.get("n_mtp_layers", 3)),
                   markov_rank=int(c.get("dspark_markov_rank", 256)), n_experts=int(c.get("dspark_n_routed_experts", 128)),
                   top_k=int(c.get("dspark_n_activated_experts", 3)), conf_threshold=conf_threshold)


class DSparkRunner:
    def __init__(self, engine, cfg: DSparkConfig, seed: int = 21):
        tgt = engine.model
        assert isinstance(tgt, DSV4Model) and engine.comm.size == 1
        self.e, self.cfg = engine, cfg
        dev, tc = engine.device, tgt.cfg
        dcfg = copy.copy(tc)
        dcfg.n_layers, dcfg.compress_ratios = cfg.stages, (0,) * cfg.stages
        dcfg.kv_sources = dcfg.index_sources = dcfg.engram_layers = ()
        dcfg.candidate_source, dcfg.n_experts, dcfg.top_k = -1, cfg.n_experts, cfg.top_k
        self.model = DSV4Model(dcfg, dev).init_random(seed=seed)
        self.model.embed, self.model.lm_head, self.model.vocab_local = tgt.embed, tgt.lm_head, tgt.vocab_local   # shared with the trunk
        self.ring = TapRing(engine.kv.max_slots, cfg.tap_cap, cfg.target_layer_ids, tc.hidden, dev)
        tgt.tap_ring = self.ring
        g = torch.Generator().manual_seed(seed + 1)
        H, R, bf = tc.hidden, cfg.markov_rank, torch.bfloat16
        self.main_proj = LinearBF16((torch.randn(H, self.ring.n * H, generator=g) * 0.02).to(bf).to(dev))
        self.main_norm = torch.ones(H, dtype=bf, device=dev)
        self.markov_embed = (torch.randn(tc.vocab, R, generator=g) * 0.05).to(bf).to(dev)
        self.markov_head = LinearBF16((torch.randn(tgt.vocab_local, R, generator=g) * 0.05).to(bf).to(dev))
        self.conf_w = (torch.randn(H + R, generator=g) / math.sqrt(H + R)).to(dev)
        self.ingested = [0] * engine.kv.max_slots
        self.stats = {"rounds": 0, "proposed": 0, "kept": 0}

    def release(self, slot: int) -> None:
        self.ingested[slot] = 0

    # ---- window KV of every stage for the committed positions [ingested, upto), derived from their taps
    def ingest(self, slot: int, upto: int) -> int:
        lo = max(self.ingested[slot], upto - V.WINDOW, upto - self.cfg.tap_cap, 0)
        if upto <= lo:
            return 0
        m, eps = self.model, self.model.cfg.rms_eps
        st = m._state(self.e.kv)
        main_x = K.rmsnorm(self.main_proj.forward(self.ring.rows(slot, lo, upto)), self.main_norm, eps, 0.0)
        pos = torch.arange(lo, upto, dtype=torch.int32, device=main_x.device)
        sl = torch.full((upto - lo,), slot, dtype=torch.int32, device=main_x.device)
        for si, L in enumerate(m.layers):
            c0, c1 = L.cols["kv"]
            kv_n = K.rmsnorm(L.x_proj.forward(main_x)[:, c0:c1], L.kv_norm, eps, m.cfg.norm_bias)
            V.window_store(st, si, kv_n, m.rope_plain, sl, pos)
        self.ingested[slot] = upto
        return upto - lo

    # ---- one round: drafts for positions pos + 1 ... (at most block_size), cut by the confidence head
    def draft(self, slot: int, anchor: int, pos: int, depth: int | None = None) -> list[int]:
        drafts, conf = self.draft_block(slot, anchor, pos)
        n = 0
        while n < len(drafts) and 1.0 / (1.0 + math.exp(-conf[n])) >= self.cfg.conf_threshold:
            n += 1
        if depth is not None:
            n = min(n, max(0, depth))
        self.stats["rounds"] += 1
        self.stats["proposed"] += len(drafts)
        self.stats["kept"] += n
        return drafts[:n]

    def draft_block(self, slot: int, anchor: int, pos: int):
        """-> (drafts [B] for positions pos + 1 .. pos + B, confidence logits [B])."""
        cfg, m, dev = self.cfg, self.model, self.e.device
        B = cfg.block_size
        self.ingest(slot, pos)
        ids = [anchor] + [cfg.noise_token_id] * (B - 1)
        b = BatchRows.make(ids, [pos + i for i in range(B)], [slot] * B, dev, LOGITS_ALL, m.nq, nsplit=1)
        m.block_keys = (torch.full((B,), pos + B - 1, dtype=torch.int32, device=dev), V.WINDOW + B)
        try:
            logits = m.forward(b, self.e.kv).float()[:, : m.cfg.vocab]
        finally:
            m.block_keys = None
        # the collapsed, un-normalised hidden rows of the block: input of the confidence head
        fn, base, scale = m.layers[-1].mlp_hc
        hid = S.hc_collapse(m.last_streams, fn, base, scale, 1, m.cfg.hc_eps, rms_eps=m.cfg.rms_eps, pre_in=m.last_pre).collapsed
        tok = torch.tensor([anchor], dtype=torch.long, device=dev)
        out, embeds = [], []
        for i in range(B):                      # sequential bigram-biased argmax; everything stays on the device
            me = self.markov_embed[tok]                                               # [1, R]
            bias = self.markov_head.forward(me, out_f32=True)[:, : m.cfg.vocab]
            tok = (logits[i:i + 1] + bias).argmax(-1)
            out.append(tok)
            embeds.append(me)
        feats = torch.cat((hid.float(), torch.cat(embeds).float()), 1)                # [B, H + R]
        conf = feats @ self.conf_w
        return [int(t) for t in torch.cat(out).tolist()], [float(c) for c in conf.tolist()]
