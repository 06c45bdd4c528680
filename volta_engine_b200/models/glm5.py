"""GLM-5-Next-style assembly: Kimi-delta-attention (KDA) linear mixers on most layers, absorbed multi-head latent
attention with the sparse-attention indexer (DSA) on every ``full_interval``-th layer, routed experts with a sigmoid
router beside a shared expert (the first layers dense), four fp32 hyper-connection residual streams, and the
checkpoint's MTP head. Every part is the one the other families use:

  * KDA mixers, their convolution / recurrent state per slot, the verify-block journal and tensor-parallel head split:
    :class:`.hybrid.HybridModel` (``linear_mixer = "kda"``);
  * latent attention (low-rank query, 512 + 64 latent cache row shared by all heads, absorbed decode kernel, expanded
    prefill) and the indexer that picks a decode row's tokens: :class:`.mla.MLAModel`;
  * experts, router, shared expert, expert tiers: :class:`.moe.MoEModel`; hyper-connection streams and the MTP head:
    :class:`.dense.DenseModel`.

The cache holds one latent row per token for the latent-attention layers only (``kv_layers`` = their count plus the MTP
block); the linear layers keep their state outside the pool. A sequence snapshot is therefore cache pages + recurrent
state, except with the indexer on (its pooled keys live outside the pool), where sequences do not resume from snapshots.

Reference: src/models/glm5_next.cpp:499-552 (layer kinds), :1612-1764 (linear / latent attention blocks), :1766-2308
(forward with streams, experts, MTP); inc/engine/models/glm5_next.h:33-52 (shape: 45 layers of hidden 4096, 11 latent
attention layers, 288 experts top-8 of width 2048, dense width 12288, vocabulary 154880); src/models/glm5_next.cpp:107
(64 heads in all, divided over the ranks).
"""
from __future__ import annotations

from dataclasses import dataclass

from ..runtime.batch import BatchRows
from .hybrid import HybridConfig, HybridLayer, HybridModel
from .mla import MLALayer, MLAModel


@dataclass
class Glm5NextConfig(HybridConfig):
    q_lora_rank: int = 1536
    kv_lora_rank: int = 512
    qk_nope: int = 128
    qk_rope: int = 64
    v_head_dim: int = 128
    dsa: bool = True
    model_type: str = "glm5_next"

    @classmethod
    def glm5_next(cls):
        """The published shape: 45 layers (34 KDA + 11 latent attention), hidden 4096, 64 KDA heads of 128 x 128 (q, k and
        v projections of 8192 rows each), 64 latent-attention heads (192 + 64 query dims, 256 value dims, query rank 1536),
        288 experts top-8 (sigmoid, scaled 2.5) of width 2048 + shared expert, 3 leading dense layers of width 12288, MTP
        head. (The reference's ``kda_heads = 16`` is the per-rank count of its four-GPU layout: 64 / tp,
        src/models/glm5_next.cpp:107.)"""
        return cls(n_layers=45, hidden=4096, n_q=64, n_kv=1, head_dim=576, ffn=12288, vocab=154880, n_experts=288, top_k=8,
                   expert_ffn=2048, shared_ffn=2048, router="sigmoid", router_scale=2.5, first_dense_layers=3,
                   full_interval=4, linear_mixer="kda", gdn_k_heads=64, gdn_v_heads=64, gdn_dk=128, gdn_dv=128, kda_rank=128,
                   attn_gate=False, qk_norm=False, norm_bias=1.0, residual="hc", mtp_layers=1, q_lora_rank=1536, dsa=True,
                   qk_nope=192, v_head_dim=256)

    @classmethod
    def tiny_glm5(cls, **kw):
        c = cls(n_layers=4, hidden=256, n_q=4, n_kv=1, head_dim=576, ffn=512, vocab=1024, n_experts=8, top_k=2, expert_ffn=128,
                shared_ffn=128, router="sigmoid", first_dense_layers=1, full_interval=2, linear_mixer="kda", gdn_k_heads=2,
                gdn_v_heads=2, gdn_dk=64, gdn_dv=64, kda_rank=64, attn_gate=False, qk_norm=False, residual="plain",
                mtp_layers=0, q_lora_rank=128, dsa=False)
        for k, v in kw.items():
            setattr(c, k, v)
        return c


class Glm5NextLayer(HybridLayer):
    __slots__ = tuple(s for s in MLALayer.__slots__)


class Glm5NextModel(HybridModel, MLAModel):
    """Method resolution: HybridModel -> MLAModel -> MoEModel -> DenseModel. The hybrid model decides per layer whether
    the mixer is linear; where it asks its base class for a full-attention layer it gets the latent-attention one."""

    layer_cls = Glm5NextLayer

    @property
    def prefix_resume(self):
        return None if self.cfg.dsa else "kv+state"

    def __init__(self, cfg: Glm5NextConfig, device, comm=None):
        assert not cfg.qsa and not cfg.attn_gate and not cfg.qk_norm, "the latent-attention layers have no gate / indexer of the GQA form"
        super().__init__(cfg, device, comm)

    def _attn_bytes(self, L) -> int:
        if L.gdn is not None:
            return HybridModel._attn_bytes(self, L)
        return MLAModel._attn_bytes(self, L)

    def attn_block(self, li, L, x, b: BatchRows, kv, pbuf):
        if L.gdn is not None:
            return HybridModel.attn_block(self, li, L, x, b, kv, pbuf)
        # latent attention: the cache layer (and the indexer state) is the layer's index among the attention layers
        return MLAModel.attn_block(self, L.kv_index, L, x, b, kv, pbuf)

    def make_cache(self, pages: int, max_slots: int, max_seq: int, **kw):
        """The paged latent cache this model runs on (one 576-wide row per token and attention layer)."""
        from ..runtime.kv_cache import PagedKVCache
        return PagedKVCache(self.kv_layers, 1, 576, pages, max_slots, max_seq, self.device, v_head_dim=8, **kw)
