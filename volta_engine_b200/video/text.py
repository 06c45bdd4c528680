"""Text tower of the video pipeline: the first ``layers`` decoder layers of a Qwen3-VL-32B-shaped language model (hidden
5120, 64 query / 8 KV heads of 128, MLP 25600) run over the prompt once; the residual stream after the last of them is the
condition the transformer reads. It is the engine's dense GQA decoder (NVFP4 / EXL3 / bf16 linears, tensor parallel like
any other model), run as one prefill with no logits.
Reference: src/video/h3_text.cu (the tower), docs/video.md:156-176 (first 50 decoder layers, resident conversions).
"""
from __future__ import annotations

import torch

from ..models.dense import DenseConfig, DenseModel
from ..runtime.batch import BatchRows, LOGITS_NONE
from ..runtime.kv_cache import PagedKVCache


class H3TextTower:
    def __init__(self, cfg: DenseConfig, device="cpu", comm=None, max_tokens: int = 1024):
        self.cfg, self.device = cfg, torch.device(device)
        self.model = DenseModel(cfg, self.device, comm)
        self.max_tokens = max_tokens
        self.kv = None

    @classmethod
    def qwen3_vl_32b(cls, device="cpu", comm=None, layers: int = 50):
        cfg = DenseConfig(n_layers=layers, hidden=5120, n_q=64, n_kv=8, head_dim=128, ffn=25600, vocab=151936, rope_theta=5e6,
                          qk_norm=True)
        return cls(cfg, device, comm)

    @classmethod
    def tiny(cls, device="cpu", hidden: int = 64, layers: int = 2):
        cfg = DenseConfig(n_layers=layers, hidden=hidden, n_q=2, n_kv=1, head_dim=64, ffn=128, vocab=512, qk_norm=True, quant="bf16")
        return cls(cfg, device)

    def init_random(self, seed: int = 0):
        self.model.init_random(seed=seed)
        return self

    def encode(self, ids: list[int]) -> torch.Tensor:
        """Token ids -> [n, hidden] states after the tower's last layer (before any final norm), bf16 on the device."""
        n = len(ids)
        assert 0 < n <= self.max_tokens
        m = self.model
        if self.kv is None:
            pages = PagedKVCache.pages_for(self.max_tokens) + 2
            self.kv = PagedKVCache(self.cfg.n_layers, m.nkv, self.cfg.head_dim, pages, 1, self.max_tokens, self.device)
        self.kv.release(0)
        self.kv.reserve(0, n + 1)
        b = BatchRows.make(list(ids), list(range(n)), [0] * n, self.device, LOGITS_NONE, m.nq // m.nkv, prefill=n > 16)
        m.forward(b, self.kv)
        return m.last_residual[:n].to(torch.bfloat16)
