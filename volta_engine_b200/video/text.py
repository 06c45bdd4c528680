"""Text tower of the video pipeline: the first ``layers`` decoder layers of a Qwen3-VL-32B-shaped language model (hidden
5120, 64 query / 8 KV heads of 128, MLP 25600) run over the prompt once; the residual stream after the last of them is the
condition the transformer reads. It is the engine's dense GQA decoder (NVFP4 / EXL3 / bf16 linears, tensor parallel like
any other model), run as one prefill with no logits.

Captions: a tower built with all its layers (``encode_layers`` below the layer count) also writes text. ``encode`` then
reads the residual stream after layer ``encode_layers`` while the rest of the stack runs on; ``generate`` prefills a chat
prompt (image rows from the vision front end when there is one), keeps its keys and values in the paged cache and decodes
one row per token, greedy or sampled from the top candidates (temperature 0.7, top-k 20, top-p 0.8 by default), until an
end token or ``max_new`` tokens. :class:`H3Captioner` builds the prompt (a fixed instruction, or the user's idea to be kept
and filled in with what the picture shows) and returns one paragraph.
Reference: src/video/h3_text.cu (the tower), docs/video.md:156-176 (first 50 decoder layers, resident conversions),
:177-193 (captions: the last 14 layers, head and cache; sampling settings; 400 tokens; prompt wording).
"""
from __future__ import annotations

import torch

from ..models.dense import DenseConfig, DenseModel
from ..runtime.batch import BatchRows, LOGITS_NONE
from ..runtime.kv_cache import PagedKVCache


class _ResidualTap:
    """Stands where a block drafter's tap ring would: keeps the residual stream after one layer of a forward."""

    def __init__(self, layer: int):
        self.index, self.rows = {layer: 0}, None

    def publish(self, li, h, pos, slot, n):
        self.rows = h[:n].clone()


class H3TextTower:
    def __init__(self, cfg: DenseConfig, device="cpu", comm=None, max_tokens: int = 1024, encode_layers: int = 0):
        self.cfg, self.device = cfg, torch.device(device)
        self.model = DenseModel(cfg, self.device, comm)
        self.max_tokens = max_tokens
        self.kv = None
        # 0 or the layer count: the tower ends where the condition is read. Less: the layers past it exist for captions
        self.encode_layers = encode_layers if 0 < encode_layers < cfg.n_layers else cfg.n_layers
        self._engine = None

    @classmethod
    def qwen3_vl_32b(cls, device="cpu", comm=None, layers: int = 50, captioner: bool = False):
        """The tower's first ``layers`` decoder layers; with ``captioner`` all 64 (the condition is still read after
        ``layers``)."""
        cfg = DenseConfig(n_layers=64 if captioner else layers, hidden=5120, n_q=64, n_kv=8, head_dim=128, ffn=25600, vocab=151936,
                          rope_theta=5e6, qk_norm=True)
        return cls(cfg, device, comm, max_tokens=8192 if captioner else 1024, encode_layers=layers)

    @classmethod
    def tiny(cls, device="cpu", hidden: int = 64, layers: int = 2, captioner: bool = False):
        cfg = DenseConfig(n_layers=layers + (1 if captioner else 0), hidden=hidden, n_q=2, n_kv=1, head_dim=64, ffn=128, vocab=512,
                          qk_norm=True, quant="bf16")
        return cls(cfg, device, encode_layers=layers)

    @property
    def can_generate(self) -> bool:
        return self.encode_layers < self.cfg.n_layers

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
        if not self.can_generate:
            m.forward(b, self.kv)
            return m.last_residual[:n].to(torch.bfloat16)
        tap = _ResidualTap(self.encode_layers - 1)
        had = getattr(m, "tap_ring", None)
        m.tap_ring = tap
        try:
            m.forward(b, self.kv)
        finally:
            m.tap_ring = had
        return tap.rows.to(torch.bfloat16)

    def generate(self, ids: list[int], max_new: int = 400, eos_ids=(), mm=None, temperature: float = 0.0, top_k: int = 20,
                 top_p: float = 0.8, seed: int = 0, forced: list[int] | None = None) -> list[int]:
        """Continue the prompt ``ids`` (``mm``: its image rows, a ``runtime.multimodal.MmPrompt``). ``temperature`` 0 is
        greedy; otherwise a token is drawn from the top candidates of every step. ``forced``: tokens the answer starts
        with (they are decoded one row at a time like generated ones). Returns the new tokens (forced ones included)."""
        import random
        from ..runtime.engine import Engine
        assert self.can_generate, "this tower was built without the layers past the condition tap, the final norm and the head"
        n = len(ids)
        assert 0 < n + max_new <= self.max_tokens
        if self.kv is None:
            pages = PagedKVCache.pages_for(self.max_tokens) + 2
            self.kv = PagedKVCache(self.cfg.n_layers, self.model.nkv, self.cfg.head_dim, pages, 1, self.max_tokens, self.device)
        if self._engine is None:
            self._engine = Engine(self.model, self.kv, use_graphs=False, prefill_chunk=2048)
        eng, rng = self._engine, random.Random(seed)
        self.kv.release(0)
        eos, forced = set(eos_ids), list(forced or [])
        first = eng.prefill(0, list(ids), mm=mm)
        out, pos = [], n

        def pick(greedy_tok, cands):
            if forced:
                return forced.pop(0)
            if temperature <= 0 or cands is None:
                return greedy_tok
            pairs = sorted(zip(cands.logits, cands.ids), reverse=True)[:max(1, top_k)]      # (the engine returns the top 16)
            mx = pairs[0][0]
            w = [pow(2.718281828459045, (v - mx) / temperature) for v, _ in pairs]
            tot, acc, keep = sum(w), 0.0, 0
            for x in w:                                   # smallest prefix holding top_p of the mass
                acc += x
                keep += 1
                if acc >= top_p * tot:
                    break
            r, acc = rng.random() * sum(w[:keep]), 0.0
            for x, (_, t) in zip(w[:keep], pairs):
                acc += x
                if r <= acc:
                    return t
            return pairs[keep - 1][1]
        tok = pick(first, None)               # (the first token comes from the prefill's arg-max unless forced)
        while True:
            out.append(tok)
            if tok in eos or len(out) >= max_new:
                break
            if temperature > 0 and not forced:
                c = eng.step_candidates([tok], [pos], [0])[0]
                tok = pick(c.ids[0], c)
            else:
                tok = pick(eng.step([tok], [pos], [0])[0], None)
            pos += 1
        return out


CAPTION_INSTRUCTION = ("Describe this picture as a detailed prompt for a video generator, in one paragraph: the subject, what it "
                       "wears or looks like, the setting, the light and the colors, and how the camera sees it.")
CAPTION_WITH_IDEA = ("The user's idea for the video: {idea}\nKeep this idea and fill it in with what the picture shows (subject, "
                     "clothing, setting, light and colors, camera), as one detailed paragraph.")


class H3Captioner:
    """Turns a picture (and optionally the text already in the prompt box) into a detailed video prompt with the text
    tower. ``tokenize`` / ``detokenize`` map text to ids and back; ``frontend`` (``runtime.multimodal.MultimodalFrontend``)
    turns image bytes into embedding rows, ``image_token_id`` is the placeholder the chat prompt carries for them."""

    def __init__(self, tower: H3TextTower, tokenize, detokenize, frontend=None, image_token_id: int | None = None,
                 eos_ids=(), max_new: int = 400):
        assert tower.can_generate, "captions need a tower with all its layers and the head"
        self.tower, self.tokenize, self.detokenize = tower, tokenize, detokenize
        self.frontend, self.image_token_id, self.eos_ids, self.max_new = frontend, image_token_id, tuple(eos_ids), max_new

    @staticmethod
    def instruction(idea: str = "") -> str:
        idea = " ".join(idea.split())
        return CAPTION_WITH_IDEA.format(idea=idea) if idea else CAPTION_INSTRUCTION

    def chat(self, idea: str, with_image: bool) -> str:
        pic = "<|vision_start|><|image_pad|><|vision_end|>" if with_image else ""
        return f"<|im_start|>user\n{pic}{self.instruction(idea)}<|im_end|>\n<|im_start|>assistant\n"

    def caption(self, image: bytes | None, idea: str = "", greedy: bool = False, seed: int = 0) -> str:
        ids, mm = self.tokenize(self.chat(idea, image is not None and self.frontend is not None)), None
        if image is not None and self.frontend is not None:
            from ..runtime.multimodal import MmPrompt
            ids, layout, feats = self.frontend.prepare(ids, [image])
            mm = MmPrompt.build(layout, feats)
        room = self.tower.max_tokens - len(ids)
        if room < 8:
            raise ValueError(f"the picture and the prompt take {len(ids)} of the tower's {self.tower.max_tokens} rows")
        out = self.tower.generate(ids, min(self.max_new, room), self.eos_ids, mm=mm, temperature=0.0 if greedy else 0.7, seed=seed)
        if out and out[-1] in self.eos_ids:
            out = out[:-1]
        return " ".join(self.detokenize(out).split())
