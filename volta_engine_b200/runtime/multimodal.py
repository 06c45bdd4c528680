"""Multimodal prompt layout: where image spans sit in a token sequence, the three-axis rotary positions they imply, and
the keys that make prefix-cache lookups depend on image content.

Positions (Qwen2-VL scheme): text tokens advance all three axes together; the tokens of an image placed at running
position p0 get (t, h, w) = (p0, p0 + row, p0 + col) over its merged grid; the text after it continues at
p0 + max(rows, cols). The cache index of a token stays its sequence index; only the rotary angle uses these positions, so
after the prompt every decode row rotates with ``sequence index + delta``.
Reference: inc/engine/runtime/multimodal.h (``MmLayout`` / ``MmImage``: image spans, M-RoPE position derivation,
content-hash keys), use in src/runtime/cluster.cpp:273-317.
"""
from __future__ import annotations

import hashlib
from dataclasses import dataclass, field

import torch


@dataclass
class MmImage:
    start: int            # index of the span's first token in the expanded prompt
    rows: int             # merged grid (tokens = rows * cols)
    cols: int
    key: int = 0          # content hash folded to a negative pseudo token id

    @property
    def tokens(self) -> int:
        return self.rows * self.cols


@dataclass
class MmLayout:
    n_tokens: int
    images: list = field(default_factory=list)

    def positions3(self) -> torch.Tensor:
        """int32 [3, n_tokens]: (time, height, width) rotary position of every prompt token."""
        pos = torch.zeros(3, self.n_tokens, dtype=torch.int32)
        run, i = 0, 0
        for im in sorted(self.images, key=lambda m: m.start):
            n_text = im.start - i
            if n_text > 0:
                pos[:, i:im.start] = torch.arange(run, run + n_text, dtype=torch.int32)
                run += n_text
            r = torch.arange(im.rows, dtype=torch.int32).repeat_interleave(im.cols)
            c = torch.arange(im.cols, dtype=torch.int32).repeat(im.rows)
            pos[0, im.start:im.start + im.tokens] = run
            pos[1, im.start:im.start + im.tokens] = run + r
            pos[2, im.start:im.start + im.tokens] = run + c
            run += max(im.rows, im.cols)
            i = im.start + im.tokens
        if i < self.n_tokens:
            pos[:, i:] = torch.arange(run, run + self.n_tokens - i, dtype=torch.int32)
            run += self.n_tokens - i
        self._next = run
        return pos

    def delta(self) -> int:
        """Rotary position of the first generated token minus its sequence index."""
        self.positions3()
        return self._next - self.n_tokens

    def cache_tokens(self, ids: list[int]) -> list[int]:
        """The prompt as the prefix cache sees it: image placeholder tokens replaced by ids derived from the image content,
        so the same text around different images never shares a snapshot."""
        out = list(ids)
        for im in self.images:
            for k in range(im.tokens):
                out[im.start + k] = -(1 + ((im.key + k * 0x9E3779B1) & 0x3FFFFFFF))
        return out


@dataclass
class MmPrompt:
    """What a prefill needs beside the token ids: rotary positions of every prompt token and the embedding rows of the
    image tokens."""
    pos3: torch.Tensor            # int32 [3, N] (host)
    feat_index: torch.Tensor      # int64 [N]: row of ``feats`` for image tokens, -1 for text
    feats: torch.Tensor | None    # [image tokens, H]
    delta: int

    @classmethod
    def build(cls, layout: MmLayout, feats: torch.Tensor | None) -> "MmPrompt":
        idx = torch.full((layout.n_tokens,), -1, dtype=torch.int64)
        k = 0
        for im in sorted(layout.images, key=lambda m: m.start):
            idx[im.start:im.start + im.tokens] = torch.arange(k, k + im.tokens)
            k += im.tokens
        return cls(layout.positions3(), idx, feats, layout.delta())

    def chunk(self, start: int, end: int, device, hidden: int):
        """(pos3 [3, n], embeds [n, H] or None, mask [n] or None) of prompt rows [start, end)."""
        pos3 = self.pos3[:, start:end].contiguous().to(device)
        idx = self.feat_index[start:end]
        m = idx >= 0
        if self.feats is None or not bool(m.any()):
            return pos3, None, None
        emb = torch.zeros(end - start, hidden, dtype=self.feats.dtype, device=device)
        emb[m.to(device)] = self.feats.to(device)[idx[m].to(device)]
        return pos3, emb, m.to(device)


def content_key(data: bytes) -> int:
    return int.from_bytes(hashlib.sha256(data).digest()[:8], "little")


def expand_placeholders(ids: list[int], image_token_id: int, grids: list[tuple[int, int]], raw: list[bytes] | None = None):
    """Every occurrence of ``image_token_id`` (one per image, in order) becomes rows * cols copies.
    Returns (expanded ids, MmLayout)."""
    out, images, k = [], [], 0
    for t in ids:
        if t == image_token_id and k < len(grids):
            r, c = grids[k]
            images.append(MmImage(len(out), r, c, content_key(raw[k]) if raw else k))
            out.extend([image_token_id] * (r * c))
            k += 1
        else:
            out.append(t)
    if k != len(grids):
        raise ValueError(f"{len(grids)} images for {k} image placeholders")
    return out, MmLayout(len(out), images)


class MultimodalFrontend:
    """Turns the images of a request into embedding rows: decode -> smart resize -> patches -> vision tower."""

    def __init__(self, tower, params, image_token_id: int):
        self.tower, self.params, self.image_token_id = tower, params, image_token_id

    def prepare(self, ids: list[int], images: list[bytes]):
        """-> (expanded ids, layout, embeds [sum of image tokens, H] on the tower's device)."""
        from ..loader.image import decode_image, prepare_image
        grids, feats = [], []
        m = self.tower.cfg.merge
        for data in images:
            img = prepare_image(decode_image(data), self.params)
            e = self.tower.forward(torch.as_tensor(img.patches).to(self.tower.device), img.grid_h, img.grid_w)
            grids.append((img.grid_h // m, img.grid_w // m))
            feats.append(e)
        out, layout = expand_placeholders(ids, self.image_token_id, grids, images)
        return out, layout, (torch.cat(feats, 0) if feats else None)
