"""Image inputs for the vision towers: decode (alpha composited onto white), Qwen2-VL "smart resize" onto the patch
grid, aspect-preserving canvas variant, normalisation and patch extraction in merge-block order.

Plain arithmetic on pixel arrays; the container decoding itself is delegated to Pillow (the reference delegates it
to stb_image). Reference: inc/engine/loader/image.h:10-62, src/loader/image.cpp.
"""
from __future__ import annotations

import hashlib
import io
import math
from dataclasses import dataclass, field

import numpy as np
import torch


@dataclass
class VisionParams:
    patch_size: int = 16
    merge_size: int = 2
    temporal_patch_size: int = 2
    min_pixels: int = 65536
    max_pixels: int = 1048576
    canvas: bool = False            # aspect-preserving resize onto a zero-padded canvas instead of the warp
    mean: tuple = (0.5, 0.5, 0.5)
    std: tuple = (0.5, 0.5, 0.5)

    @classmethod
    def from_config(cls, pre: dict, vision: dict | None = None):
        vision = vision or {}
        size = pre.get("size") or {}
        return cls(patch_size=pre.get("patch_size", vision.get("patch_size", 16)),
                   merge_size=pre.get("merge_size", vision.get("spatial_merge_size", 2)),
                   temporal_patch_size=pre.get("temporal_patch_size", vision.get("temporal_patch_size", 2)),
                   min_pixels=pre.get("min_pixels", size.get("shortest_edge", 65536)),
                   max_pixels=pre.get("max_pixels", size.get("longest_edge", 1048576)),
                   mean=tuple(pre.get("image_mean", (0.5, 0.5, 0.5))), std=tuple(pre.get("image_std", (0.5, 0.5, 0.5))))


@dataclass
class PreparedImage:
    grid_h: int
    grid_w: int
    patches: torch.Tensor           # [grid_h * grid_w, 3 * temporal * patch * patch] fp32, merge-block order
    hash: str = ""

    def num_patches(self) -> int:
        return self.grid_h * self.grid_w

    def tokens(self, merge_size: int) -> int:
        return self.num_patches() // (merge_size * merge_size)


def decode_image(data: bytes) -> np.ndarray:
    """JPEG / PNG / BMP / GIF (first frame) bytes -> uint8 [H, W, 3]; alpha is composited onto white."""
    from PIL import Image
    im = Image.open(io.BytesIO(data))
    im.seek(0)
    if im.mode in ("RGBA", "LA", "P") or "transparency" in im.info:
        rgba = im.convert("RGBA")
        bg = Image.new("RGBA", rgba.size, (255, 255, 255, 255))
        im = Image.alpha_composite(bg, rgba).convert("RGB")
    else:
        im = im.convert("RGB")
    return np.asarray(im, dtype=np.uint8)


def smart_resize(height: int, width: int, factor: int, min_pixels: int, max_pixels: int) -> tuple[int, int]:
    """Dimensions rounded to multiples of ``factor`` with the area inside [min_pixels, max_pixels], aspect kept as
    closely as the rounding allows."""
    if min(height, width) <= 0:
        raise ValueError("empty image")
    if max(height, width) / min(height, width) > 200:
        raise ValueError("aspect ratio above 200")
    h = max(factor, round(height / factor) * factor)
    w = max(factor, round(width / factor) * factor)
    if h * w > max_pixels:
        beta = math.sqrt(height * width / max_pixels)
        h = max(factor, math.floor(height / beta / factor) * factor)
        w = max(factor, math.floor(width / beta / factor) * factor)
    elif h * w < min_pixels:
        beta = math.sqrt(min_pixels / (height * width))
        h = math.ceil(height * beta / factor) * factor
        w = math.ceil(width * beta / factor) * factor
    return h, w


def canvas_size(height: int, width: int, factor: int, min_pixels: int, max_pixels: int) -> tuple[int, int, int, int]:
    """Aspect-preserving variant: -> (canvas_h, canvas_w, image_h, image_w); the image is scaled uniformly to fit
    the pixel budget and the canvas is its size rounded up to multiples of ``factor``."""
    area = height * width
    scale = 1.0
    if area > max_pixels:
        scale = math.sqrt(max_pixels / area)
    elif area < min_pixels:
        scale = math.sqrt(min_pixels / area)
    ih, iw = max(1, int(height * scale)), max(1, int(width * scale))
    ch, cw = math.ceil(ih / factor) * factor, math.ceil(iw / factor) * factor
    while ch * cw > max_pixels and (ch > factor or cw > factor):       # rounding up may step over the budget
        if ch >= cw and ch > factor:
            ch -= factor
        else:
            cw -= factor
        ih, iw = min(ih, ch), min(iw, cw)
    return ch, cw, ih, iw


def _resize_bicubic(rgb: np.ndarray, h: int, w: int) -> np.ndarray:
    from PIL import Image
    return np.asarray(Image.fromarray(rgb).resize((w, h), resample=Image.BICUBIC), dtype=np.uint8)


def prepare_image(rgb: np.ndarray, p: VisionParams) -> PreparedImage:
    H, W = rgb.shape[:2]
    factor = p.patch_size * p.merge_size
    if p.canvas:
        ch, cw, ih, iw = canvas_size(H, W, factor, p.min_pixels, p.max_pixels)
        img = np.zeros((ch, cw, 3), dtype=np.float32)
        small = _resize_bicubic(rgb, ih, iw).astype(np.float32) / 255.0
        img[:ih, :iw] = (small - np.asarray(p.mean, dtype=np.float32)) / np.asarray(p.std, dtype=np.float32)
        h, w = ch, cw
    else:
        h, w = smart_resize(H, W, factor, p.min_pixels, p.max_pixels)
        img = _resize_bicubic(rgb, h, w).astype(np.float32) / 255.0
        img = (img - np.asarray(p.mean, dtype=np.float32)) / np.asarray(p.std, dtype=np.float32)
    t = torch.from_numpy(img).permute(2, 0, 1).contiguous()                # [3, h, w]
    gh, gw, ps, ms, tp = h // p.patch_size, w // p.patch_size, p.patch_size, p.merge_size, p.temporal_patch_size
    frames = t[None].expand(tp, 3, h, w)                                   # a still image repeats along time
    x = frames.reshape(tp, 3, gh // ms, ms, ps, gw // ms, ms, ps)
    x = x.permute(2, 5, 3, 6, 1, 0, 4, 7)                                  # [gh/ms, gw/ms, ms, ms, C, T, ps, ps]
    patches = x.reshape(gh * gw, 3 * tp * ps * ps).contiguous()
    digest = hashlib.blake2b(rgb.tobytes() + bytes([gh & 255, gh >> 8, gw & 255, gw >> 8]), digest_size=8).hexdigest()
    return PreparedImage(gh, gw, patches, digest)
