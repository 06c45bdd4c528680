"""LoRA adapters of the MiniMax-H3 denoiser: PEFT-style A / B pairs kept apart from the INT8 base weights and added to
the four projections of a block (fused q | k | v, attention output, fused gate | up, down) as
``y[:, offset:offset + width] += scale * alpha_scale * (x A^T) B^T``; several adapters at once, each with its own scale
that can change between jobs.

Three key layouts are read:

  * diffusers (the few-step "turbo" adapters): ``transformer_blocks.<n>.attn.to_q|to_k|to_v|to_out.0`` and
    ``ff.net.0.proj|ff.net.2`` with ``.lora_A.default.weight`` [rank, in] / ``.lora_B.default.weight`` [out, rank]; q, k
    and v land at their offsets of the fused projection; alpha from the file's metadata (``"alpha"``, default 8), the
    delta is scaled by alpha / rank;
  * kohya: ``lora_unet_blocks_<n>_attn_qkv_proj.lora_down.weight / .lora_up.weight / .alpha`` (dots of the native names
    as underscores; without an alpha tensor the delta is not rescaled);
  * ai-toolkit: ``diffusion_model.blocks.<n>.attn.qkv_proj.lora_A.weight / .lora_B.weight`` (alpha = rank).

The last two address the fused native projections (``attn.qkv_proj``, ``attn.out_proj``, ``mlp.fc1``, ``mlp.fc2``) whole.
Tensor parallel: a column-parallel projection (q | k | v, gate | up) keeps A and this rank's rows of B per segment; a
row-parallel one (output, down) keeps B and this rank's columns of A, so the partial deltas add up in the block's
all-reduce like the base products.
Reference: src/video/h3_dit.cu:211-226 (parts per layer and slot), :421-430 (application), :643-790 (``add_lora``: key
layouts, alpha, sharding); src/server/video/adapters.h:8-24 (the catalogue); docs/video.md:46.
"""
from __future__ import annotations

import json
import struct
from dataclasses import dataclass, field
from pathlib import Path

import torch

SLOT_QKV, SLOT_OUT, SLOT_FC1, SLOT_FC2 = 0, 1, 2, 3
NATIVE = ("attn.qkv_proj", "attn.out_proj", "mlp.fc1", "mlp.fc2")
MAX_RANK = 256


@dataclass
class LoraPart:
    a: torch.Tensor            # [rank, in] (this rank's columns for a row-parallel projection)
    b: torch.Tensor            # [width, rank] (this rank's rows for a column-parallel projection)
    offset: int                # first output column the delta lands on (local to this rank's projection)
    alpha_scale: float

    @property
    def rank(self) -> int:
        return self.a.shape[0]


@dataclass
class Adapter:
    name: str
    scale: float
    parts: dict = field(default_factory=dict)      # (layer, slot) -> [LoraPart]
    rank: int = 0
    alpha: float = 8.0
    layout: str = ""

    def targets(self) -> int:
        return sum(len(v) for v in self.parts.values())


def apply_lora(adapters: list, layer: int, slot: int, x: torch.Tensor, y: torch.Tensor) -> torch.Tensor:
    """y [rows, out] += the deltas of every active adapter for projection ``slot`` of block ``layer`` on input x."""
    for ad in adapters:
        if ad.scale == 0.0:
            continue
        for p in ad.parts.get((layer, slot), ()):
            t = x.to(p.a.dtype) @ p.a.t()
            d = (t @ p.b.t()).to(y.dtype) * (ad.scale * p.alpha_scale)
            y[:, p.offset:p.offset + p.b.shape[0]] += d
    return y


def _read_header(path) -> dict:
    with open(path, "rb") as f:
        (n,) = struct.unpack("<Q", f.read(8))
        if n > 64 << 20:
            raise ValueError(f"{path}: implausible header length {n}")
        return json.loads(f.read(n))


def detect_layout(names) -> str:
    for n in names:
        if n.startswith("lora_unet_"):
            return "kohya"
        if n.startswith("diffusion_model."):
            return "ai-toolkit"
        if ".lora_A.default.weight" in n or n.startswith("transformer_blocks."):
            return "diffusers"
    return ""


def load_adapter(path, cfg, scale: float = 1.0, tp_rank: int = 0, tp_ranks: int = 1, device="cpu", dtype=torch.bfloat16) -> Adapter:
    """Read an adapter file for a denoiser of shape ``cfg`` (``cfg.layers`` blocks). Raises ValueError when the file has
    no usable target or a pair does not fit."""
    from ..loader.safetensors import SafeTensorsRepo
    repo = SafeTensorsRepo(path)
    hdr = _read_header(path)
    alpha = 8.0
    try:
        alpha = float(hdr.get("__metadata__", {}).get("alpha", 8.0))
    except (TypeError, ValueError):
        pass
    ad = Adapter(name=str(path), scale=float(scale), alpha=alpha, layout=detect_layout(repo.names()))
    qd, F = cfg.heads * cfg.head_dim, cfg.ffn
    T, tr = tp_ranks, tp_rank
    ql, fl = qd // T, F // T

    def scalar(name: str, default: float) -> float:
        if not repo.has(name):
            return default
        t = repo.load(name)
        return float(t.flatten()[0]) if t.numel() else default

    def add(layer: int, slot: int, an: str, bn: str, offset: int, alpha_in: float, alpha_from_rank: bool) -> None:
        if not (repo.has(an) and repo.has(bn)):
            return
        a, b = repo.load(an).to(dtype, copy=True), repo.load(bn).to(dtype, copy=True)      # (own memory: the file is closed below)
        if a.dim() != 2 or b.dim() != 2 or b.shape[1] != a.shape[0] or a.shape[0] > MAX_RANK:
            raise ValueError(f"{path}: pair {an} / {bn} unusable (A {tuple(a.shape)}, B {tuple(b.shape)})")
        rank, width = a.shape[0], b.shape[0]
        asc = 1.0 if alpha_from_rank else alpha_in / rank
        ad.rank = max(ad.rank, rank)
        dst = ad.parts.setdefault((layer, slot), [])
        if T == 1:
            dst.append(LoraPart(a.to(device), b.to(device), offset, asc))
            return
        if rank % 8:
            raise ValueError(f"{path}: tensor-parallel adapters need a rank that is a multiple of 8 (got {rank})")
        if slot in (SLOT_QKV, SLOT_FC1):
            seg, segl = (qd, ql) if slot == SLOT_QKV else (F, fl)
            if offset % seg or width % seg:
                raise ValueError(f"{path}: a tensor-parallel adapter part must cover whole q / k / v (gate / up) segments")
            for g in range(width // seg):
                rows = b[g * seg + tr * segl:g * seg + (tr + 1) * segl]
                dst.append(LoraPart(a.to(device), rows.contiguous().to(device), (offset // seg + g) * segl, asc))
        else:
            K, kl = (qd, ql) if slot == SLOT_OUT else (F, fl)
            if a.shape[1] != K or offset:
                raise ValueError(f"{path}: unexpected adapter shape for a row-parallel projection ({an}: {tuple(a.shape)})")
            dst.append(LoraPart(a[:, tr * kl:(tr + 1) * kl].contiguous().to(device), b.to(device), 0, asc))

    dtargets = (("attn.to_q", SLOT_QKV, 0), ("attn.to_k", SLOT_QKV, qd), ("attn.to_v", SLOT_QKV, 2 * qd),
                ("attn.to_out.0", SLOT_OUT, 0), ("ff.net.0.proj", SLOT_FC1, 0), ("ff.net.2", SLOT_FC2, 0))
    for L in range(cfg.layers):
        dp, np_ = f"transformer_blocks.{L}.", f"blocks.{L}."
        for suffix, slot, off in dtargets:
            add(L, slot, dp + suffix + ".lora_A.default.weight", dp + suffix + ".lora_B.default.weight", off, alpha, False)
        for slot in range(4):
            kohya = ("lora_unet_" + np_ + NATIVE[slot]).replace(".", "_")
            ka = scalar(kohya + ".alpha", -1.0)
            add(L, slot, kohya + ".lora_down.weight", kohya + ".lora_up.weight", 0, ka if ka > 0 else 0.0, ka <= 0)
            add(L, slot, "diffusion_model." + np_ + NATIVE[slot] + ".lora_A.weight",
                "diffusion_model." + np_ + NATIVE[slot] + ".lora_B.weight", 0, 0.0, True)
    repo.close()
    if ad.targets() == 0 or ad.rank <= 0:
        raise ValueError(f"{path}: no usable adapter targets")
    return ad


@dataclass
class AdapterInfo:
    file: str
    path: str
    label: str
    format: str          # diffusers | kohya | ai-toolkit
    task: str            # fl2v | ref2v (turbo) or ref2va (community)
    turbo: bool
    mb: int


class AdapterCatalog:
    """The adapter files of the configured directories. A "turbo" file is a few-step distillation adapter (it fixes the
    step count and the flow shift of a job); reference-to-video turbo adapters are listed only when the reference-to-video
    transformer is configured."""

    def __init__(self):
        self.list: list[AdapterInfo] = []

    def scan(self, dirs, ref2va: bool = False) -> "AdapterCatalog":
        self.list = []
        for d in dirs:
            for p in sorted(Path(d).glob("*.safetensors")):
                try:
                    names = [k for k in _read_header(p) if k != "__metadata__"]
                except (OSError, ValueError):
                    continue
                fmt = detect_layout(names)
                if not fmt:
                    continue
                low = p.name.lower()
                turbo = "turbo" in low
                task = ("ref2v" if "ref2v" in low else "fl2v") if turbo else "ref2va"
                if turbo and task == "ref2v" and not ref2va:
                    continue
                label = p.stem.replace("_", " ")
                self.list.append(AdapterInfo(p.name, str(p), label, fmt, task, turbo, p.stat().st_size >> 20))
        return self

    def find(self, file: str):
        return next((a for a in self.list if a.file == file), None)

    def all(self):
        return list(self.list)
