"""Hessian accumulation for calibration: H += X^T X over batches of layer inputs (fp32 accumulator).

The product runs on the tcgen05 GEMM (bf16 operands, fp32 accumulation): with W = X^T as the weight operand and X^T as
the activation operand, out[a, b] = sum_t X[t, a] X[t, b]. Rows are zero-padded to a multiple of 64 (the GEMM's k tile).
Reference: src/backend/cuda/modules/hessian.cu (``transpose_pad_kernel`` + GEMM).
"""
from __future__ import annotations

import torch

from . import kernels as K


class HessianAccumulator:
    def __init__(self, features: int, device):
        self.features = features
        self.H = torch.zeros(features, features, dtype=torch.float32, device=device)
        self.rows = 0

    def add(self, x: torch.Tensor):
        """x [rows, features] (any float dtype)."""
        rows = x.shape[0]
        if not x.is_cuda:
            xf = x.float()
            self.H += xf.t() @ xf
        else:
            pad = (rows + 63) // 64 * 64
            xt = torch.zeros(self.features, pad, dtype=torch.bfloat16, device=x.device)
            xt[:, :rows] = x.to(torch.bfloat16).t()
            self.H += K.gemm_bf16(xt, xt, out_f32=True)
        self.rows += rows
        return self

    def mean(self) -> torch.Tensor:
        return self.H / max(1, self.rows)


# ------------------------------------------------------------------------------------------------ capture files
MAGIC = 0x48455353          # "SSEH" little-endian: the capture file's first word


def write_hessian(path, H: torch.Tensor, rows: int) -> None:
    """One capture file: int32 magic, int32 k, int64 rows, then k*k fp32 (the SUM of x^T x, not the mean).
    Reference: inc/engine/modules/hessian.h:22-24 (same layout, so captures of either engine can be compared)."""
    import struct
    k = H.shape[0]
    with open(path, "wb") as f:
        f.write(struct.pack("<iiq", MAGIC, k, int(rows)))
        f.write(H.detach().to("cpu", torch.float32).contiguous().numpy().tobytes())


def read_hessian(path):
    """-> (H [k, k] fp32 sum, rows) or None when the file is missing, short or not a capture."""
    import os
    import struct
    import numpy as np
    try:
        with open(path, "rb") as f:
            hdr = f.read(16)
            if len(hdr) != 16:
                return None
            magic, k, rows = struct.unpack("<iiq", hdr)
            if magic != MAGIC or k <= 0 or rows <= 0 or os.path.getsize(path) < 16 + 4 * k * k:
                return None
            h = np.frombuffer(f.read(4 * k * k), dtype=np.float32).reshape(k, k)
        return torch.from_numpy(h.copy()), rows
    except OSError:
        return None


def site_file(layer: int, site: int, rank: int = 0) -> str:
    return f"L{layer:02d}_s{site}_r{rank}.f32"


# capture sites of a decoder layer (the reference's numbering, src/models/qwen3_5.cpp:678-906)
SITE_ATTN_IN, SITE_FFN_IN, SITE_ATTN_OUT, SITE_FFN_MID, SITE_HEAD = 0, 1, 2, 3, 4
_SITE_OF = (("q_proj", 0), ("k_proj", 0), ("v_proj", 0), ("qkv", 0), ("gate_proj", 1), ("up_proj", 1), ("gate_up", 1),
            ("o_proj", 2), ("out_proj", 2), ("down_proj", 3), ("lm_head", 4))


def site_of_tensor(name: str):
    """Tensor name -> (layer, site) of the capture that holds its input's Hessian, or None. ``lm_head`` is (0, 4)."""
    import re
    site = next((s for key, s in _SITE_OF if key in name), None)
    if site is None:
        return None
    if site == SITE_HEAD:
        return 0, SITE_HEAD
    m = re.search(r"layers\.(\d+)\.", name)
    return (int(m.group(1)), site) if m else None


class HessianSet:
    """Accumulators of one model: ``stride`` sites per layer, each a k x k fp32 sum over the prefill rows that ran.

    A model declares the sites of this rank with ``add``; ``accumulate`` ignores undeclared sites, layers outside the
    chosen range and row counts below ``min_rows`` (decode steps and drafter blocks are not calibration rows).
    ``dump`` writes one file per site that saw rows. Reference: inc/engine/modules/hessian.h:25-77 (HessianSet)."""

    def __init__(self, layers: int, stride: int = 5, min_rows: int = 17, layer_range=None):
        self.layers, self.stride, self.min_rows = layers, stride, min_rows
        self.range = layer_range or (0, layers)
        self.sites: dict[tuple[int, int], HessianAccumulator] = {}
        self.enabled = True

    def on(self) -> bool:
        return bool(self.sites)

    def add(self, layer: int, site: int, k: int, device) -> None:
        if self.range[0] <= layer < self.range[1] or site == SITE_HEAD:
            self.sites[(layer, site)] = HessianAccumulator(k, device)

    def accumulate(self, layer: int, site: int, x: torch.Tensor) -> None:
        if not self.enabled or x.shape[0] < self.min_rows:
            return
        acc = self.sites.get((layer, site))
        if acc is None:
            return
        if acc.features != x.shape[1]:
            raise ValueError(f"hessian site L{layer} s{site}: width {x.shape[1]}, declared {acc.features}")
        acc.add(x)

    def dump(self, directory, rank: int = 0) -> list[str]:
        import os
        os.makedirs(directory, exist_ok=True)
        out = []
        for (layer, site), acc in sorted(self.sites.items()):
            if acc.rows == 0:
                continue
            fn = site_file(layer, site, rank)
            write_hessian(os.path.join(directory, fn), acc.H, acc.rows)
            out.append(fn)
        return out


def parse_layer_range(text: str, layers: int):
    """"lo-hi" (inclusive, the reference's ENGINE_HESSIAN_LAYERS form) or "" -> (lo, hi_exclusive)."""
    if not text:
        return 0, layers
    lo, _, hi = text.partition("-")
    return int(lo), (int(hi) + 1 if hi else int(lo) + 1)


def merge_dirs(out_dir, dirs, weights=None) -> list[str]:
    """Sums the capture files that EVERY directory has (Hessian sums and row counts: a calibration mixed by token
    count); ``weights`` rescales each directory's share to that fraction of the total rows instead.
    Reference: tests/tools/hess_compare.cpp (``merge``), tests/tools/hess_merge.py (weighted mixing)."""
    import os
    names = None
    for d in dirs:
        here = {f for f in os.listdir(d) if f.endswith(".f32")}
        names = here if names is None else names & here
    os.makedirs(out_dir, exist_ok=True)
    done = []
    for fn in sorted(names or ()):
        parts = [read_hessian(os.path.join(d, fn)) for d in dirs]
        if any(p is None for p in parts) or len({p[0].shape for p in parts}) != 1:
            continue
        if weights is None:
            H = sum(p[0].double() for p in parts)
            rows = sum(p[1] for p in parts)
        else:
            rows = sum(p[1] for p in parts)
            wsum = float(sum(weights))
            H = sum((p[0].double() / p[1]) * (w / wsum) for p, w in zip(parts, weights)) * rows
        write_hessian(os.path.join(out_dir, fn), H.float(), rows)
        done.append(fn)
    return done
