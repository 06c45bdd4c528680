"""Sharded safetensors repository: mmap'd shards behind one name index, tensor-parallel slicing and the quantised
linear formats (EXL3 trellis, NVFP4 in both checkpoint dialects, FP8 128x128 blocks, dense).

File format: 8-byte little-endian header length, JSON header ``{name: {dtype, shape, data_offsets}}`` (offsets
relative to the end of the header), raw little-endian tensor data.
Reference: inc/engine/loader/safetensors.h:45-351 (``load`` / ``load_slice`` / ``load_linear*`` / ``load_nvfp4*`` /
vocab-shard padding), src/loader/nvfp4.cpp:36-57 (tensor names of the two NVFP4 dialects),
src/loader/safetensors.cpp:456-504 (EXL3 tensors and codebook markers).
"""
from __future__ import annotations

import json
import mmap
import os
import struct
import warnings
from pathlib import Path

import torch

from ..ops.linear import LinearBF16, LinearNVFP4
from ..quant import exl3 as ex

_DTYPES = {
    "F64": torch.float64, "F32": torch.float32, "F16": torch.float16, "BF16": torch.bfloat16,
    "I64": torch.int64, "I32": torch.int32, "I16": torch.int16, "I8": torch.int8, "U8": torch.uint8,
    "BOOL": torch.bool, "F8_E4M3": torch.float8_e4m3fn, "F8_E5M2": torch.float8_e5m2,
    "U16": torch.int16, "U32": torch.int32,          # unsigned code words are handled as their bit patterns
}
_NAMES = {torch.float64: "F64", torch.float32: "F32", torch.float16: "F16", torch.bfloat16: "BF16",
          torch.int64: "I64", torch.int32: "I32", torch.int16: "I16", torch.int8: "I8", torch.uint8: "U8",
          torch.bool: "BOOL", torch.float8_e4m3fn: "F8_E4M3", torch.float8_e5m2: "F8_E5M2"}
MAX_SHARDS = 128


def write_safetensors(path, tensors: dict, metadata: dict | None = None, unsigned16: tuple = ()):
    """Write one shard. Names in ``unsigned16`` (int16 tensors) are tagged U16."""
    header, off = {}, 0
    blobs = []
    for name in sorted(tensors):
        t = tensors[name].detach().cpu().contiguous()
        raw = t.reshape(-1).view(torch.uint8) if t.numel() else torch.empty(0, dtype=torch.uint8)      # (0-dim scalars too)
        n = raw.numel()
        dt = "U16" if name in unsigned16 else _NAMES[t.dtype]
        header[name] = {"dtype": dt, "shape": list(t.shape), "data_offsets": [off, off + n]}
        blobs.append(raw)
        off += n
    if metadata:
        header["__metadata__"] = {str(k): str(v) for k, v in metadata.items()}
    hj = json.dumps(header, separators=(",", ":")).encode()
    hj += b" " * ((8 - len(hj) % 8) % 8)
    with open(path, "wb") as f:
        f.write(struct.pack("<Q", len(hj)))
        f.write(hj)
        for b in blobs:
            f.write(b.numpy().tobytes())


class _Shard:
    def __init__(self, path: Path):
        self.path = path
        self.f = open(path, "rb")
        (hlen,) = struct.unpack("<Q", self.f.read(8))
        if hlen > 1 << 30:
            raise ValueError(f"{path}: implausible header length {hlen}")
        self.header = json.loads(self.f.read(hlen))
        self.base = 8 + hlen
        self.mm = mmap.mmap(self.f.fileno(), 0, access=mmap.ACCESS_READ)
        self.metadata = self.header.pop("__metadata__", {})


class SafeTensorsRepo:
    """All ``*.safetensors`` shards of a model directory (or one file) behind one name -> tensor index."""

    def __init__(self, path):
        p = Path(path)
        files = [p] if p.is_file() else sorted(p.glob("*.safetensors"))
        if not files:
            raise FileNotFoundError(f"no safetensors shards under {p}")
        if len(files) > MAX_SHARDS:
            raise ValueError(f"{len(files)} shards; at most {MAX_SHARDS} are supported")
        self.dir = p if p.is_dir() else p.parent
        self.shards = [_Shard(f) for f in files]
        self.index: dict[str, tuple[int, dict]] = {}
        for si, sh in enumerate(self.shards):
            for name, meta in sh.header.items():
                self.index[name] = (si, meta)
        qc = self.dir / "quantization_config.json"
        self.quant_config = json.loads(qc.read_text()) if qc.exists() else {}
        cfgp = self.dir / "config.json"
        if not self.quant_config and cfgp.exists():
            self.quant_config = json.loads(cfgp.read_text()).get("quantization_config", {}) or {}
        # EXL3 checkpoints may store tiles in the reference engine's own lane order; weights listed as stock keep
        # the exllamav3 order (the GPU kernels consume the stock order; the other order is expanded to bf16 at load)
        self.tile_layout = self.quant_config.get("tile_layout", "stock")
        self.tile_layout_stock = set(self.quant_config.get("tile_layout_stock", []))

    # ------------------------------------------------------------------------------------------ plain tensors
    def names(self):
        return self.index.keys()

    def has(self, name: str) -> bool:
        return name in self.index

    def info(self, name: str):
        meta = self.index[name][1]
        return _DTYPES[meta["dtype"]], tuple(meta["shape"])

    def load(self, name: str, device=None, dtype=None) -> torch.Tensor:
        si, meta = self.index[name]
        sh = self.shards[si]
        lo, hi = meta["data_offsets"]
        dt = _DTYPES[meta["dtype"]]
        shape = tuple(meta["shape"])
        if hi == lo:
            t = torch.empty(shape, dtype=dt)
        else:
            with warnings.catch_warnings():          # read-only mapping: tensors from it are never written to
                warnings.simplefilter("ignore", UserWarning)
                t = torch.frombuffer(sh.mm, dtype=torch.uint8, count=hi - lo, offset=sh.base + lo)
            t = t.view(dt).reshape(shape)
        if dtype is not None and t.dtype != dtype:
            t = t.to(dtype)
        if device is not None:
            t = t.to(device)
        return t

    def load_slice(self, name: str, dim: int, rank: int, world: int, device=None, dtype=None) -> torch.Tensor:
        """Shard ``rank`` of ``world`` equal slices along ``dim`` (only that slice is copied off the mmap)."""
        t = self.load(name)
        n = t.shape[dim]
        if n % world:
            raise ValueError(f"{name}: dim {dim} of size {n} does not split {world} ways")
        per = n // world
        s = t.narrow(dim, rank * per, per).contiguous()
        if dtype is not None:
            s = s.to(dtype)
        return s.to(device) if device is not None else s

    def load_rows_padded(self, name: str, rank: int, world: int, multiple: int = 256, device=None, dtype=None):
        """Vocabulary shard: rows are padded up so each rank owns a multiple of ``multiple`` rows; rows past the
        real table are zero."""
        t = self.load(name)
        rows = t.shape[0]
        per = ((rows + world - 1) // world + multiple - 1) // multiple * multiple
        lo, hi = rank * per, min(rows, (rank + 1) * per)
        out = torch.zeros(per, *t.shape[1:], dtype=dtype or t.dtype)
        if hi > lo:
            out[: hi - lo] = t[lo:hi].to(out.dtype)
        return out.to(device) if device is not None else out

    # ------------------------------------------------------------------------------------------ linear formats
    def linear_kind(self, base: str) -> str | None:
        if self.has(base + ".trellis"):
            return "exl3"
        if self.has(base + ".weight_packed"):
            return "nvfp4_ct"
        if self.has(base + ".weight_scale_2"):
            return "nvfp4_mo"
        if self.has(base + ".weight_scale_inv"):
            return "fp8_block"
        if self.has(base + ".weight"):
            return "dense"
        return None

    @staticmethod
    def _range(n: int, split, rank: int, world: int, unit: int):
        if split is None or world == 1:
            return 0, n
        if n % (world * unit):
            raise ValueError(f"dimension {n} does not split {world} ways in units of {unit}")
        per = n // world
        return rank * per, (rank + 1) * per

    def load_dense_weight(self, base: str, split=None, rank=0, world=1) -> torch.Tensor:
        """[N, K] fp32/bf16 weight of a dense or FP8-block linear; ``split`` = "col" (slice N) / "row" (slice K)."""
        w = self.load(base + ".weight")
        if self.has(base + ".weight_scale_inv"):                       # FP8 E4M3 with 128x128 block scales
            s = self.load(base + ".weight_scale_inv").float()
            N, K = w.shape
            sf = s.repeat_interleave(128, 0)[:N].repeat_interleave(128, 1)[:, :K]
            w = w.float() * sf
        N, K = w.shape
        n0, n1 = self._range(N, "col" if split == "col" else None, rank, world, 1)
        k0, k1 = self._range(K, "row" if split == "row" else None, rank, world, 1)
        return w[n0:n1, k0:k1]

    def load_exl3(self, base: str, split=None, rank=0, world=1, device=None):
        """EXL3 linear (optionally a TP slice that keeps whole 128-wide Hadamard spans)."""
        from ..ops.linear_exl3 import LinearEXL3
        codes = self.load(base + ".trellis")
        suh, svh = self.load(base + ".suh"), self.load(base + ".svh")
        bits = codes.shape[-1] // 16
        if codes.shape[-1] % 16 not in (0, 8):
            raise ValueError(f"{base}: {codes.shape[-1]} code words per tile is neither an integer nor a half-integer rate")
        tstart = self.load(base + ".tstart") if self.has(base + ".tstart") else None      # extended trellis: per-tile
        tgain = self.load(base + ".tgain") if self.has(base + ".tgain") else None          # start states / gain codes
        if (tstart is not None or tgain is not None) and codes.shape[-1] % 16:
            raise ValueError(f"{base}: the extended trellis is defined for integer rates")
        cb = ex.CB_MUL1 if self.has(base + ".mul1") else ex.CB_MCG if self.has(base + ".mcg") else ex.CB_3INST
        layout = "volta" if self.tile_layout == "volta" and base not in self.tile_layout_stock else "stock"
        K, N = codes.shape[0] * 16, codes.shape[1] * 16
        k0, k1 = self._range(K, "row" if split == "row" else None, rank, world, 128)
        n0, n1 = self._range(N, "col" if split == "col" else None, rank, world, 128)
        tiles = lambda t: None if t is None else t.reshape(K // 16, N // 16)[k0 // 16:k1 // 16, n0 // 16:n1 // 16].contiguous()
        lin = LinearEXL3(codes[k0 // 16:k1 // 16, n0 // 16:n1 // 16].contiguous(), suh[k0:k1].contiguous(),
                         svh[n0:n1].contiguous(), bits=bits, cb=cb, layout=layout, tstart=tiles(tstart), tgain=tiles(tgain))
        if self.has(base + ".bias"):
            b = self.load(base + ".bias")
            lin.bias = b[n0:n1].contiguous() if (split != "row" or rank == 0) else None
        return lin.to(device) if device is not None else lin

    def load_nvfp4(self, base: str, split=None, rank=0, world=1, device=None, gemm_mode="w4a16"):
        """NVFP4 linear from either dialect: compressed-tensors (``weight_packed`` / ``weight_scale`` /
        ``weight_global_scale`` = divisor) or modelopt (``weight`` / ``weight_scale`` / ``weight_scale_2`` =
        multiplier). Low nibble = even k in both."""
        if self.has(base + ".weight_packed"):
            packed = self.load(base + ".weight_packed")
            g = 1.0 / float(self.load(base + ".weight_global_scale").float().reshape(-1)[0])
        else:
            packed = self.load(base + ".weight")
            g = float(self.load(base + ".weight_scale_2").float().reshape(-1)[0])
        scales = self.load(base + ".weight_scale").view(torch.uint8)
        packed = packed.view(torch.uint8)
        N, K = packed.shape[0], packed.shape[1] * 2
        n0, n1 = self._range(N, "col" if split == "col" else None, rank, world, 1)
        k0, k1 = self._range(K, "row" if split == "row" else None, rank, world, 16)
        lin = LinearNVFP4(packed[n0:n1, k0 // 2:k1 // 2].contiguous(), scales[n0:n1, k0 // 16:k1 // 16].contiguous(),
                          g, gemm_mode)
        if device is not None:
            lin.packed, lin.scales = lin.packed.to(device), lin.scales.to(device)
            lin.prepare()
        return lin

    def load_linear(self, base: str, split=None, rank=0, world=1, device=None, gemm_mode="w4a16",
                    quantize: str | None = None):
        """Linear ``base`` in whatever format the checkpoint holds it. ``quantize="nvfp4"`` turns dense / FP8-block
        sources into NVFP4 at load (round to nearest with the +-2 scale-code search)."""
        kind = self.linear_kind(base)
        if kind is None:
            raise KeyError(f"no tensors for linear {base!r}")
        if kind == "exl3":
            return self.load_exl3(base, split, rank, world, device)
        if kind in ("nvfp4_ct", "nvfp4_mo"):
            return self.load_nvfp4(base, split, rank, world, device, gemm_mode)
        w = self.load_dense_weight(base, split, rank, world)
        if device is not None:
            w = w.to(device)
        if quantize == "nvfp4":
            return LinearNVFP4.from_dense(w.float(), gemm_mode, search=True).prepare()
        return LinearBF16(w.to(torch.bfloat16).contiguous())

    def close(self):
        for sh in self.shards:
            try:
                sh.mm.close()
            except BufferError:      # tensors still alias the mapping
                pass
            sh.f.close()
