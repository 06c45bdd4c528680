"""``volta_quantize``: convert the linear layers of a safetensors model directory to NVFP4 (either checkpoint dialect)
or EXL3 (trellis) and write a new model directory; everything else (norms, embeddings, json / tokenizer files) is
carried over unchanged.

NVFP4: round to nearest with the +-2 block-scale search. EXL3: random-sign Hadamard rotation, per-matrix scale,
tail-biting Viterbi per 16x16 tile (O(2^(16+bits)) per position: hours for large models, meant to run on a GPU via
``--device cuda``). Reference: src/tools/quant/* (``volta_quantize``: work planner, source readers, safetensors writer),
src/kernels/cuda/trellis/quant/ (encoder).
"""
from __future__ import annotations

import argparse
import json
import shutil
import sys
from pathlib import Path

import torch

from ..loader.safetensors import SafeTensorsRepo, write_safetensors
from ..quant import exl3 as ex, nvfp4 as qn

_SKIP = ("embed_tokens", "lm_head", "norm", "router", "mlp.gate.weight", "shared_expert_gate", "conv1d", "A_log", "dt_bias")


def is_linear_weight(name: str, shape, min_dim: int) -> bool:
    if not name.endswith(".weight") or len(shape) != 2 or min(shape) < min_dim:
        return False
    if any(s in name for s in _SKIP):
        return False
    return shape[1] % 16 == 0


def plan(repo: SafeTensorsRepo, fmt: str, min_dim: int = 128) -> dict:
    """-> {tensor name: "quantize" | "copy"} with a size estimate."""
    out, qbytes, cbytes = {}, 0, 0
    for name in repo.names():
        dt, shape = repo.info(name)
        n = 1
        for s in shape:
            n *= s
        ok = is_linear_weight(name, shape, min_dim)
        if ok and fmt == "exl3" and (shape[0] % 128 or shape[1] % 128):
            ok = False
        out[name] = "quantize" if ok else "copy"
        if ok:
            qbytes += n
        else:
            cbytes += n * torch.empty((), dtype=dt).element_size()
    return {"actions": out, "quantized_params": qbytes, "copied_bytes": cbytes}


def quantize_dir(src_dir, dst_dir, fmt: str = "nvfp4", bits: int = 4, device: str = "cpu", shard_bytes: int = 4 << 30,
                 min_dim: int = 128, log=print) -> dict:
    src, dst = Path(src_dir), Path(dst_dir)
    dst.mkdir(parents=True, exist_ok=True)
    repo = SafeTensorsRepo(src)
    pl = plan(repo, fmt, min_dim)
    shard, size, idx, u16, shards = {}, 0, 1, [], []

    def flush():
        nonlocal shard, size, idx, u16
        if shard:
            name = f"model-{idx:05d}.safetensors"
            write_safetensors(dst / name, shard, unsigned16=tuple(u16))
            shards.append(name)
            idx += 1
        shard, size, u16 = {}, 0, []

    def put(name, t, unsigned=False):
        nonlocal size
        shard[name] = t.cpu()
        if unsigned:
            u16.append(name)
        size += t.numel() * t.element_size()
        if size >= shard_bytes:
            flush()

    nq = 0
    for name in sorted(repo.names()):
        t = repo.load(name)
        if pl["actions"][name] == "copy":
            put(name, t.clone())
            continue
        base = name[: -len(".weight")]
        w = t.to(device).float()
        if fmt in ("nvfp4", "nvfp4_modelopt"):
            p, s, g = qn.quantize_nvfp4(w, search=True)
            if fmt == "nvfp4":
                put(base + ".weight_packed", p)
                put(base + ".weight_scale", s.view(torch.float8_e4m3fn))
                put(base + ".weight_global_scale", torch.tensor([1.0 / g]))
            else:
                put(base + ".weight", p)
                put(base + ".weight_scale", s.view(torch.float8_e4m3fn))
                put(base + ".weight_scale_2", torch.tensor([g]))
        elif fmt == "exl3":
            codes, suh, svh = ex.quantize(w.t().contiguous(), bits)
            put(base + ".trellis", codes, unsigned=True)
            put(base + ".suh", suh)
            put(base + ".svh", svh)
            put(base + ".mul1", torch.zeros(1, dtype=torch.int32))
        else:
            raise ValueError(f"unknown format {fmt!r}")
        nq += 1
        log(f"quantized {name} {tuple(t.shape)} -> {fmt}")
    flush()
    for f in src.iterdir():
        if f.is_file() and f.suffix in (".json", ".txt", ".jinja", ".model") and "safetensors.index" not in f.name:
            shutil.copy(f, dst / f.name)
    qc = {"quant_method": "exl3" if fmt == "exl3" else "nvfp4", "bits": bits if fmt == "exl3" else 4,
          "format": fmt, "tile_layout": "stock"}
    (dst / "quantization_config.json").write_text(json.dumps(qc, indent=1))
    return {"quantized": nq, "shards": shards, "plan": {k: v for k, v in pl.items() if k != "actions"}}


def main(argv=None) -> int:
    ap = argparse.ArgumentParser(prog="volta_quantize")
    ap.add_argument("src")
    ap.add_argument("dst")
    ap.add_argument("--format", default="nvfp4", choices=["nvfp4", "nvfp4_modelopt", "exl3"])
    ap.add_argument("--bits", type=int, default=4)
    ap.add_argument("--device", default="cpu")
    ap.add_argument("--dry-run", action="store_true", help="print the work plan only")
    a = ap.parse_args(argv)
    if a.dry_run:
        pl = plan(SafeTensorsRepo(a.src), a.format)
        print(json.dumps({k: v for k, v in pl.items() if k != "actions"}, indent=1))
        print(sum(1 for v in pl["actions"].values() if v == "quantize"), "tensors to quantize")
        return 0
    rep = quantize_dir(a.src, a.dst, a.format, a.bits, a.device)
    print(json.dumps(rep, indent=1))
    return 0


if __name__ == "__main__":
    sys.exit(main())
