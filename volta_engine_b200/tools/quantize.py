"""``volta_quantize``: convert the linear layers of a safetensors model directory to NVFP4 (either checkpoint dialect)
or EXL3 (trellis) and write a new model directory; everything else (norms, embeddings, json / tokenizer files) is
carried over unchanged.

NVFP4: round to nearest with the +-2 block-scale search. EXL3: random-sign Hadamard rotation, per-matrix scale,
tail-biting Viterbi per 16x16 tile (O(2^(16+bits)) per position: hours for large models, meant to run on a GPU via
``--device cuda``). With ``--hess-dir`` (calibration captures, one file per layer and site) a tensor whose input
has a capture is quantised with the block LDL error feedback under that Hessian, and its proxy error
tr(E^T H E) / tr(W^T H W) is reported. Every finished tensor is written to ``<dst>/.partial/<name>.safetensors``
first, so an interrupted run continues where it stopped (``--redo`` starts over, ``--no-assemble`` stops before
the shards, ``--only`` restricts the work to tensors whose names contain one of the substrings). Reference: src/tools/quant/* (``volta_quantize``: work planner, source readers, safetensors writer),
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


def load_capture(hess_dir, name: str, k: int, ranks: int = 1):
    """The Hessian sum of the capture that belongs to tensor ``name`` (input width ``k``), or None. Captures of a
    tensor-parallel run hold the column-parallel sites whole on every rank (rank 0's file is read) and the
    row-parallel sites (o_proj, down) as per-rank diagonal blocks, which are assembled block-diagonally."""
    from ..ops import hessian as hz
    where = hz.site_of_tensor(name)
    if where is None or not hess_dir:
        return None
    layer, site = where
    parts = [hz.read_hessian(Path(hess_dir) / hz.site_file(layer, site, r)) for r in range(ranks)]
    if parts[0] is None:
        return None
    if parts[0][0].shape[0] == k:
        return parts[0][0]
    if any(p is None for p in parts) or sum(p[0].shape[0] for p in parts) != k:
        return None
    return torch.block_diag(*[p[0] for p in parts])


def _quantize_tensor(w: torch.Tensor, fmt: str, bits: int, H, sigma_reg: float) -> tuple[dict, tuple, float | None]:
    """One [N, K] checkpoint weight -> ({suffix: tensor}, suffixes stored as unsigned 16-bit, proxy error or None)."""
    from ..quant import ldlq
    err = None
    if fmt in ("nvfp4", "nvfp4_modelopt"):
        if H is not None:
            p, s, g = ldlq.quantize_nvfp4_hessian(w, H.to(w.device), sigma_reg)
            err = ldlq.proxy_error(w.t(), qn.dequantize_nvfp4(p, s, g).t(), H.to(w.device))
        else:
            p, s, g = qn.quantize_nvfp4(w, search=True)
        if fmt == "nvfp4":
            return {".weight_packed": p, ".weight_scale": s.view(torch.float8_e4m3fn),
                    ".weight_global_scale": torch.tensor([1.0 / g])}, (), err
        return {".weight": p, ".weight_scale": s.view(torch.float8_e4m3fn), ".weight_scale_2": torch.tensor([g])}, (), err
    if fmt == "exl3":
        W = w.t().contiguous()
        if H is not None:
            codes, suh, svh = ldlq.quantize_exl3_hessian(W, H.to(w.device), bits, sigma_reg=sigma_reg)
            err = ldlq.proxy_error(W, ex.effective_weight(codes, bits, suh, svh), H.to(w.device))
        else:
            codes, suh, svh = ex.quantize(W, bits)
        return {".trellis": codes, ".suh": suh, ".svh": svh, ".mul1": torch.zeros(1, dtype=torch.int32)}, (".trellis",), err
    raise ValueError(f"unknown format {fmt!r}")


def _partial_name(name: str) -> str:
    return name.replace("/", "_") + ".safetensors"


def quantize_dir(src_dir, dst_dir, fmt: str = "nvfp4", bits: int = 4, device: str = "cpu", shard_bytes: int = 4 << 30,
                 min_dim: int = 128, log=print, hess_dir=None, hess_ranks: int = 1, sigma_reg: float = 0.025,
                 only=None, redo: bool = False, assemble: bool = True) -> dict:
    src, dst = Path(src_dir), Path(dst_dir)
    dst.mkdir(parents=True, exist_ok=True)
    partial = dst / ".partial"
    if redo and partial.exists():
        shutil.rmtree(partial)
    partial.mkdir(exist_ok=True)
    repo = SafeTensorsRepo(src)
    pl = plan(repo, fmt, min_dim)
    if only:
        for name, act in pl["actions"].items():
            if act == "quantize" and not any(o in name for o in only):
                pl["actions"][name] = "copy"
    todo = [n for n in sorted(repo.names()) if pl["actions"][n] == "quantize"]
    errors, resumed = {}, 0
    for name in todo:
        pf = partial / _partial_name(name)
        if pf.exists():
            resumed += 1
            continue
        w = repo.load(name).to(device).float()
        H = load_capture(hess_dir, name, w.shape[1], hess_ranks)
        parts, u, err = _quantize_tensor(w, fmt, bits, H, sigma_reg)
        meta = {"format": fmt, "bits": str(bits), "tile_layout": "stock", "hessian": "1" if H is not None else "0"}
        if err is not None:
            meta["proxy_error"] = repr(err)
            errors[name] = err
        tmp = pf.with_suffix(".tmp")
        write_safetensors(tmp, {k: v.cpu() for k, v in parts.items()}, unsigned16=u, metadata=meta)
        tmp.rename(pf)                                   # a tensor is either wholly there or not at all
        log(f"quantized {name} {tuple(w.shape)} -> {fmt}" + (f"  proxy error {err:.5f}" if err is not None else ""))
    if not assemble:
        return {"quantized": len(todo) - resumed, "resumed": resumed, "shards": [], "proxy_errors": errors,
                "plan": {k: v for k, v in pl.items() if k != "actions"}}
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
        if pl["actions"][name] == "copy":
            put(name, repo.load(name).clone())
            continue
        base = name[: -len(".weight")]
        pr = SafeTensorsRepo(partial / _partial_name(name))
        for suffix in pr.names():
            put(base + suffix, pr.load(suffix).clone(), unsigned=suffix == ".trellis")
        nq += 1
    flush()
    for f in src.iterdir():
        if f.is_file() and f.suffix in (".json", ".txt", ".jinja", ".model") and "safetensors.index" not in f.name:
            shutil.copy(f, dst / f.name)
    qc = {"quant_method": "exl3" if fmt == "exl3" else "nvfp4", "bits": bits if fmt == "exl3" else 4,
          "format": fmt, "tile_layout": "stock"}
    (dst / "quantization_config.json").write_text(json.dumps(qc, indent=1))
    return {"quantized": nq, "resumed": resumed, "shards": shards, "proxy_errors": errors,
            "plan": {k: v for k, v in pl.items() if k != "actions"}}


def main(argv=None) -> int:
    ap = argparse.ArgumentParser(prog="volta_quantize")
    ap.add_argument("src")
    ap.add_argument("dst")
    ap.add_argument("--format", default="nvfp4", choices=["nvfp4", "nvfp4_modelopt", "exl3"])
    ap.add_argument("--bits", type=int, default=4)
    ap.add_argument("--device", default="cpu")
    ap.add_argument("--dry-run", action="store_true", help="print the work plan only")
    ap.add_argument("--hess-dir", default="", help="calibration captures (L<layer>_s<site>_r<rank>.f32): Hessian-aware rounding")
    ap.add_argument("--ranks", type=int, default=1, help="tensor-parallel ranks of the capture run")
    ap.add_argument("--sigma-reg", type=float, default=0.025, help="damping, as a fraction of the Hessian's mean diagonal")
    ap.add_argument("--only", default="", help="comma-separated substrings: quantise only the tensors that contain one")
    ap.add_argument("--redo", action="store_true", help="discard <dst>/.partial and quantise everything again")
    ap.add_argument("--no-assemble", action="store_true", help="stop after <dst>/.partial (no shards)")
    a = ap.parse_args(argv)
    if a.dry_run:
        pl = plan(SafeTensorsRepo(a.src), a.format)
        print(json.dumps({k: v for k, v in pl.items() if k != "actions"}, indent=1))
        print(sum(1 for v in pl["actions"].values() if v == "quantize"), "tensors to quantize")
        return 0
    rep = quantize_dir(a.src, a.dst, a.format, a.bits, a.device, hess_dir=a.hess_dir or None, hess_ranks=a.ranks,
                       sigma_reg=a.sigma_reg, only=[o for o in a.only.split(",") if o] or None, redo=a.redo,
                       assemble=not a.no_assemble)
    print(json.dumps(rep, indent=1))
    return 0


if __name__ == "__main__":
    sys.exit(main())
