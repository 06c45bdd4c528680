"""``hess_compare``: calibration sources and the quantisation each leads to, compared.

  hess_compare stats <dir_a> <dir_b>
      per capture file both mean Hessians (sum / rows): |A - B| / |B| (Frobenius), the same for the diagonals,
      tr(A) / tr(B); per site the mean and the worst, and the ten worst files
  hess_compare merge <out dir> <dir> <dir> ...
      the capture files every directory has, summed (Hessian sums and row counts: a calibration mixed by token count)
  hess_compare cross --src <original> --tensor <name> --a <file> --b <file> [--format nvfp4|exl3] [--bits 3]
      the tensor quantised with each Hessian, both results' proxy errors under both mean Hessians: when A's
      quantisation scores under B as B's own does, A is as good a calibration source as B for that tensor
  hess_compare score --src <original> --tensors A,B,... (--hess-dir <captures> [--ranks 1] | --route <dump>) --ckpt <dir> ...
      each tensor of each quantised checkpoint (NVFP4 in either dialect, EXL3, or a quantiser's ``.partial`` directory)
      against the original: the proxy error tr(E^T H E) / tr(W^T H W) under the capture's Hessian, or for a routed
      expert's projection under the Hessian of its input over the dump's rows (``--affinity-eps E``: each row weighted
      by its routing weight + E)
  hess_compare routes --route <dump> --layers L,L,... [--top 32] [--prefix ...]
      per layer the experts most rows route to, most first, and their projections as a quantiser ``--only`` list
  hess_compare moe --src <original> --route <dump> --layers L,L,... [--max-rows 8192] --ckpt <dir> [--ckpt <dir> ...]
      each routed expert: its output's error against the original expert's over the dump's rows routed to it, every
      row weighted by its routing weight squared (its share of the block's output), relative to the original output;
      per layer the mean, and each checkpoint relative to the first

Reference: tests/tools/hess_compare.cpp (the six sub-commands), docs/QUANTIZATION.md:97.
"""
from __future__ import annotations

import argparse
import math
import os
import re
import sys
from pathlib import Path

import torch

from ..ops import hessian as hz
from ..quant import exl3 as ex, ldlq, nvfp4 as qn


# ------------------------------------------------------------------------------------------------ stats / merge
def kind_of(fn: str) -> str:
    """"s1", "s2", "expert down": the site part of a capture file name."""
    if re.fullmatch(r"L\d+_E\d+_down\.f32", fn):
        return "expert down"
    m = re.fullmatch(r"L\d+_s(\d+)_r\d+\.f32", fn)
    return f"s{m.group(1)}" if m else "other"


def compare_pair(a, b) -> dict:
    """Two captures (sum, rows) -> relative Frobenius distance of the means, of their diagonals, and the trace ratio."""
    A, B = a[0].double() / a[1], b[0].double() / b[1]
    da, db = A.diagonal(), B.diagonal()
    return {"fro": float((A - B).norm() / B.norm().clamp(min=1e-300)),
            "diag": float((da - db).norm() / db.norm().clamp(min=1e-300)),
            "trace": float(da.sum() / db.sum().clamp(min=1e-300))}


def stats(dir_a, dir_b, out=print) -> dict:
    names = sorted(f for f in os.listdir(dir_a) if f.endswith(".f32"))
    rows, by_kind, missing = [], {}, 0
    for fn in names:
        a = hz.read_hessian(os.path.join(dir_a, fn))
        if a is None:
            continue
        b = hz.read_hessian(os.path.join(dir_b, fn))
        if b is None:
            missing += 1
            continue
        if a[0].shape != b[0].shape:
            out(f"  {fn}: k {a[0].shape[0]} against {b[0].shape[0]}")
            continue
        r = dict(compare_pair(a, b), name=fn)
        rows.append(r)
        by_kind.setdefault(kind_of(fn), []).append(r["fro"])
    out(f"[*] hess_compare: {len(rows)} files in both, {missing} only in {dir_a}")
    out(f"  {'site':<14} {'files':>6} {'mean':>12} {'worst':>12}   (|A - B| / |B| of the mean Hessians)")
    summary = {}
    for kind, v in sorted(by_kind.items()):
        summary[kind] = {"files": len(v), "mean": sum(v) / len(v), "worst": max(v)}
        out(f"  {kind:<14} {len(v):>6} {summary[kind]['mean']:>12.5f} {summary[kind]['worst']:>12.5f}")
    rows.sort(key=lambda r: -r["fro"])
    out(f"  {'worst files':<24} {'fro':>10} {'diag':>10} {'tr A / tr B':>12}")
    for r in rows[:10]:
        out(f"  {r['name']:<24} {r['fro']:>10.5f} {r['diag']:>10.5f} {r['trace']:>12.5f}")
    return {"files": rows, "sites": summary, "missing": missing}


# ------------------------------------------------------------------------------------------------ checkpoints
def _find(repo, base: str, suffixes) -> str | None:
    for s in suffixes:
        if repo.has(base + s):
            return base + s
    return None


def load_quantized(ckpt, base: str, device="cpu") -> torch.Tensor | None:
    """The effective weight [K, N] (y = x W) of tensor ``base`` in a quantised checkpoint directory: NVFP4 in the
    compressed-tensors or the ModelOpt dialect, EXL3, or a quantiser's ``.partial`` directory (one file per tensor,
    the names are the suffixes alone and the file's metadata names the format)."""
    from ..loader.safetensors import SafeTensorsRepo
    ckpt = Path(ckpt)
    pf = ckpt / (base.replace("/", "_") + ".weight.safetensors")
    if pf.exists():
        repo, base = SafeTensorsRepo(pf), ""
    elif (ckpt / ".partial" / pf.name).exists():
        repo, base = SafeTensorsRepo(ckpt / ".partial" / pf.name), ""
    else:
        repo = SafeTensorsRepo(ckpt)
    if repo.has(base + ".trellis"):
        codes = repo.load(base + ".trellis", device=device)
        bits = codes.shape[-1] // 16
        cb = ex.CB_MUL1 if repo.has(base + ".mul1") else ex.CB_MCG if repo.has(base + ".mcg") else ex.CB_3INST
        layout = "volta" if repo.tile_layout == "volta" and base not in repo.tile_layout_stock else "stock"
        side = lambda n: repo.load(base + n, device=device).reshape(codes.shape[0], codes.shape[1]) if repo.has(base + n) else None
        return ex.effective_weight(codes, bits, repo.load(base + ".suh", device=device),
                                   repo.load(base + ".svh", device=device), cb, layout, side(".tstart"), side(".tgain")).float()
    if repo.has(base + ".weight_packed"):
        g = 1.0 / float(repo.load(base + ".weight_global_scale").float().reshape(-1)[0])
        return qn.dequantize_nvfp4(repo.load(base + ".weight_packed", device=device),
                                   repo.load(base + ".weight_scale", device=device).view(torch.uint8), g).t().contiguous()
    if repo.has(base + ".weight_scale_2"):
        g = float(repo.load(base + ".weight_scale_2").float().reshape(-1)[0])
        return qn.dequantize_nvfp4(repo.load(base + ".weight", device=device),
                                   repo.load(base + ".weight_scale", device=device).view(torch.uint8), g).t().contiguous()
    if repo.has(base + ".weight"):
        return repo.load(base + ".weight", device=device).float().t().contiguous()
    return None


def input_hessian(rows: torch.Tensor, wts: torch.Tensor | None = None, eps: float | None = None) -> torch.Tensor:
    """x^T diag(r) x over dump rows; r = 1, or routing weight + eps when ``eps`` is given."""
    x = rows.double()
    if eps is not None and wts is not None:
        x = x * (wts.double() + eps).clamp(min=0).sqrt()[:, None]
    return (x.t() @ x).float()


def _expert_of(name: str):
    m = re.search(r"layers\.(\d+)\..*experts\.(\d+)\.(gate|up|down)_proj", name)
    return (int(m.group(1)), int(m.group(2)), m.group(3)) if m else None


def expert_site_hessian(src, dump, layer, expert, proj, prefix, device, eps=None, act="silu"):
    """The Hessian of a routed expert's projection input over the dump's rows: the block input for gate / up, the
    ORIGINAL expert's activation (act(gate) * up) for down."""
    if layer not in dump or expert not in dump[layer]:
        return None
    rows, wts = dump[layer][expert]
    rows = rows.to(device).float()
    if proj != "down":
        return input_hessian(rows, wts.to(device), eps)
    g = src.load(prefix.format(layer=layer, expert=expert, proj="gate") + ".weight").to(device).float()
    u = src.load(prefix.format(layer=layer, expert=expert, proj="up") + ".weight").to(device).float()
    gate = rows @ g.t()
    a = (torch.nn.functional.silu(gate) if act == "silu" else torch.nn.functional.gelu(gate, approximate="tanh")) * (rows @ u.t())
    return input_hessian(a, wts.to(device), eps)


# ------------------------------------------------------------------------------------------------ cross / score
def cross(src_dir, tensor: str, file_a, file_b, fmt: str = "nvfp4", bits: int = 3, device="cpu", sigma_reg=0.025,
          out=print) -> dict:
    from ..loader.safetensors import SafeTensorsRepo
    name = tensor if tensor.endswith(".weight") else tensor + ".weight"
    w = SafeTensorsRepo(src_dir).load(name).to(device).float()                      # [N, K]
    caps = {"A": hz.read_hessian(file_a), "B": hz.read_hessian(file_b)}
    for k, c in caps.items():
        if c is None or c[0].shape[0] != w.shape[1]:
            raise ValueError(f"capture {k} does not fit {name} (input width {w.shape[1]})")
    mean = {k: (c[0] / c[1]).to(device) for k, c in caps.items()}
    res = {}
    for k in ("A", "B"):
        if fmt == "exl3":
            codes, suh, svh = ldlq.quantize_exl3_hessian(w.t().contiguous(), mean[k], bits, sigma_reg=sigma_reg)
            wq = ex.effective_weight(codes, bits, suh, svh)
        else:
            p, s, g = ldlq.quantize_nvfp4_hessian(w, mean[k], sigma_reg)
            wq = qn.dequantize_nvfp4(p, s, g).t()
        res[k] = {f"under_{h}": ldlq.proxy_error(w.t(), wq, mean[h]) for h in ("A", "B")}
    out(f"[*] {name} {tuple(w.shape)} as {fmt}: proxy error tr(E^T H E) / tr(W^T H W)")
    out(f"  {'quantised with':<16} {'under A':>12} {'under B':>12}")
    for k in ("A", "B"):
        out(f"  {k:<16} {res[k]['under_A']:>12.6f} {res[k]['under_B']:>12.6f}")
    ratio = res["A"]["under_B"] / max(res["B"]["under_B"], 1e-300)
    out(f"  A's quantisation under B against B's own: {ratio:.4f}x")
    res["ratio"] = ratio
    return res


def score(src_dir, tensors, ckpts, hess_dir=None, ranks: int = 1, route=None, prefix=None, affinity_eps=None,
          device="cpu", out=print) -> dict:
    from ..loader.safetensors import SafeTensorsRepo
    from ..runtime.route_dump import load_dumps
    from .quantize import load_capture
    src = SafeTensorsRepo(src_dir)
    dump = load_dumps(route) if route else None
    table = {}
    out(f"  {'tensor':<56} " + " ".join(f"{Path(c).name[:14]:>14}" for c in ckpts))
    for t in tensors:
        base = t[:-len(".weight")] if t.endswith(".weight") else t
        w = src.load(base + ".weight").to(device).float()
        H = None
        eo = _expert_of(base)
        if dump is not None and eo is not None:
            H = expert_site_hessian(src, dump, eo[0], eo[1], eo[2], prefix, device, affinity_eps)
        elif hess_dir:
            H = load_capture(hess_dir, base + ".weight", w.shape[1], ranks)
            H = H.to(device) if H is not None else None
        if H is None:
            out(f"  {base:<56} no Hessian for this tensor")
            continue
        row = []
        for c in ckpts:
            wq = load_quantized(c, base, device)
            row.append(float("nan") if wq is None else ldlq.proxy_error(w.t(), wq, H))
        table[base] = row
        out(f"  {base:<56} " + " ".join(f"{v:>14.6f}" for v in row))
    return table


# ------------------------------------------------------------------------------------------------ routes / moe
DEFAULT_PREFIX = "model.layers.{layer}.mlp.experts.{expert}.{proj}_proj"


def routes(route, layers, top: int = 32, prefix: str = DEFAULT_PREFIX, out=print) -> dict:
    from ..runtime.route_dump import load_dumps
    dump = load_dumps(route)
    res = {}
    for layer in layers:
        per = dump.get(layer, {})
        order = sorted(per, key=lambda e: -per[e][0].shape[0])[:top]
        total = sum(v[0].shape[0] for v in per.values())
        res[layer] = [(e, per[e][0].shape[0]) for e in order]
        out(f"[*] layer {layer}: {len(per)} experts saw rows, {total} routes; the {len(order)} busiest:")
        out("  " + " ".join(f"{e}:{n}" for e, n in res[layer]))
        out("  --only " + ",".join(prefix.format(layer=layer, expert=e, proj=p) + "." for e, _ in res[layer]
                                   for p in ("gate", "up", "down")))
    return res


def _expert_out(g, u, d, x, act):
    gate = x @ g
    a = (torch.nn.functional.silu(gate) if act == "silu" else torch.nn.functional.gelu(gate, approximate="tanh")) * (x @ u)
    return a @ d


def moe(src_dir, route, layers, ckpts, max_rows: int = 8192, prefix: str = DEFAULT_PREFIX, device="cpu", act="silu",
        out=print) -> dict:
    from ..loader.safetensors import SafeTensorsRepo
    from ..runtime.route_dump import load_dumps
    src, dump = SafeTensorsRepo(src_dir), load_dumps(route)
    res = {}
    for layer in layers:
        per_ckpt = [[] for _ in ckpts]
        for e, (rows, wts) in sorted(dump.get(layer, {}).items()):
            x, r2 = rows[:max_rows].to(device).float(), wts[:max_rows].to(device).float() ** 2
            W = [src.load(prefix.format(layer=layer, expert=e, proj=p) + ".weight").to(device).float().t() for p in ("gate", "up", "down")]
            y = _expert_out(*W, x, act)
            den = float((r2[:, None] * y * y).sum())
            for ci, c in enumerate(ckpts):
                Q = [load_quantized(c, prefix.format(layer=layer, expert=e, proj=p), device) for p in ("gate", "up", "down")]
                if any(q is None for q in Q):
                    continue
                yq = _expert_out(*Q, x, act)
                per_ckpt[ci].append((e, float((r2[:, None] * (yq - y) ** 2).sum()) / max(den, 1e-300)))
        means = [sum(v for _, v in p) / len(p) if p else math.nan for p in per_ckpt]
        res[layer] = {"experts": per_ckpt, "mean": means}
        out(f"[*] layer {layer}: mean relative output error per checkpoint: " +
            "  ".join(f"{m:.6f}" + (f" ({m / means[0]:.3f}x of [0])" if i and means[0] > 0 else "") for i, m in enumerate(means)))
    return res


# ------------------------------------------------------------------------------------------------ CLI
def main(argv=None) -> int:
    ap = argparse.ArgumentParser(prog="hess_compare", description=__doc__.split("\n\n")[0])
    sub = ap.add_subparsers(dest="cmd", required=True)
    p = sub.add_parser("stats"); p.add_argument("dir_a"); p.add_argument("dir_b")
    p = sub.add_parser("merge"); p.add_argument("out"); p.add_argument("dirs", nargs="+")
    p.add_argument("--weights", default="", help="comma list: each directory's share of the mix instead of its row count")
    p = sub.add_parser("cross")
    p.add_argument("--src", required=True); p.add_argument("--tensor", required=True)
    p.add_argument("--a", required=True); p.add_argument("--b", required=True)
    p.add_argument("--format", default="nvfp4", choices=["nvfp4", "exl3"]); p.add_argument("--bits", type=int, default=3)
    p.add_argument("--device", default="cpu"); p.add_argument("--sigma-reg", type=float, default=0.025)
    p = sub.add_parser("score")
    p.add_argument("--src", required=True); p.add_argument("--tensors", required=True)
    p.add_argument("--hess-dir", default=""); p.add_argument("--ranks", type=int, default=1)
    p.add_argument("--route", default=""); p.add_argument("--affinity-eps", type=float, default=None)
    p.add_argument("--ckpt", action="append", required=True); p.add_argument("--prefix", default=DEFAULT_PREFIX)
    p.add_argument("--device", default="cpu")
    p = sub.add_parser("routes")
    p.add_argument("--route", required=True); p.add_argument("--layers", required=True)
    p.add_argument("--top", type=int, default=32); p.add_argument("--prefix", default=DEFAULT_PREFIX)
    p = sub.add_parser("moe")
    p.add_argument("--src", required=True); p.add_argument("--route", required=True); p.add_argument("--layers", required=True)
    p.add_argument("--max-rows", type=int, default=8192); p.add_argument("--ckpt", action="append", required=True)
    p.add_argument("--prefix", default=DEFAULT_PREFIX); p.add_argument("--device", default="cpu")
    p.add_argument("--act", default="silu", choices=["silu", "gelu"])
    a = ap.parse_args(argv)
    ints = lambda s: [int(x) for x in s.split(",") if x]
    if a.cmd == "stats":
        stats(a.dir_a, a.dir_b)
    elif a.cmd == "merge":
        w = [float(x) for x in a.weights.split(",") if x] or None
        done = hz.merge_dirs(a.out, a.dirs, w)
        print(f"[*] hess_compare: {len(done)} files written to {a.out}")
    elif a.cmd == "cross":
        cross(a.src, a.tensor, a.a, a.b, a.format, a.bits, a.device, a.sigma_reg)
    elif a.cmd == "score":
        if not a.hess_dir and not a.route:
            ap.error("score needs --hess-dir or --route")
        score(a.src, [t for t in a.tensors.split(",") if t], a.ckpt, a.hess_dir or None, a.ranks, a.route or None,
              a.prefix, a.affinity_eps, a.device)
    elif a.cmd == "routes":
        routes(a.route, ints(a.layers), a.top, a.prefix)
    elif a.cmd == "moe":
        moe(a.src, a.route, ints(a.layers), a.ckpt, a.max_rows, a.prefix, a.device, a.act)
    return 0


if __name__ == "__main__":
    sys.exit(main())
