"""``volta_tune``: tune the scale vectors of a quantised gated expert so that its output matches the original expert's on
the rows routed to it.

An expert is three linears, each a frozen core between a per-input-channel and a per-output-channel scale
(``W = diag(su) T diag(sv)``: for EXL3 the core is the Hadamard-rotated trellis decode, for any other format the
dequantised matrix with unit scales). All six scale vectors are multiplied by ``exp(a)`` with ``a`` trained by Adam on the
row-weighted squared error against the original expert (rows weighted by their routing weight squared); every tenth row is
held out and the step with the lowest held-out error is kept. Built on the training primitives of train/grad.py
(SwiGLU forward / backward, scaled-linear gradients, weighted squared error, Adam on log scales).
Reference: docs/QUANTIZATION.md:103 (``volta_tune``), src/tools/volta_tune.cpp, inc/engine/train/grad.h.
"""
from __future__ import annotations

import argparse
import json
import sys
from dataclasses import dataclass
from pathlib import Path

import torch

from ..train import grad as G


@dataclass
class TuneResult:
    scales: dict            # name -> (su, sv) tuned
    err_before: float       # held-out relative error before
    err_after: float        # held-out relative error at the kept step
    best_step: int
    train_curve: list


def expert_forward(lin: dict, X, limit: float = 0.0):
    """lin: {"gate", "up", "down"} of ScaledLinear. Returns (y, saved activations for the backward)."""
    g, zg = G.scaled_linear_forward(lin["gate"], X)
    u, zu = G.scaled_linear_forward(lin["up"], X)
    a = G.swiglu_forward(g, u, limit)
    y, zd = G.scaled_linear_forward(lin["down"], a)
    return y, (g, zg, u, zu, a, zd)


def expert_backward(lin: dict, X, saved, dy, limit: float = 0.0):
    g, zg, u, zu, a, zd = saved
    da = G.scaled_linear_backward(lin["down"], a, zd, dy)
    dg, du = G.swiglu_backward(g, u, da, limit)
    G.scaled_linear_backward(lin["gate"], X, zg, dg, want_dx=False)
    G.scaled_linear_backward(lin["up"], X, zu, du, want_dx=False)


def tune_expert(orig: dict, quant: dict, X: torch.Tensor, row_w: torch.Tensor | None = None, steps: int = 100, lr: float = 1e-3,
                limit: float = 0.0, holdout: int = 10) -> TuneResult:
    """orig: {"gate","up","down"} dense [in, out] fp32 weights (y = x @ W). quant: the same names -> ScaledLinear (core + the
    checkpoint's scales). X [rows, hidden] the rows routed to the expert, row_w their routing weights."""
    dev = X.device
    X = X.float()
    rows = X.shape[0]
    w2 = (row_w.float() ** 2 if row_w is not None else torch.ones(rows, device=dev))
    hold = torch.arange(rows, device=dev) % holdout == holdout - 1
    Xt, Xh, wt, wh = X[~hold].contiguous(), X[hold].contiguous(), w2[~hold].contiguous(), w2[hold].contiguous()

    def target(Xs):
        return (G.swiglu_forward(Xs @ orig["gate"].float(), Xs @ orig["up"].float(), limit) @ orig["down"].float()).contiguous()
    Tt, Th = target(Xt), target(Xh)
    norm_h = max(G.weighted_sq_norm(Th, wh), 1e-30)
    norm_t = max(G.weighted_sq_norm(Tt, wt), 1e-30)
    lin, state = {}, {}
    for n, q in quant.items():
        l = G.ScaledLinear(q.T.float().contiguous(), q.su.float().clone(), q.sv.float().clone())
        l.dsu, l.dsv = torch.zeros_like(l.su), torch.zeros_like(l.sv)
        lin[n] = l
        state[n] = {k: {"s0": getattr(l, k).clone(), "a": torch.zeros_like(getattr(l, k)), "m": torch.zeros_like(getattr(l, k)),
                        "v": torch.zeros_like(getattr(l, k))} for k in ("su", "sv")}
    opt = G.AdamOptions(lr=lr)

    def held_out():
        y, _ = expert_forward(lin, Xh, limit)
        return G.weighted_sq_error(y.contiguous(), Th, wh)[0] / norm_h
    before = held_out()
    best = (before, 0, {n: (l.su.clone(), l.sv.clone()) for n, l in lin.items()})
    curve = []
    for step in range(1, steps + 1):
        for l in lin.values():
            l.dsu.zero_()
            l.dsv.zero_()
        y, saved = expert_forward(lin, Xt, limit)
        loss, dy = G.weighted_sq_error(y.contiguous(), Tt, wt, want_dy=True, scale=1.0 / norm_t)
        curve.append(loss / norm_t)
        expert_backward(lin, Xt, saved, dy, limit)
        for n, l in lin.items():
            for k, gname in (("su", "dsu"), ("sv", "dsv")):
                st = state[n][k]
                G.adam_log_scales(st["s0"], st["a"], getattr(l, k), getattr(l, gname), st["m"], st["v"], step, 1.0, opt)
        e = held_out()
        if e < best[0]:
            best = (e, step, {n: (l.su.clone(), l.sv.clone()) for n, l in lin.items()})
    return TuneResult(best[2], before, best[0], best[1], curve)


def exl3_scaled_linear(codes, bits, suh, svh, cb=2, layout="stock") -> G.ScaledLinear:
    """The trainable view of an EXL3 tensor: core = H128 . decode(codes) . H128 (both Hadamards folded in), scales suh / svh."""
    from ..quant import exl3 as ex
    W = ex.reconstruct(codes, bits, cb, layout)                       # [K, N] in the rotated basis
    core = ex.had128(ex.had128(W.t()).t())                            # undo nothing: fold the two rotations into the core
    return G.ScaledLinear(core.contiguous(), suh.float().clone(), svh.float().clone())


def main(argv=None) -> int:
    ap = argparse.ArgumentParser(prog="volta_tune", description=__doc__.split("\n\n")[0])
    ap.add_argument("--src", required=True, help="original model directory (safetensors)")
    ap.add_argument("--exl3", required=True, help="quantised model directory")
    ap.add_argument("--route", required=True, help="route dump: torch file with {layer: {expert: (rows [n, H], weights [n])}}")
    ap.add_argument("--out", required=True)
    ap.add_argument("--layers", required=True, help="comma list of layer indices")
    ap.add_argument("--steps", type=int, default=100)
    ap.add_argument("--lr", type=float, default=1e-3)
    ap.add_argument("--max-rows", type=int, default=8192)
    ap.add_argument("--device", default="cuda" if torch.cuda.is_available() else "cpu")
    ap.add_argument("--prefix", default="model.layers.{layer}.mlp.experts.{expert}.{proj}_proj")
    a = ap.parse_args(argv)
    from ..loader.safetensors import SafeTensorsRepo, write_safetensors
    src, q = SafeTensorsRepo(a.src), SafeTensorsRepo(a.exl3)
    dump = torch.load(a.route, weights_only=True)
    out = Path(a.out) / ".partial"
    out.mkdir(parents=True, exist_ok=True)
    report = {}
    for layer in (int(x) for x in a.layers.split(",")):
        for expert, (rows, wts) in sorted(dump.get(layer, {}).items()):
            rows, wts = rows[: a.max_rows].to(a.device), wts[: a.max_rows].to(a.device)
            orig, quant = {}, {}
            for proj in ("gate", "up", "down"):
                base = a.prefix.format(layer=layer, expert=expert, proj=proj)
                orig[proj] = src.load(base + ".weight").to(a.device).float().t().contiguous()
                t = q.load_exl3(base, device=a.device)
                quant[proj] = exl3_scaled_linear(t.codes, t.bits, t.suh, t.svh, t.cb)
            res = tune_expert(orig, quant, rows, wts, a.steps, a.lr)
            tensors = {}
            for proj, (su, sv) in res.scales.items():
                base = a.prefix.format(layer=layer, expert=expert, proj=proj)
                tensors[base + ".suh"], tensors[base + ".svh"] = su.half().cpu(), sv.half().cpu()
            write_safetensors(out / f"L{layer}_E{expert}.safetensors", tensors)
            report[f"{layer}.{expert}"] = {"before": res.err_before, "after": res.err_after, "step": res.best_step}
            print(f"layer {layer} expert {expert}: held-out error {res.err_before:.5f} -> {res.err_after:.5f} (step {res.best_step})")
    (out / "tune_report.json").write_text(json.dumps(report, indent=1))
    return 0


if __name__ == "__main__":
    sys.exit(main())
