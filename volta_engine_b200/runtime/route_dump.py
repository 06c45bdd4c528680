"""Route dumps: the MoE block's input rows with the experts each row was routed to and the routing weights.

A dump is what the expert-level quantisation tools work from (scale tuning, expert scoring, activation Hessians of
the expert down projections): ``{layer: {expert: (rows [n, H] bf16, weights [n] fp32)}}`` saved with ``torch.save``.
The recorder keeps at most ``max_rows`` rows per expert and ignores decode-sized batches, as the Hessian capture does.
Reference: docs/CONFIG.md (``route_dump``), docs/QUANTIZATION.md:97-103 (what consumes a dump).
"""
from __future__ import annotations

import torch


class RouteRecorder:
    def __init__(self, layers=None, max_rows: int = 8192, min_rows: int = 17):
        self.layers = set(layers) if layers is not None else None
        self.max_rows, self.min_rows = max_rows, min_rows
        self.data: dict[int, dict[int, list]] = {}
        self.count: dict[tuple[int, int], int] = {}

    def record(self, layer: int, x: torch.Tensor, ids: torch.Tensor, w: torch.Tensor) -> None:
        """x [rows, H], ids [rows, k] global expert ids, w [rows, k]."""
        if x.shape[0] < self.min_rows or (self.layers is not None and layer not in self.layers):
            return
        xc, ic, wc = x.detach().to("cpu", torch.bfloat16), ids.detach().cpu().long(), w.detach().cpu().float()
        per = self.data.setdefault(layer, {})
        for e in ic.unique().tolist():
            if e < 0:
                continue
            have = self.count.get((layer, e), 0)
            if have >= self.max_rows:
                continue
            r, c = (ic == e).nonzero(as_tuple=True)
            r, c = r[: self.max_rows - have], c[: self.max_rows - have]
            per.setdefault(e, []).append((xc[r], wc[r, c]))
            self.count[(layer, e)] = have + r.numel()

    def result(self) -> dict:
        return {layer: {e: (torch.cat([p[0] for p in parts]), torch.cat([p[1] for p in parts]))
                        for e, parts in sorted(per.items())} for layer, per in sorted(self.data.items())}

    def save(self, path) -> None:
        torch.save(self.result(), path)


def load_dumps(paths: str) -> dict:
    """One dump or several, comma-separated: their rows in that order."""
    out: dict = {}
    for p in [q for q in paths.split(",") if q]:
        d = torch.load(p, weights_only=True)
        for layer, per in d.items():
            tgt = out.setdefault(int(layer), {})
            for e, (rows, wts) in per.items():
                if int(e) in tgt:
                    tgt[int(e)] = (torch.cat([tgt[int(e)][0], rows]), torch.cat([tgt[int(e)][1], wts]))
                else:
                    tgt[int(e)] = (rows, wts)
    return out
