"""Request-time probe steering: measure, for THIS prompt, where the model's states sit between "accepting" and
"declining" continuations, and clamp the declining direction out of the residual stream when the prompt leans that way.

Procedure (requests with ``steer_probe``; reference: docs/CONFIG.md:108-120, src/runtime/steer_probe.cpp,
src/runtime/generator_probe.cpp):
  1. After the prompt is in the cache, every forced opening (a few accepting, declining, plain and hedged first words of a
     reply) is run at the positions behind the prompt and the residual state of its last token is read at every band
     layer (``StateCapture`` hooks the model's steering call).
  2. Per edit layer the first direction is the unit vector from the accepting openings' mean to the declining openings'
     mean; further directions (``steer_directions`` up to 4) are the strongest remaining variations of the declining
     openings once the first direction and the accepting openings' own spread are removed.
  3. The gate: the state of the prompt's last token, placed on that axis in the middle band layer (0 = like the accepting
     openings, 1 = like the declining ones). Above ``steer_gate_threshold`` the clamps are installed.
  4. A clamp removes the part of a row's projection that exceeds a reference level: the accepting openings' mean
     projection minus ``steer_edit_strength`` standard deviations (so more negative strengths leave more in place).
     ``steer_keep_norm`` rescales an edited row to its old norm. ``steer_hedge_strength`` >= 0 adds a second clamp on the
     plain -> hedged axis at that fraction of the gap. ``steer_push`` adds the declining direction (times the gap between
     the two groups) whether or not the gate fires; negative values push towards accepting.
The probe's scores are reported in the request's usage.
"""
from __future__ import annotations

from dataclasses import dataclass, field

import torch

from .batch import BatchRows, LOGITS_NONE
from .steering import (SCOPE_ALL, STEER_ADD, STEER_CLAMP, STEER_CLAMP_KEEP, SteerEntry, SteerFile, parse_steer_layers, probe_axis,
                       probe_fraction)

DEFAULT_OPENINGS = {
    "accept": ["Sure, here is", "Of course! Here is", "Certainly. Let me", "Yes, I can help with that"],
    "decline": ["I'm sorry, but I can't", "I cannot help with", "Sorry, I won't be able to", "I must decline"],
    "plain": ["The answer is", "Here is how", "First,"],
    "hedged": ["It is important to note that", "However, please be aware", "While I can explain, keep in mind"],
}
AUTO_GATE, AUTO_STRENGTH = 0.5, 1.0


def load_openings(path: str | None) -> dict:
    """Lines ``accept: TEXT`` / ``decline: TEXT`` / ``plain: TEXT`` / ``hedged: TEXT``; a kind with no line keeps the
    built-in openings."""
    out = {k: list(v) for k, v in DEFAULT_OPENINGS.items()}
    if not path:
        return out
    seen = {}
    with open(path, encoding="utf-8") as f:
        for line in f:
            kind, sep, text = line.partition(":")
            kind = kind.strip().lower()
            if sep and kind in out and text.strip():
                seen.setdefault(kind, []).append(text.strip())
    out.update(seen)
    return out


@dataclass
class ProbeSettings:
    gate_threshold: float = AUTO_GATE
    edit_strength: float = AUTO_STRENGTH
    hedge_strength: float = -1.0
    directions: int = 1
    keep_norm: bool = False
    push: float = 0.0
    band: tuple = (0, 0)             # layers the probe reads (first, last inclusive)
    edit: tuple = (0, 0)             # layers the clamps edit
    openings: dict = field(default_factory=lambda: {k: list(v) for k, v in DEFAULT_OPENINGS.items()})

    @classmethod
    def from_options(cls, o, n_layers: int, steer_first: int, steer_last: int) -> "ProbeSettings":
        def num(v, auto):
            return auto if str(v).strip().lower() in ("auto", "") else float(v)
        band = parse_steer_layers(getattr(o, "steer_band", "") or "1/3-2/3", n_layers)
        band = (max(band[0], steer_first), min(band[1], steer_last))
        ed = getattr(o, "steer_edit_layers", "") or ""
        edit = parse_steer_layers(ed, n_layers) if ed else band
        edit = (max(edit[0], band[0]), min(edit[1], band[1]))
        return cls(num(getattr(o, "steer_gate_threshold", "auto"), AUTO_GATE), num(getattr(o, "steer_edit_strength", "auto"), AUTO_STRENGTH),
                   float(getattr(o, "steer_hedge_strength", -1.0)), max(1, min(4, int(getattr(o, "steer_directions", 1)))),
                   bool(getattr(o, "steer_keep_norm", False)), float(getattr(o, "steer_push", 0.0)), band, edit,
                   load_openings(getattr(o, "steer_openings", "") or None))


class StateCapture:
    """Hooked into ``SteerTables.apply``: keeps the residual row ``row`` of every band layer of the forward in flight."""

    def __init__(self, tables, band: tuple):
        self.t, self.band, self.row, self.states = tables, band, -1, {}

    def __enter__(self):
        self._orig = self.t.apply

        def apply(hidden, pos, slot, layer):
            if self.band[0] <= layer <= self.band[1] and self.row >= 0:
                self.states[layer] = hidden[self.row].detach().float().cpu().clone()
            return self._orig(hidden, pos, slot, layer)
        self.t.apply = apply
        return self

    def __exit__(self, *exc):
        self.t.apply = self._orig


def _run_rows(engine, slot: int, ids: list[int], pos0: int):
    """An eager forward of ``ids`` at positions pos0.. of ``slot`` (no logits, no graph: the capture hook must run)."""
    n = len(ids)
    engine.kv.reserve(slot, pos0 + n + 1)
    m = engine.model
    b = BatchRows.make(ids, [pos0 + i for i in range(n)], [slot] * n, engine.device, LOGITS_NONE, m.nq // m.nkv,
                       prefill=n > 16, nsplit=1)
    m.forward(b, engine.kv)


def collect_states(engine, tables, slot: int, prompt_len: int, last_prompt_token: int, openings: dict, tokenizer, band: tuple) -> dict:
    """-> {"prompt": {layer: state}, kind: {layer: [n openings, H]}}: the state of the last prompt token and of the last
    token of every opening. The openings' cache rows lie behind the prompt and are overwritten by the reply."""
    out = {}
    with StateCapture(tables, band) as cap:
        cap.row = 0
        _run_rows(engine, slot, [last_prompt_token], prompt_len - 1)          # same values as the prefill wrote
        out["prompt"] = dict(cap.states)
        for kind, texts in openings.items():
            per_layer = {}
            for text in texts:
                ids = tokenizer.encode(text, allow_special=False) if hasattr(tokenizer, "encode") else []
                if not ids:
                    continue
                cap.states, cap.row = {}, len(ids) - 1
                _run_rows(engine, slot, list(ids), prompt_len)
                for layer, st in cap.states.items():
                    per_layer.setdefault(layer, []).append(st)
            out[kind] = {layer: torch.stack(v) for layer, v in per_layer.items()}
    return out


def extra_directions(accept: torch.Tensor, decline: torch.Tensor, first: torch.Tensor, count: int) -> list[torch.Tensor]:
    """The strongest remaining variations of the declining states once ``first`` and the accepting states' own spread are
    projected out (singular vectors of the residual deviations)."""
    if count <= 0 or decline.shape[0] < 2:
        return []
    dev = (decline - decline.mean(0)).double()
    basis = [first.double()] + [r for r in (accept - accept.mean(0)).double()]
    ortho = []
    for v in basis:                                   # Gram-Schmidt of what must not be touched
        for u in ortho:
            v = v - (v @ u) * u
        n = float(v.norm())
        if n > 1e-9:
            ortho.append(v / n)
    for u in ortho:
        dev = dev - (dev @ u)[:, None] * u[None, :]
    _, s, vt = torch.linalg.svd(dev, full_matrices=False)
    return [vt[i].float() for i in range(min(count, vt.shape[0])) if float(s[i]) > 1e-6]


def build_edits(states: dict, cfg: ProbeSettings, hidden: int, n_layers: int) -> tuple[SteerFile | None, dict]:
    """-> (the edits to install or None when the gate stays shut and there is no push, scores for the usage record)."""
    acc, dec = states.get("accept", {}), states.get("decline", {})
    layers = sorted(set(acc) & set(dec))
    if not layers:
        return None, {"gate": 0.0, "fired": False}
    mid = layers[len(layers) // 2]
    axis_mid = probe_axis(acc[mid], dec[mid])
    gate = probe_fraction(axis_mid, states["prompt"][mid]) if mid in states.get("prompt", {}) else 0.0
    fired = gate > cfg.gate_threshold
    scores = {"gate": round(float(gate), 4), "fired": bool(fired), "layer": mid, "threshold": cfg.gate_threshold}
    entries = []
    kind = STEER_CLAMP_KEEP if cfg.keep_norm else STEER_CLAMP
    for layer in layers:
        if not cfg.edit[0] <= layer <= cfg.edit[1]:
            continue
        axis = probe_axis(acc[layer], dec[layer])
        if cfg.push:
            entries.append(SteerEntry(layer, STEER_ADD, cfg.push * (axis.pb - axis.pa), axis.dir.clone()))
        if not fired:
            continue
        entries.append(SteerEntry(layer, kind, axis.pa - cfg.edit_strength * axis.sd, axis.dir.clone()))
        for d in extra_directions(acc[layer], dec[layer], axis.dir, cfg.directions - 1):
            pa = (acc[layer].double() @ d.double())
            entries.append(SteerEntry(layer, kind, float(pa.mean() - cfg.edit_strength * pa.std(unbiased=False)), d))
        pl, hd = states.get("plain", {}).get(layer), states.get("hedged", {}).get(layer)
        if cfg.hedge_strength >= 0 and pl is not None and hd is not None:
            hx = probe_axis(pl, hd)
            entries.append(SteerEntry(layer, kind, hx.pa + cfg.hedge_strength * (hx.pb - hx.pa), hx.dir.clone()))
    per_layer = {}
    kept = []
    for e in entries:                                  # the tables hold four edits per layer
        if per_layer.get(e.layer, 0) < 4:
            per_layer[e.layer] = per_layer.get(e.layer, 0) + 1
            kept.append(e)
    scores["edits"] = len(kept)
    if not kept:
        return None, scores
    return SteerFile(hidden=hidden, layers=n_layers, scope=SCOPE_ALL, scale=1.0, entries=kept), scores


def probe_request(engine, tables, tokenizer, slot: int, prompt: list[int], cfg: ProbeSettings):
    """Runs the whole procedure for the request in ``slot`` (its prompt already in the cache). Returns (SteerFile or None,
    scores)."""
    m = engine.model
    states = collect_states(engine, tables, slot, len(prompt), prompt[-1], cfg.openings, tokenizer, cfg.band)
    return build_edits(states, cfg, m.cfg.hidden, m.cfg.n_layers)


# ---------------------------------------------------------------------------------------------- probe files
def load_probe_files(names: str, steer_dir: str) -> dict:
    """Launch option ``probe``: comma list of probe files inside ``steer_dir`` (at most 4). A probe file is a control-vector
    file whose probe entries (kind 8) name a layer, a unit direction and an offset; its score for a state is the
    projection on the direction minus the offset, averaged over its entries."""
    import os
    from .steering import STEER_PROBE, load_steer_file
    out = {}
    for name in [n.strip() for n in names.split(",") if n.strip()][:4]:
        if "/" in name or name.startswith("."):
            raise ValueError("probe names files inside steer_dir, not paths")
        path = os.path.join(steer_dir, name if name.endswith(".steer") else name + ".steer")
        entries = [e for e in load_steer_file(path).entries if e.kind == STEER_PROBE and e.vec is not None]
        if not entries:
            raise ValueError(f"{path} holds no probe entries")
        out[name] = entries
    return out


def score_probe_files(engine, tables, slot: int, prompt: list[int], probes: dict) -> dict:
    """-> {file: score at the prompt's last token}: the last prompt row runs once more with the capture hook on."""
    layers = sorted({e.layer for es in probes.values() for e in es})
    if not layers:
        return {}
    with StateCapture(tables, (layers[0], layers[-1])) as cap:
        cap.row = 0
        _run_rows(engine, slot, [prompt[-1]], len(prompt) - 1)
        st = dict(cap.states)
    out = {}
    for name, es in probes.items():
        vals = [float(st[e.layer] @ e.vec.float()) - e.par for e in es if e.layer in st]
        if vals:
            out[name] = round(sum(vals) / len(vals), 4)
    return out
