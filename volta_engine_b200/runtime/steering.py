"""Runtime steering: control-vector files, per-slot device tables, the residual edit after steered layers, the
reasoning-marker logit penalty, and the host maths of the steering probe.

File (``.steer``, little-endian): ``VSTR``, int32 version (1-3), hidden, model layers, default scope bits, entries,
[version >= 2: float scale], then per entry int32 layer, int32 kind, float par, [version 3: int32 expert],
float vec[hidden] (no vector for a router entry).
Reference: inc/engine/runtime/steer_file.h:10-28, src/runtime/steer_file.cpp (format, layer / scope specs),
inc/engine/modules/steer.h:11-80 (kinds, scopes, tables), inc/engine/runtime/steer_probe.h (probe axes).
"""
from __future__ import annotations

import struct
from dataclasses import dataclass, field

import torch

from .._lib import call, ptr

STEER_OFF, STEER_ADD, STEER_CLAMP, STEER_CLAMP_KEEP, STEER_PROBE, STEER_ROUTE = 0, 1, 2, 3, 8, 9
SCOPE_PROMPT, SCOPE_THINK, SCOPE_ANSWER, SCOPE_GENERATED, SCOPE_ALL = 1, 2, 4, 6, 7
ENTRIES_PER_LAYER = 4
PENALTY_IDS = 256
INT_MAX = 2 ** 31 - 1


@dataclass
class SteerEntry:
    layer: int = 0
    kind: int = STEER_ADD
    par: float = 0.0
    vec: torch.Tensor | None = None
    expert: int = -1


@dataclass
class SteerFile:
    hidden: int = 0
    layers: int = 0
    scope: int = SCOPE_ALL
    scale: float = 1.0
    entries: list = field(default_factory=list)


def load_steer_file(path) -> SteerFile:
    with open(path, "rb") as f:
        data = f.read()
    if len(data) < 24 or data[:4] != b"VSTR":
        raise ValueError(f"{path}: not a control-vector file")
    ver, hidden, layers, scope, n = struct.unpack_from("<5i", data, 4)
    if not 1 <= ver <= 3:
        raise ValueError(f"{path}: not a control-vector file (version 1 to 3)")
    off = 24
    scale = 1.0
    if ver >= 2:
        (scale,) = struct.unpack_from("<f", data, off)
        off += 4
    if hidden <= 0 or hidden > 65536 or n < 0 or n > 4096:
        raise ValueError(f"{path}: bad header")
    out = SteerFile(hidden, layers, scope, scale)
    try:
        for _ in range(n):
            layer, kind, par = struct.unpack_from("<iif", data, off)
            off += 12
            expert = -1
            if ver >= 3:
                (expert,) = struct.unpack_from("<i", data, off)
                off += 4
            vec = None
            if kind != STEER_ROUTE:
                if off + 4 * hidden > len(data):
                    raise struct.error
                vec = torch.frombuffer(bytearray(data[off:off + 4 * hidden]), dtype=torch.float32).clone()
                off += 4 * hidden
            out.entries.append(SteerEntry(layer, kind, par, vec, expert))
    except struct.error:
        raise ValueError(f"{path}: truncated") from None
    return out


def save_steer_file(path, sf: SteerFile):
    v3 = any(e.kind == STEER_ROUTE for e in sf.entries)
    blob = bytearray(b"VSTR" + struct.pack("<5i", 3 if v3 else 2, sf.hidden, sf.layers, sf.scope, len(sf.entries)))
    blob += struct.pack("<f", sf.scale)
    for e in sf.entries:
        blob += struct.pack("<iif", e.layer, e.kind, e.par)
        if v3:
            blob += struct.pack("<i", e.expert)
        if e.kind != STEER_ROUTE:
            blob += e.vec.detach().float().cpu().contiguous().numpy().tobytes()
    with open(path, "wb") as f:
        f.write(blob)


def parse_steer_scope(spec: str) -> int:
    words = {"prompt": SCOPE_PROMPT, "think": SCOPE_THINK, "answer": SCOPE_ANSWER, "generated": SCOPE_GENERATED, "all": SCOPE_ALL}
    bits = 0
    for w in spec.split(","):
        if not w:
            continue
        if w not in words:
            raise ValueError(f"unknown steering scope '{w}'")
        bits |= words[w]
    if bits == 0:
        raise ValueError("empty steering scope")
    return bits


def _layer_token(t: str, n: int) -> int:
    if t == "last":
        return n - 1
    if "/" in t:
        a, b = t.split("/", 1)
        return int(round(float(a) / float(b) * n))
    return int(round(float(t) * n)) if "." in t else int(t)


def parse_steer_layers(spec: str, n_layers: int) -> tuple[int, int]:
    """"first-last": each side an index, a fraction of the layer count (0.33, 1/3) or "last"; empty = 1/3 - 2/3."""
    if not spec:
        return int(round(n_layers / 3.0)), int(round(n_layers * 2.0 / 3.0))
    if "-" not in spec:
        raise ValueError(f"steer_layers '{spec}': expected first-last")
    a, b = spec.split("-", 1)
    try:
        first, last = _layer_token(a, n_layers), _layer_token(b, n_layers)
    except (ValueError, ZeroDivisionError):
        raise ValueError(f"steer_layers '{spec}' is malformed") from None
    if not (0 <= first <= last < n_layers):
        raise ValueError(f"steer_layers '{spec}' is outside 0..{n_layers - 1}")
    return first, last


class SteerTables:
    """Device state: vec [slots][layers][4][hidden] fp32, par / kind [slots][layers][4], ctl [slots][8] int32
    (scope, prompt_len, think_end, penalty_n, penalty (float bits), pad x3), penalty ids [slots][256]."""

    def __init__(self, hidden: int, first_layer: int, last_layer: int, slots: int, device):
        self.hidden, self.first, self.layers, self.slots = hidden, first_layer, last_layer - first_layer + 1, slots
        self.device = torch.device(device)
        z = lambda *s, dt=torch.float32: torch.zeros(*s, dtype=dt, device=self.device)
        self.vec = z(slots, self.layers, ENTRIES_PER_LAYER, hidden)
        self.par = z(slots, self.layers, ENTRIES_PER_LAYER)
        self.kind = z(slots, self.layers, ENTRIES_PER_LAYER, dt=torch.int32)
        self.ctl = z(slots, 8, dt=torch.int32)
        self.penalty_ids = z(slots, PENALTY_IDS, dt=torch.int32)

    def clear_slot(self, slot: int):
        self.kind[slot].zero_()
        self.ctl[slot].zero_()

    def set_slot(self, slot: int, sf: SteerFile, prompt_len: int, scale: float = 1.0, scope: int | None = None,
                 think_end: int = INT_MAX, penalty_ids=(), penalty: float = 0.0):
        if sf is not None and sf.hidden != self.hidden:
            raise ValueError(f"control vectors are for hidden {sf.hidden}, the model has {self.hidden}")
        self.clear_slot(slot)
        used = {}
        for e in (sf.entries if sf is not None else []):
            if e.kind in (STEER_ROUTE, STEER_PROBE) or not self.first <= e.layer < self.first + self.layers:
                continue
            li = e.layer - self.first
            k = used.get(li, 0)
            if k >= ENTRIES_PER_LAYER:
                raise ValueError(f"more than {ENTRIES_PER_LAYER} edits on layer {e.layer}")
            used[li] = k + 1
            self.vec[slot, li, k].copy_(e.vec)
            self.par[slot, li, k] = e.par * (sf.scale * scale if e.kind == STEER_ADD else 1.0)
            self.kind[slot, li, k] = e.kind
        ids = list(penalty_ids)[:PENALTY_IDS]
        if ids:
            self.penalty_ids[slot, :len(ids)] = torch.tensor(ids, dtype=torch.int32)
        pbits = struct.unpack("<i", struct.pack("<f", float(penalty)))[0]
        sc = scope if scope is not None else (sf.scope if sf is not None else 0)
        self.ctl[slot] = torch.tensor([sc if used else 0, prompt_len, think_end, len(ids), pbits, 0, 0, 0], dtype=torch.int32)

    def set_think_end(self, slot: int, pos: int):
        self.ctl[slot, 2] = pos

    # ------------------------------------------------------------------------------------------ application
    def apply(self, hidden: torch.Tensor, pos: torch.Tensor, slot: torch.Tensor, layer: int):
        """Edit the residual rows after model layer ``layer`` (no-op outside the steered range)."""
        if not self.first <= layer < self.first + self.layers:
            return hidden
        li = layer - self.first
        if hidden.is_cuda:
            call("steer_apply", "plpppppp" + "iiii", ptr(hidden), hidden.stride(0), ptr(pos), ptr(slot), ptr(self.ctl),
                 ptr(self.vec), ptr(self.par), ptr(self.kind), hidden.shape[0], self.layers, li, self.hidden)
            return hidden
        for r in range(hidden.shape[0]):
            s = int(slot[r])
            if s < 0:
                continue
            scope, plen, tend = (int(v) for v in self.ctl[s, :3])
            p = int(pos[r])
            bit = SCOPE_PROMPT if p < plen else (SCOPE_THINK if p < tend else SCOPE_ANSWER)
            if not scope & bit:
                continue
            x = hidden[r].float()
            for k in range(ENTRIES_PER_LAYER):
                kind = int(self.kind[s, li, k])
                if kind == STEER_OFF:
                    continue
                v, par = self.vec[s, li, k], float(self.par[s, li, k])
                if kind == STEER_ADD:
                    x = (x + par * v).to(hidden.dtype).float()
                    continue
                over = max(float(x @ v) - par, 0.0)
                if over <= 0:
                    continue
                y = x - over * v
                if kind == STEER_CLAMP_KEEP and float(y.norm()) > 0:
                    y = y * (x.norm() / y.norm())
                x = y.to(hidden.dtype).float()
            hidden[r] = x.to(hidden.dtype)
        return hidden

    def penalize(self, logits: torch.Tensor, pos: torch.Tensor, slot: torch.Tensor, id0: int = 0):
        if logits.is_cuda:
            call("steer_penalize", "plpppp" + "iiii", ptr(logits), logits.stride(0), ptr(pos), ptr(slot), ptr(self.ctl),
                 ptr(self.penalty_ids), PENALTY_IDS, id0, logits.shape[1], logits.shape[0])
            return logits
        for r in range(logits.shape[0]):
            s = int(slot[r])
            if s < 0:
                continue
            _, plen, tend, n, pbits = (int(v) for v in self.ctl[s, :5])
            p = int(pos[r]) + 1
            if n <= 0 or p < plen or p >= tend:
                continue
            pen = struct.unpack("<f", struct.pack("<i", pbits))[0]
            for t in self.penalty_ids[s, :n].tolist():
                if id0 <= t < id0 + logits.shape[1]:
                    logits[r, t - id0] -= pen
        return logits


# ---------------------------------------------------------------------------------------------- probe maths
@dataclass
class ProbeAxis:
    dir: torch.Tensor
    pa: float = 0.0
    pb: float = 0.0
    sd: float = 0.0


def probe_axis(a: torch.Tensor, b: torch.Tensor, orthogonalize: bool = False) -> ProbeAxis:
    """Unit direction from the mean of state set ``a`` [na, H] to the mean of ``b`` [nb, H]; with ``orthogonalize`` the
    direction is first stripped of what varies inside ``a`` (its samples' deviations, projected out one after the other)."""
    a, b = a.double(), b.double()
    ma = a.mean(0)
    d = b.mean(0) - ma
    if orthogonalize:
        for row in a - ma:
            n = float(row @ row)
            if n > 1e-20:
                d = d - (d @ row) / n * row
    n = float(d.norm())
    d = d / n if n > 0 else d
    pa_all = a @ d
    return ProbeAxis(d.float(), float(pa_all.mean()), float((b @ d).mean()), float(pa_all.std(unbiased=False)))


def probe_fraction(axis: ProbeAxis, state: torch.Tensor) -> float:
    """0 at a's mean, 1 at b's mean along the axis (the gap floored so a degenerate axis does not blow up)."""
    gap = axis.pb - axis.pa
    gap = gap if abs(gap) > 1e-6 else (1e-6 if gap >= 0 else -1e-6)
    return (float(state.float() @ axis.dir) - axis.pa) / gap


# ---------------------------------------------------------------------------------------------- launch configuration
class SteerConfig:
    """What the launch options say about steering, resolved once: mode (off | on | file), the default control-vector
    file, the directory requests may name files in, scale / scope defaults and the reasoning-marker penalty.
    ``for_request`` turns a request's steering fields into the arguments of ``SteerTables.set_slot``.
    Reference: docs/CONFIG.md (``steer``, ``steer_layers``, ``steer_file``, ``steer_dir``, ``steer_scale``,
    ``steer_scope``, ``think_penalty``, ``think_penalty_words``)."""

    DEFAULT_WORDS = ("Wait", " Wait", "Hmm", " Hmm", "Alternatively", " Alternatively", "But wait", " But wait")

    def __init__(self, options, n_layers: int, tokenizer=None):
        self.mode = str(getattr(options, "steer", "off") or "off").lower()
        if self.mode not in ("off", "on", "file"):
            raise ValueError(f"steer = '{self.mode}': off, on or file")
        self.first, self.last = parse_steer_layers(getattr(options, "steer_layers", "") or "1/3-2/3", n_layers)
        self.dir = getattr(options, "steer_dir", "") or ""
        self.scale = float(getattr(options, "steer_scale", 1.0))
        sc = getattr(options, "steer_scope", "") or ""
        self.scope = parse_steer_scope(sc) if sc else None
        self.default = None
        path = getattr(options, "steer_file", "") or ""
        if self.mode == "file":
            if not path:
                raise ValueError("steer = file needs steer_file")
            self.default = load_steer_file(path)
        elif path and self.mode == "on":
            self.default_path = path
        self.penalty = float(getattr(options, "think_penalty", 0.0) or 0.0)
        words = getattr(options, "think_penalty_words", "") or ""
        words = [w for w in words.split("|") if w] if words else list(self.DEFAULT_WORDS)
        self.penalty_ids = []
        if tokenizer is not None:
            for w in words:
                ids = tokenizer.encode(w, allow_special=False) if hasattr(tokenizer, "encode") else []
                if ids and ids[0] not in self.penalty_ids:
                    self.penalty_ids.append(ids[0])              # the first token of a marker is what gets the penalty
        self._files: dict = {}

    @property
    def enabled(self) -> bool:
        return self.mode != "off"

    def tables(self, hidden: int, slots: int, device) -> "SteerTables":
        return SteerTables(hidden, self.first, self.last, slots, device)

    def _named(self, name: str) -> SteerFile:
        if not self.dir:
            raise ValueError("the server has no steer_dir: requests cannot name control-vector files")
        if "/" in name or "\\" in name or name.startswith("."):
            raise ValueError("steer_vector is a file name inside steer_dir, not a path")
        sf = self._files.get(name)
        if sf is None:
            import os
            sf = self._files[name] = load_steer_file(os.path.join(self.dir, name if name.endswith(".steer") else name + ".steer"))
        return sf

    def for_request(self, fields: dict) -> dict:
        """-> keyword arguments for the request: steer (SteerFile or None), steer_scale, steer_scope, think_penalty."""
        out = {"steer": self.default, "steer_scale": self.scale, "steer_scope": self.scope, "think_penalty": self.penalty}
        if not self.enabled:
            return dict(out, steer=None, think_penalty=0.0)
        name = fields.get("steer_vector")
        if name is not None:
            out["steer"] = None if name.lower() in ("off", "none", "") else self._named(name)
        if "steer_scale" in fields:
            out["steer_scale"] = float(fields["steer_scale"])
        if "steer_scope" in fields:
            out["steer_scope"] = parse_steer_scope(fields["steer_scope"])
        if "think_penalty" in fields:
            out["think_penalty"] = float(fields["think_penalty"])
        if fields.get("steer_probe"):
            out["steer_probe"] = True
        return out
