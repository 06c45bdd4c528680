"""Offline-training dumps of the speculation path.

``CandLog``: a binary log of the block drafter's candidates, one record per speculation round and one per finished request,
so a candidate re-ranker can be trained and tested offline. Little endian:
    round    int32 0xC0DE0001, slot, pos, anchor, active, valid, then per valid position: chosen, target (int32),
             16 float32 candidate values, 16 int32 candidate ids   (valid = the positions up to the first mismatch)
    request  int32 0xC0DE0002, slot, n_tokens, then n_tokens int32 (prompt and output)
``TargetSpool``: the target's top-k candidates at the positions a round emitted, kept per slot and taken (with the request's
taps) when the request finishes, so a drafter can be trained against the target's distribution and not its tokens alone.

``TapSpool``: the file those two feed. One record per finished request, little endian:
    int32 0xC0DE0003, n_tokens, first_pos, n_pos, width, n_targets; n_tokens int32 (prompt and output);
    n_pos x width fp16 (the drafter taps of positions first_pos .. first_pos + n_pos - 1, width = taps x hidden);
    n_targets x (int32 pos, 16 float32 values, 16 int32 ids)

Reference: inc/engine/runtime/cand_log.h:10-40, inc/engine/runtime/target_spool.h:11-40; docs/CONFIG.md:192-193 (tap_spool).
"""
from __future__ import annotations

import struct
import threading

ROUND_MAGIC, REQUEST_MAGIC, TAPS_MAGIC = 0xC0DE0001, 0xC0DE0002, 0xC0DE0003
CANDS = 16


class CandLog:
    def __init__(self):
        self._f = None
        self._lock = threading.Lock()

    def open(self, path) -> bool:
        with self._lock:
            if self._f is None:
                try:
                    self._f = open(path, "wb")
                except OSError:
                    return False
        return True

    def on(self) -> bool:
        return self._f is not None

    def round(self, slot: int, pos: int, anchor: int, active: int, rows) -> None:
        """``rows``: per valid position (chosen, target, values[16], ids[16])."""
        if self._f is None:
            return
        buf = [struct.pack("<Iiiiii", ROUND_MAGIC, slot, pos, anchor, active, len(rows))]
        for chosen, target, vals, ids in rows:
            vals, ids = list(vals)[:CANDS], list(ids)[:CANDS]
            vals += [float("-inf")] * (CANDS - len(vals))
            ids += [-1] * (CANDS - len(ids))
            buf.append(struct.pack("<ii16f16i", chosen, target, *vals, *ids))
        with self._lock:
            self._f.write(b"".join(buf))

    def request(self, slot: int, tokens) -> None:
        if self._f is None:
            return
        with self._lock:
            self._f.write(struct.pack(f"<Iii{len(tokens)}i", REQUEST_MAGIC, slot, len(tokens), *tokens))

    def flush(self) -> None:
        with self._lock:
            if self._f is not None:
                self._f.flush()

    def close(self) -> None:
        with self._lock:
            if self._f is not None:
                self._f.close()
                self._f = None


def read_cand_log(path) -> list[dict]:
    """Parses a candidate log back into records (for tests and offline tools)."""
    out = []
    with open(path, "rb") as f:
        data = f.read()
    at = 0
    while at + 4 <= len(data):
        (magic,) = struct.unpack_from("<I", data, at)
        if magic == ROUND_MAGIC:
            slot, pos, anchor, active, valid = struct.unpack_from("<iiiii", data, at + 4)
            at += 24
            rows = []
            for _ in range(valid):
                v = struct.unpack_from("<ii16f16i", data, at)
                rows.append({"chosen": v[0], "target": v[1], "vals": list(v[2:18]), "ids": list(v[18:34])})
                at += 8 + 64 + 64
            out.append({"kind": "round", "slot": slot, "pos": pos, "anchor": anchor, "active": active, "rows": rows})
        elif magic == REQUEST_MAGIC:
            slot, n = struct.unpack_from("<ii", data, at + 4)
            toks = list(struct.unpack_from(f"<{n}i", data, at + 12))
            at += 12 + 4 * n
            out.append({"kind": "request", "slot": slot, "tokens": toks})
        else:
            raise ValueError(f"candidate log: unknown record 0x{magic:08x} at byte {at}")
    return out


class TargetSpool:
    def __init__(self):
        self._on = False
        self._lock = threading.Lock()
        self._rows: dict[int, list] = {}

    def enable(self) -> None:
        self._on = True

    def on(self) -> bool:
        return self._on

    def add(self, slot: int, pos: int, vals, ids) -> None:
        """The target's candidates for the token at ``pos`` (the position these logits predict)."""
        if not self._on:
            return
        with self._lock:
            self._rows.setdefault(slot, []).append((pos, list(vals), list(ids)))

    def take(self, slot: int) -> list:
        with self._lock:
            return self._rows.pop(slot, [])


class TapSpool:
    """Appends a record per finished request: its tokens, the drafter taps of its last ``window`` positions and the target's
    candidates at the positions speculation emitted."""

    def __init__(self, path, window: int = 768):
        self.path, self.window = path, max(1, int(window))
        self._lock = threading.Lock()
        self.records = 0

    def write(self, tokens, taps, first_pos: int, targets) -> None:
        """taps: tensor [n_pos, width] (any float type) or None; targets: [(pos, vals, ids)] from ``TargetSpool.take``."""
        import torch
        n_pos, width = (int(taps.shape[0]), int(taps.shape[1])) if taps is not None else (0, 0)
        blob = [struct.pack("<Iiiiii", TAPS_MAGIC, len(tokens), int(first_pos), n_pos, width, len(targets)),
                struct.pack(f"<{len(tokens)}i", *[int(t) for t in tokens])]
        if n_pos:
            blob.append(taps.detach().to("cpu", torch.float16).contiguous().numpy().tobytes())
        for pos, vals, ids in targets:
            v = (list(vals) + [0.0] * CANDS)[:CANDS]
            i = (list(ids) + [-1] * CANDS)[:CANDS]
            blob.append(struct.pack("<i16f16i", int(pos), *[float(x) for x in v], *[int(x) for x in i]))
        with self._lock:
            with open(self.path, "ab") as f:
                f.write(b"".join(blob))
            self.records += 1


def read_tap_spool(path) -> list[dict]:
    import numpy as np
    out, at = [], 0
    with open(path, "rb") as f:
        data = f.read()
    while at + 24 <= len(data):
        magic, n_tok, first, n_pos, width, n_tgt = struct.unpack_from("<Iiiiii", data, at)
        if magic != TAPS_MAGIC:
            raise ValueError(f"tap spool: unknown record 0x{magic:08x} at byte {at}")
        at += 24
        toks = list(struct.unpack_from(f"<{n_tok}i", data, at))
        at += 4 * n_tok
        taps = np.frombuffer(data, dtype=np.float16, count=n_pos * width, offset=at).reshape(n_pos, width).copy()
        at += 2 * n_pos * width
        tg = []
        for _ in range(n_tgt):
            v = struct.unpack_from("<i16f16i", data, at)
            tg.append({"pos": v[0], "vals": list(v[1:17]), "ids": list(v[17:33])})
            at += 4 + 64 + 64
        out.append({"tokens": toks, "first_pos": first, "taps": taps, "targets": tg})
    return out
