"""Offline-training dumps of the speculation path.

``CandLog``: a binary log of the block drafter's candidates, one record per speculation round and one per finished request,
so a candidate re-ranker can be trained and tested offline. Little endian:
    round    int32 0xC0DE0001, slot, pos, anchor, active, valid, then per valid position: chosen, target (int32),
             16 float32 candidate values, 16 int32 candidate ids   (valid = the positions up to the first mismatch)
    request  int32 0xC0DE0002, slot, n_tokens, then n_tokens int32 (prompt and output)
``TargetSpool``: the target's top-k candidates at the positions a round emitted, kept per slot and taken (with the request's
taps) when the request finishes, so a drafter can be trained against the target's distribution and not its tokens alone.

Reference: inc/engine/runtime/cand_log.h:10-40, inc/engine/runtime/target_spool.h:11-40.
"""
from __future__ import annotations

import struct
import threading

ROUND_MAGIC, REQUEST_MAGIC = 0xC0DE0001, 0xC0DE0002
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
