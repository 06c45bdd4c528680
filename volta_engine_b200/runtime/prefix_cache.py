"""Prefix cache: a host-memory tree of sequence snapshots keyed by exact token prefixes, with LRU eviction
over leaves, pinned nodes and an optional disk tier.

Reference behaviour (inc/engine/runtime/prefix_cache.h:12-119, src/runtime/prefix_cache.cpp): a node
stores the state needed to continue after its token segment (here: the KV rows of that segment from the
paged cache); a lookup walks the tree along the prompt and returns the chain of snapshots covering the
longest cached prefix; the disk tier lives in ``<dir>/<fingerprint>/`` and is read back on demand after a
restart. The fingerprint ties the files to one model / option set.
"""
from __future__ import annotations

import hashlib
import os
import queue
import threading
import time
from dataclasses import dataclass, field

import torch


def _digest(tokens) -> str:
    h = hashlib.sha256()
    h.update(b",".join(str(int(t)).encode() for t in tokens))
    return h.hexdigest()[:32]


@dataclass
class Node:
    tokens: tuple                 # segment tokens (after the parent's prefix)
    start: int                    # absolute position of the first token of the segment
    snap: dict | None             # KV rows [start, start + len(tokens)); None when only on disk
    parent: "Node | None" = None
    children: dict = field(default_factory=dict)   # first token -> list[Node]
    pinned: bool = False
    last_used: float = 0.0
    nbytes: int = 0
    key: str = ""                 # digest of the full prefix up to the end of this node

    @property
    def end(self) -> int:
        return self.start + len(self.tokens)


class PrefixCache:
    def __init__(self, budget_bytes: int, disk_dir: str = "", fingerprint: str = "default", disk_budget_bytes: int = 0):
        self.budget = budget_bytes
        self.root = Node((), 0, None)
        self.bytes = 0
        self.entries = 0
        self.stats = {"lookups": 0, "hits": 0, "hit_tokens": 0, "inserts": 0, "evictions": 0,
                      "disk_hits": 0, "disk_entries": 0, "disk_bytes": 0}
        self.lock = threading.Lock()
        self.disk_dir = os.path.join(disk_dir, fingerprint) if disk_dir else ""
        self.disk_budget = int(disk_budget_bytes)          # 0: the disk tier is not trimmed
        self._q: queue.Queue | None = None
        self._writer = None
        if self.disk_dir:
            os.makedirs(self.disk_dir, exist_ok=True)
            self._q = queue.Queue()
            self._writer = threading.Thread(target=self._write_loop, daemon=True)
            self._writer.start()
            self._scan_disk()

    # ------------------------------------------------------------------------------------------- lookup
    def find(self, tokens) -> list[Node]:
        """Chain of nodes (root excluded) whose segments concatenate to the longest cached prefix of ``tokens``.
        At least one prompt token is always left uncached so the caller has a row to run."""
        with self.lock:
            self.stats["lookups"] += 1
            chain, node, pos = [], self.root, 0
            limit = len(tokens) - 1
            while pos < limit:
                nxt = None
                for cand in node.children.get(int(tokens[pos]), []):
                    n = len(cand.tokens)
                    if pos + n <= limit and tuple(int(t) for t in tokens[pos:pos + n]) == cand.tokens:
                        if nxt is None or n > len(nxt.tokens):
                            nxt = cand
                if nxt is None:
                    break
                chain.append(nxt)
                node, pos = nxt, pos + len(nxt.tokens)
            now = time.monotonic()
            for c in chain:
                c.last_used = now
            if chain:
                self.stats["hits"] += 1
                self.stats["hit_tokens"] += pos
            return chain

    def load(self, node: Node) -> dict | None:
        """Snapshot of a node, reading the disk tier when it is not resident."""
        if node.snap is not None:
            return node.snap
        if not self.disk_dir:
            return None
        path = os.path.join(self.disk_dir, node.key + ".pt")
        if not os.path.exists(path):
            return None
        snap = torch.load(path, map_location="cpu", weights_only=True)
        try:
            os.utime(path)             # the disk tier trims by last use
        except OSError:
            pass
        with self.lock:
            self.stats["disk_hits"] += 1
            node.snap = snap["snap"]
            node.nbytes = _snap_bytes(node.snap)
            self.bytes += node.nbytes
            self._evict_locked()
        return node.snap

    # ------------------------------------------------------------------------------------------- insert
    def insert(self, tokens, upto: int, make_snapshot, pinned: bool = False) -> Node | None:
        """Cache the prefix ``tokens[:upto]``. ``make_snapshot(from_pos, to_pos)`` is called for the part that
        is not cached yet and must return the snapshot dict of those rows."""
        chain = self.find(list(tokens[:upto]) + [0])
        with self.lock:
            self.stats["lookups"] -= 1
            if chain:
                self.stats["hits"] -= 1
                self.stats["hit_tokens"] -= chain[-1].end
        parent = chain[-1] if chain else self.root
        start = parent.end if chain else 0
        if upto <= start:
            if pinned and chain:
                chain[-1].pinned = True
            return chain[-1] if chain else None
        seg = tuple(int(t) for t in tokens[start:upto])
        snap = make_snapshot(start, upto)
        node = Node(seg, start, snap, parent, pinned=pinned, last_used=time.monotonic(), nbytes=_snap_bytes(snap),
                    key=_digest(tokens[:upto]))
        with self.lock:
            # the snapshot was taken outside the lock: a parent evicted meanwhile (no disk copy: unlinked from the tree)
            # must not get a child, or the new node would hang off a detached subtree and still be counted
            if parent is not self.root and not self._linked_locked(parent):
                return None
            parent.children.setdefault(seg[0], []).append(node)
            self.bytes += node.nbytes
            self.entries += 1
            self.stats["inserts"] += 1
            self._evict_locked()
        if self._q is not None:
            self._q.put(node)
        return node

    def _linked_locked(self, node) -> bool:
        while node is not None and node is not self.root:
            par = node.parent
            if par is None or node not in par.children.get(node.tokens[0], []):
                return False
            node = par
        return node is self.root

    def _evict_locked(self):
        while self.bytes > self.budget:
            leaves = [n for n in self._iter(self.root) if n.snap is not None and not n.pinned and
                      not any(c.snap is not None for c in self._iter(n) if c is not n)]
            if not leaves:
                return
            victim = min(leaves, key=lambda n: n.last_used)
            self.bytes -= victim.nbytes
            victim.snap, victim.nbytes = None, 0
            self.stats["evictions"] += 1
            if not self.disk_dir:      # without a disk copy the node is gone
                sib = victim.parent.children.get(victim.tokens[0], [])
                if victim in sib and not victim.children:
                    sib.remove(victim)
                    self.entries -= 1

    def _iter(self, node):
        stack = [node]
        while stack:
            n = stack.pop()
            if n is not self.root:
                yield n
            for lst in n.children.values():
                stack.extend(lst)

    # ------------------------------------------------------------------------------------------- disk tier
    def _write_loop(self):
        while True:
            node = self._q.get()
            if node is None:
                return
            snap = node.snap
            if snap is None:
                continue
            path = os.path.join(self.disk_dir, node.key + ".pt")
            tmp = path + ".tmp"
            prefix = []
            n = node
            while n is not None and n is not self.root:
                prefix = list(n.tokens) + prefix
                n = n.parent
            torch.save({"snap": snap, "tokens": prefix, "start": node.start}, tmp)
            os.replace(tmp, path)
            with self.lock:
                self.stats["disk_entries"] += 1
                self.stats["disk_bytes"] += os.path.getsize(path)
            if self.disk_budget > 0 and self.stats["disk_bytes"] > self.disk_budget:
                self._trim_disk(keep=path)

    def _trim_disk(self, keep: str = ""):
        """Remove the least recently used snapshot files until the tier fits its budget. A node whose file went and
        that holds no resident snapshot is unlinked with its subtree (its descendants resume from it)."""
        files = []
        for name in os.listdir(self.disk_dir):
            if name.endswith(".pt"):
                fp = os.path.join(self.disk_dir, name)
                try:
                    st = os.stat(fp)
                except OSError:
                    continue
                files.append((max(st.st_atime, st.st_mtime), st.st_size, fp, name[:-3]))
        files.sort()
        total = sum(f[1] for f in files)
        gone = set()
        for _, size, fp, key in files:
            if total <= self.disk_budget:
                break
            if fp == keep:
                continue
            try:
                os.remove(fp)
            except OSError:
                continue
            total -= size
            gone.add(key)
        with self.lock:
            self.stats["disk_bytes"] = total
            self.stats["disk_entries"] = len(files) - len(gone)
            for node in list(self._iter(self.root)):
                if node.key in gone and node.snap is None and node.parent is not None:
                    sib = node.parent.children.get(node.tokens[0], [])
                    if node in sib:
                        sib.remove(node)
                        self.entries -= sum(1 for _ in self._iter(node)) + 1
                        for sub in self._iter(node):         # resident descendants can no longer be reached
                            if sub.snap is not None:
                                self.bytes -= sub.nbytes
                                sub.snap, sub.nbytes = None, 0

    def _scan_disk(self):
        """Rebuild the tree skeleton from the files of an earlier run (snapshots stay on disk until used)."""
        metas = []
        for name in os.listdir(self.disk_dir):
            if name.endswith(".pt"):
                try:
                    d = torch.load(os.path.join(self.disk_dir, name), map_location="cpu", weights_only=True)
                    metas.append((d["tokens"], d["start"], name[:-3]))
                except Exception:
                    continue
        metas.sort(key=lambda m: len(m[0]))
        for toks, start, key in metas:
            chain = self.find(list(toks) + [0])
            parent = chain[-1] if chain else self.root
            if (parent.end if chain else 0) != start:
                continue
            seg = tuple(int(t) for t in toks[start:])
            if not seg:
                continue
            node = Node(seg, start, None, parent, key=key)
            parent.children.setdefault(seg[0], []).append(node)
            self.entries += 1
            self.stats["disk_entries"] += 1
        self.stats["lookups"] = self.stats["hits"] = self.stats["hit_tokens"] = 0

    def flush(self, timeout: float = 10.0):
        if self._q is None:
            return
        t0 = time.time()
        while not self._q.empty() and time.time() - t0 < timeout:
            time.sleep(0.01)
        time.sleep(0.05)

    def summary(self) -> dict:
        s = dict(self.stats)
        s.update(entries=self.entries, bytes=self.bytes, budget_bytes=self.budget)
        return s


def model_fingerprint(model_dir: str, **facts) -> str:
    """Directory name of the disk tier for one model and option set: hash of ``config.json``, the names, sizes and
    modification times of the weight files, and the facts the caller passes (KV format, head dims, layer count, TP size,
    format version). Snapshots of another checkpoint or cache format then never meet this model's pool."""
    import hashlib
    import json
    h = hashlib.sha256(b"volta-prefix-cache-v2")
    cfg = os.path.join(model_dir or "", "config.json")
    if os.path.exists(cfg):
        with open(cfg, "rb") as f:
            h.update(f.read())
    if model_dir and os.path.isdir(model_dir):
        for name in sorted(os.listdir(model_dir)):
            if name.endswith((".safetensors", ".gguf", ".bin")):
                st = os.stat(os.path.join(model_dir, name))
                h.update(f"{name}:{st.st_size}:{int(st.st_mtime)}".encode())
    h.update(json.dumps(facts, sort_keys=True, default=str).encode())
    return h.hexdigest()[:24]


def _snap_bytes(snap: dict) -> int:
    return sum(v.numel() * v.element_size() for v in snap.values() if isinstance(v, torch.Tensor))
