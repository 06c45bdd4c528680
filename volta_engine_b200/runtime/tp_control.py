"""Multi-rank serving control: rank 0 hosts the scheduler and replicates every engine call to the other ranks,
which execute the same call on their own shard; plus host-side failure detection between launches.

Design: the scheduler talks to a ``LeaderEngine`` with the same surface as ``Engine``. Each call is first
published as a small pickled command on a CPU (gloo) group, then executed locally; followers sit in
``follower_loop`` and mirror it. Device work of all ranks therefore enters the collectives in the same order.
KV snapshots stay rank-local: the leader's cache holds handles, followers keep the matching rows.
Failure detection never touches the GPU: every rank publishes a heartbeat in the rendezvous store from a host
thread; the leader checks the peers' heartbeats before each launch and raises ``RankFailure`` instead of entering
a collective with a missing peer; a follower that stops hearing commands leaves after ``idle_timeout``.
Reference: src/runtime/cluster.cpp:26-219 (rank pool driving one pipeline per GPU), src/runtime/rank_pool.cpp
(persistent rank threads with a command mailbox); the reference runs ranks as threads of one process, here they
are processes and the mailbox is this channel.
"""
from __future__ import annotations

import threading
import time

import torch.distributed as dist


class RankFailure(RuntimeError):
    """A peer rank stopped answering (heartbeat too old, or the control channel timed out)."""


class Heartbeat:
    """Per-rank liveness in a key/value store (``torch.distributed`` TCPStore / FileStore / HashStore)."""

    def __init__(self, store, rank: int, size: int, period_s: float = 0.2, timeout_s: float = 2.0):
        self.store, self.rank, self.size = store, rank, size
        self.period, self.timeout = period_s, timeout_s
        self._stop = threading.Event()
        self._thread = None
        self.beat()

    def beat(self):
        self.store.set(f"hb/{self.rank}", repr(time.time()))

    def start(self):
        def run():
            while not self._stop.wait(self.period):
                try:
                    self.beat()
                except Exception:
                    return
        self._thread = threading.Thread(target=run, daemon=True, name="volta-heartbeat")
        self._thread.start()
        return self

    def stop(self):
        self._stop.set()
        if self._thread:
            self._thread.join(timeout=1.0)

    def age(self, rank: int) -> float:
        try:
            return time.time() - float(self.store.get(f"hb/{rank}").decode())
        except Exception:
            return float("inf")

    def dead_ranks(self) -> list[int]:
        return [r for r in range(self.size) if r != self.rank and self.age(r) > self.timeout]

    def check(self):
        dead = self.dead_ranks()
        if dead:
            raise RankFailure(f"rank(s) {dead} missed their heartbeat for more than {self.timeout:.1f} s")


class ControlChannel:
    """Rank-0 -> all command broadcast on a CPU group."""

    def __init__(self, group=None, heartbeat: Heartbeat | None = None):
        self.group = group
        self.rank = dist.get_rank(group)
        self.size = dist.get_world_size(group)
        self.heartbeat = heartbeat

    def send(self, cmd):
        if self.heartbeat is not None:
            self.heartbeat.check()
        try:
            dist.broadcast_object_list([cmd], src=0, group=self.group)
        except RuntimeError as e:        # gloo timeout / connection reset: a peer is gone
            raise RankFailure(f"control channel: {e}") from e

    def recv(self):
        box = [None]
        try:
            dist.broadcast_object_list(box, src=0, group=self.group)
        except RuntimeError as e:
            raise RankFailure(f"control channel: {e}") from e
        return box[0]


class _SnapHandle:
    """Sits inside a leader-side snapshot; when the cache drops the snapshot the followers are told to drop theirs."""

    def __init__(self, owner, hid: int):
        self.owner, self.hid = owner, hid

    def __del__(self):
        try:
            self.owner._drops.append(self.hid)
        except Exception:
            pass

    def __reduce__(self):                # a pickled snapshot (disk tier) carries no live handle
        return (int, (self.hid,))


_ENGINE_CALLS = ("prefill", "prefill_rows", "step", "step_candidates", "decode_chain", "set_rows")
_KV_CALLS = ("reserve", "release")


class _LeaderKV:
    def __init__(self, owner, kv):
        self._o, self._kv = owner, kv

    def __getattr__(self, name):
        attr = getattr(self._kv, name)
        if name in _KV_CALLS:
            def call(*a, **k):
                self._o._publish(("kv." + name, a, k))
                return attr(*a, **k)
            return call
        return attr

    def save_rows(self, slot, a, b):
        hid = self._o._next_handle()
        self._o._publish(("kv.save_rows", (slot, a, b), {"hid": hid}))
        snap = self._kv.save_rows(slot, a, b)
        snap["_h"] = _SnapHandle(self._o, hid)
        return snap

    def load_rows(self, slot, snap):
        h = snap.get("_h")
        if not isinstance(h, _SnapHandle):
            raise RankFailure("snapshot has no live handle on the follower ranks")
        self._o._publish(("kv.load_rows", (slot,), {"hid": h.hid}))
        return self._kv.load_rows(slot, snap)


class LeaderEngine:
    """``Engine`` front on rank 0: publishes each call, then runs it."""

    def __init__(self, engine, chan: ControlChannel):
        self._e, self._chan = engine, chan
        self._drops: list[int] = []
        self._hid = 0
        self.kv = _LeaderKV(self, engine.kv)

    def _next_handle(self) -> int:
        self._hid += 1
        return self._hid

    def _publish(self, cmd):
        drops, self._drops = self._drops, []
        self._chan.send((cmd, drops))

    def __getattr__(self, name):
        attr = getattr(self._e, name)
        if name in _ENGINE_CALLS:
            def call(*a, **k):
                self._publish((name, a, k))
                return attr(*a, **k)
            return call
        return attr

    def shutdown(self):
        self._publish(("stop", (), {}))


_DRAFTER_CALLS = ("draft", "release", "ingest", "observe_prompt", "observe_commit")


class LeaderDrafter:
    """A tensor-parallel block drafter on rank 0: every call that runs the drafter's model (or changes its per-slot state)
    is published first, so the follower ranks make the same call on their shard (``follower_loop`` routes names that
    start with ``drafter.`` to ``engine.drafter``)."""

    def __init__(self, drafter, leader: LeaderEngine):
        self._d, self._lead = drafter, leader

    def __getattr__(self, name):
        attr = getattr(self._d, name)
        if name in _DRAFTER_CALLS:
            def call(*a, **k):
                self._lead._publish(("drafter." + name, a, k))
                return attr(*a, **k)
            return call
        return attr


def follower_loop(engine, chan: ControlChannel, on_command=None) -> int:
    """Mirror the leader's calls until it says stop. Returns the number of commands executed."""
    snaps: dict[int, dict] = {}
    n = 0
    while True:
        (name, a, k), drops = chan.recv()
        for hid in drops:
            snaps.pop(hid, None)
        if name == "stop":
            return n
        if on_command is not None:
            on_command(name, a, k)
        if name == "kv.save_rows":
            snaps[k["hid"]] = engine.kv.save_rows(*a)
        elif name == "kv.load_rows":
            engine.kv.load_rows(a[0], snaps[k["hid"]])
        elif name.startswith("kv."):
            getattr(engine.kv, name[3:])(*a, **k)
        elif name.startswith("drafter."):
            getattr(engine.drafter, name[8:])(*a, **k)
        else:
            getattr(engine, name)(*a, **k)
        n += 1
