"""Device memory arena and named scratch registry.

``Arena``: one allocation per GPU at start-up, bump-pointer sub-allocation, nothing is allocated while decoding, so
pointers stay stable for CUDA-graph replay and the caching allocator is never entered on the hot path. A pinned
host variant holds data the GPU reads in place (cold experts, host embedding tables).
``ScratchRegistry``: named persistent workspaces carved from the arena (split-K partials, reconstructed weights,
attention partials); asking again for a name returns the same memory, asking for more grows it once.
Reference: inc/engine/core/arena.h, inc/engine/core/scratch.h (boot-time cudaMalloc, bump allocation, named scratch).
"""
from __future__ import annotations

import math

import torch

_ALIGN = 256


class ArenaError(MemoryError):
    pass


class Arena:
    def __init__(self, nbytes: int, device="cuda:0", pinned: bool = False):
        self.device = torch.device("cpu") if pinned else torch.device(device)
        self.pinned = pinned
        self.capacity = int(nbytes)
        if pinned:
            self.buf = torch.empty(self.capacity, dtype=torch.uint8, pin_memory=torch.cuda.is_available())
        else:
            self.buf = torch.empty(self.capacity, dtype=torch.uint8, device=self.device)
        self.top = 0
        self.high_water = 0
        self.frozen = False
        self.log: list[tuple[str, int]] = []

    @classmethod
    def from_free_memory(cls, device, reserve_mib: int = 2048, fraction: float = 1.0):
        """Size the arena from the device's free memory minus a reserve (graphs, library workspaces)."""
        free, _ = torch.cuda.mem_get_info(torch.device(device))
        return cls(max(0, int((free - (reserve_mib << 20)) * fraction)), device)

    def alloc(self, shape, dtype=torch.uint8, name: str = "") -> torch.Tensor:
        if self.frozen:
            raise ArenaError(f"arena is frozen (serving): allocation '{name}' refused")
        shape = tuple(int(s) for s in (shape if isinstance(shape, (tuple, list)) else (shape,)))
        n = math.prod(shape) * torch.empty((), dtype=dtype).element_size()
        base = self.buf.data_ptr()
        start = (base + self.top + _ALIGN - 1) // _ALIGN * _ALIGN - base        # aligned address, not just offset
        if start + n > self.capacity:
            raise ArenaError(f"arena exhausted: '{name}' needs {n} B, {self.capacity - start} B left of {self.capacity}")
        self.top = start + n
        self.high_water = max(self.high_water, self.top)
        self.log.append((name, n))
        return self.buf[start:start + n].view(dtype).reshape(shape)

    def mark(self) -> int:
        return self.top

    def release_to(self, mark: int):
        """Drop everything allocated after ``mark`` (load-time temporaries)."""
        if self.frozen:
            raise ArenaError("arena is frozen")
        self.top = mark

    def freeze(self):
        """Called when loading is done: later allocations are programming errors."""
        self.frozen = True

    def free_bytes(self) -> int:
        return self.capacity - self.top

    def report(self) -> dict:
        by = {}
        for n, b in self.log:
            key = n.split("/")[0] or "unnamed"
            by[key] = by.get(key, 0) + b
        return {"capacity": self.capacity, "used": self.top, "high_water": self.high_water, "by_name": by}


class ScratchRegistry:
    def __init__(self, arena: Arena | None = None, device="cuda:0", overflow: bool = False):
        """``overflow``: a workspace that no longer fits the arena is allocated by itself (and counted in
        ``overflow_bytes``) instead of raising."""
        self.arena, self.device = arena, torch.device(device if arena is None else arena.device)
        self.items: dict[str, torch.Tensor] = {}
        self.overflow, self.overflow_bytes = overflow, 0

    def get(self, name: str, nbytes: int) -> torch.Tensor:
        """uint8 workspace of at least ``nbytes``; the same tensor for the same name on every call."""
        t = self.items.get(name)
        if t is not None and t.numel() >= nbytes:
            return t
        if t is not None and self.arena is not None and self.arena.frozen:
            raise ArenaError(f"scratch '{name}' would grow from {t.numel()} to {nbytes} B after start-up")
        if self.arena is not None:
            try:
                t = self.arena.alloc(nbytes, torch.uint8, f"scratch/{name}")
            except ArenaError:
                if not self.overflow:
                    raise
                self.overflow_bytes += nbytes
                t = torch.empty(nbytes, dtype=torch.uint8, device=self.device)
        else:
            t = torch.empty(nbytes, dtype=torch.uint8, device=self.device)
        self.items[name] = t
        return t

    def typed(self, name: str, shape, dtype) -> torch.Tensor:
        shape = tuple(shape)
        n = math.prod(shape) * torch.empty((), dtype=dtype).element_size()
        return self.get(name, n)[:n].view(dtype).reshape(shape)

    def total_bytes(self) -> int:
        return sum(t.numel() for t in self.items.values())
