"""Model utilities shared by tests and tools."""
from __future__ import annotations

import copy

import torch

_GPU_ONLY = ("_gv", "_sf_k128", "_sf_atoms", "gu_sf", "dn_sf", "attn_ws", "mla_ws")


def to_device(obj, device, _memo=None):
    """Deep copy of a model / layer / linear with every tensor moved to ``device``; load-time kernel layouts that
    only exist for the GPU are dropped (they are rebuilt lazily where needed)."""
    if _memo is None:
        _memo = {}
    if id(obj) in _memo:
        return _memo[id(obj)]
    if isinstance(obj, torch.Tensor):
        return obj.to(device)
    if isinstance(obj, (int, float, str, bool, type(None), torch.device, torch.dtype)):
        return obj
    if isinstance(obj, (list, tuple)):
        return type(obj)(to_device(x, device, _memo) for x in obj)
    if isinstance(obj, dict):
        return {k: to_device(v, device, _memo) for k, v in obj.items()}
    if type(obj).__module__.startswith("volta_engine_b200.parallel"):
        return obj
    new = copy.copy(obj)
    _memo[id(obj)] = new
    names = list(getattr(obj, "__dict__", {}).keys())
    for klass in type(obj).__mro__:
        names += [n for n in getattr(klass, "__slots__", ()) if hasattr(obj, n)]
    for n in names:
        if n in _GPU_ONLY:
            setattr(new, n, None)
        elif n == "device":
            setattr(new, n, torch.device(device))
        else:
            setattr(new, n, to_device(getattr(obj, n), device, _memo))
    return new
