"""Per-layer NVTX ranges (launch option ``trace_layers``): every attention and feed-forward sub-layer of a forward
pass is bracketed by a named range (``L12.attn``, ``L12.ffn``), so a timeline of the process groups its kernels by
layer. The ranges are host-side markers: they cost a few hundred nanoseconds each and are skipped inside a CUDA-graph
replay (the capture pass shows them once).
Reference: inc/engine/runtime/options.def (``trace_layers``: NVTX range per layer), docs/PROFILING.md.
"""
from __future__ import annotations

import functools

import torch


def _ranges():
    if torch.cuda.is_available():
        return torch.cuda.nvtx.range_push, torch.cuda.nvtx.range_pop
    return None, None


def enable_layer_trace(model, push=None, pop=None) -> list[str]:
    """Wrap the model's sub-layer methods; returns the wrapped names. ``push`` / ``pop`` replace the NVTX calls (tests,
    or another tracer); with neither given and no CUDA runtime nothing is wrapped."""
    if push is None or pop is None:
        push, pop = _ranges()
    if push is None:
        return []
    done = []
    model._trace_mark = (push, pop)        # forward paths that inline their sub-layers mark whole layers with this
    for name, tag in (("attn_block", "attn"), ("ffn_block", "ffn")):
        fn = getattr(model, name, None)
        if fn is None or getattr(fn, "_traced", False):
            continue

        def make(fn, tag):
            @functools.wraps(fn)
            def wrapped(li, *a, **kw):
                push(f"L{li}.{tag}")
                try:
                    return fn(li, *a, **kw)
                finally:
                    pop()
            wrapped._traced = True
            return wrapped

        setattr(model, name, make(fn, tag))
        done.append(name)
    return done
