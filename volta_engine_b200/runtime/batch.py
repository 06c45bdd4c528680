"""Per-forward row descriptor, resident on the device so one CUDA graph per row count serves every step.

Equivalent of the reference's ``BatchRows`` / ``SlotRef`` (inc/engine/core/batch.h:11-105): each row
names its sequence slot and position; prefill chunks carry the tile grouping for the attention kernel;
the logits mode says which rows reach the LM head.
"""
from __future__ import annotations

from dataclasses import dataclass, field

import torch

MAX_GRAPH_ROWS = 16    # decode / verify row counts that get a captured graph
MAX_CHUNK_ROWS = 4096  # prefill chunk upper bound

LOGITS_ALL = "all"
LOGITS_LAST = "last"
LOGITS_NONE = "none"


@dataclass
class BatchRows:
    ids: torch.Tensor      # [n] int32
    pos: torch.Tensor      # [n] int32
    slot: torch.Tensor     # [n] int32 (-1 = padding row)
    n: int
    logits: str = LOGITS_ALL
    tiles: tuple | None = None      # (tile_first, tile_count, ntiles) for prefill attention
    nsplit: int = 1                 # split-KV factor for decode attention
    key_end: torch.Tensor | None = None
    host_slots: list = field(default_factory=list)
    host_pos: list = field(default_factory=list)
    pos3: torch.Tensor | None = None        # [3, n] int32 rotary positions (time, height, width) of multimodal prompts
    embeds: torch.Tensor | None = None      # [n, H] rows that replace the token embedding where embed_mask is set
    embed_mask: torch.Tensor | None = None  # [n] bool
    tree: tuple | None = None               # (base int32 [n], mask int64 [n]): rows of a verification tree (ops.kernels.attention)

    @classmethod
    def make(cls, ids, pos, slots, device, logits=LOGITS_ALL, G=1, prefill=False, nsplit=1):
        from ..ops.kernels import make_prefill_tiles
        n = len(ids)
        t_ids = torch.tensor(ids, dtype=torch.int32).to(device, non_blocking=True)
        t_pos = torch.tensor(pos, dtype=torch.int32).to(device, non_blocking=True)
        t_slot = torch.tensor(slots, dtype=torch.int32).to(device, non_blocking=True)
        tiles = make_prefill_tiles(list(slots), G, device) if prefill else None
        return cls(t_ids, t_pos, t_slot, n, logits, tiles, nsplit, None, list(slots), list(pos))
