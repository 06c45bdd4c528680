"""Paged KV cache shared by every sequence slot.

One pool per layer ``[pages, kv_heads, 64, head_dim]`` (a page is exactly one attention key tile), one
device page table ``[slots, max_pages]`` read by the kernels, and a host free list. The reference keeps
a dense ``[slot][layer][max_seq]`` pool for most models and pages only the GLM latent cache
(src/runtime/kv_cache.cpp, inc/engine/core/kv_format.h:51-93); here every model is paged so 262144-token
contexts and many short slots share the same 180 GB.
"""
from __future__ import annotations

import torch

PAGE = 64


class OutOfPages(RuntimeError):
    pass


# whole-cache element formats: bf16, E5M2 bytes, or the scaled forms "k8v4" (int8 keys + 4-bit Hadamard-rotated values, one
# fp16 scale per 64 elements) and "nvfp4" (E2M1 with one E4M3 scale per 16). Attention expands pages to bf16 on chip.
KV_FORMATS = {"bf16": torch.bfloat16, "fp16": torch.bfloat16, "fp8": torch.float8_e5m2, "k8v4": "k8v4", "nvfp4": "nvfp4"}


class PagedKVCache:
    def __init__(self, n_layers: int, n_kv: int, head_dim: int, num_pages: int, max_slots: int, max_seq: int,
                 device, dtype=torch.bfloat16, v_head_dim: int | None = None, arena=None):
        """``arena``: a ``runtime.arena.Arena`` that the page pools are carved from (one device allocation for the
        serving process); ``None`` allocates each pool by itself."""
        def pool(name, *shape, dtype):
            if arena is None:
                return torch.zeros(*shape, dtype=dtype, device=device)
            return arena.alloc(shape, dtype, name).zero_()
        if isinstance(dtype, str):
            dtype = KV_FORMATS[dtype]
        self.n_layers, self.n_kv, self.head_dim = n_layers, n_kv, head_dim
        self.v_head_dim = v_head_dim or head_dim
        self.num_pages, self.max_slots = num_pages, max_slots
        self.max_pages = (max_seq + PAGE - 1) // PAGE
        self.device = device
        # page 0 is the null page: unassigned table entries point at it
        self.fmt = 0
        self.ks = self.vs = None
        if isinstance(dtype, str):                  # scaled formats: byte pools plus scale pools
            from ..quant import kv_codec as C
            self.fmt = C.FORMAT_CODES[dtype]
            kq, vq = C.FORMATS[self.fmt]
            assert head_dim % 64 == 0 and self.v_head_dim % 64 == 0, "scaled KV formats need head dims that are multiples of 64"
            self.k = pool("kv/k", n_layers, num_pages, n_kv, PAGE, C.data_bytes(kq, head_dim), dtype=torch.uint8)
            self.v = pool("kv/v", n_layers, num_pages, n_kv, PAGE, C.data_bytes(vq, self.v_head_dim), dtype=torch.uint8)
            self.ks = pool("kv/k_scales", n_layers, num_pages, n_kv, PAGE, C.scale_bytes(kq, head_dim), dtype=torch.uint8)
            self.vs = pool("kv/v_scales", n_layers, num_pages, n_kv, PAGE, C.scale_bytes(vq, self.v_head_dim), dtype=torch.uint8)
        else:
            self.fmt = 1 if dtype == torch.float8_e5m2 else 0
            self.k = pool("kv/k", n_layers, num_pages, n_kv, PAGE, head_dim, dtype=dtype)
            self.v = pool("kv/v", n_layers, num_pages, n_kv, PAGE, self.v_head_dim, dtype=dtype)
        self.page_table = torch.zeros(max_slots, self.max_pages, dtype=torch.int32, device=device)
        self.host_table = torch.zeros(max_slots, self.max_pages, dtype=torch.int32)
        self.free = list(range(num_pages - 1, 0, -1))
        self.slot_pages = [0] * max_slots  # logical pages covered per slot (high-water mark)
        self.slot_first = [0] * max_slots  # first logical page still held (pages below were recycled by release_prefix)

    @staticmethod
    def pool_bytes(n_layers: int, n_kv: int, head_dim: int, num_pages: int, dtype="bf16", v_head_dim: int | None = None) -> int:
        """Device bytes of the page pools for these dimensions (alignment slack of the four pools included)."""
        vd = v_head_dim or head_dim
        fmt = KV_FORMATS[dtype] if isinstance(dtype, str) else dtype
        rows = n_layers * num_pages * n_kv * PAGE
        if isinstance(fmt, str):
            from ..quant import kv_codec as C
            kq, vq = C.FORMATS[C.FORMAT_CODES[fmt]]
            per = C.data_bytes(kq, head_dim) + C.data_bytes(vq, vd) + C.scale_bytes(kq, head_dim) + C.scale_bytes(vq, vd)
        else:
            per = (head_dim + vd) * torch.empty((), dtype=fmt).element_size()
        return rows * per + 4 * 256

    @staticmethod
    def pages_for(n_tokens: int) -> int:
        return (n_tokens + PAGE - 1) // PAGE

    def free_pages(self) -> int:
        return len(self.free)

    def can_reserve(self, slot: int, n_tokens: int) -> bool:
        return self.pages_for(n_tokens) - self.slot_pages[slot] <= len(self.free)

    def reserve(self, slot: int, n_tokens: int) -> None:
        """Make sure ``slot`` owns pages covering positions [0, n_tokens)."""
        need = self.pages_for(n_tokens)
        if need > self.max_pages:
            raise OutOfPages(f"sequence of {n_tokens} tokens exceeds max_seq")
        have = self.slot_pages[slot]
        if need <= have:
            return
        if need - have > len(self.free):
            raise OutOfPages(f"need {need - have} pages, {len(self.free)} free")
        for i in range(have, need):
            self.host_table[slot, i] = self.free.pop()
        self.slot_pages[slot] = need
        self.page_table[slot, have:need].copy_(self.host_table[slot, have:need], non_blocking=True)

    def release(self, slot: int, keep_tokens: int = 0) -> None:
        keep = self.pages_for(keep_tokens)
        for i in range(keep, self.slot_pages[slot]):
            if int(self.host_table[slot, i]):
                self.free.append(int(self.host_table[slot, i]))
            self.host_table[slot, i] = 0
        self.slot_first[slot] = min(self.slot_first[slot], keep)
        if self.slot_pages[slot] > keep:
            self.page_table[slot, keep:self.slot_pages[slot]].zero_()
        self.slot_pages[slot] = keep

    def release_prefix(self, slot: int, below_tokens: int) -> int:
        """Recycle the pages that lie wholly below position ``below_tokens`` (a sliding-window consumer never reads them
        again): the cache then behaves as a ring of window-sized storage over an unbounded position range. The table
        entries point at the null page afterwards. Returns the number of pages freed."""
        first = self.slot_first[slot]
        upto = min(below_tokens // PAGE, self.slot_pages[slot])
        if upto <= first:
            return 0
        n = 0
        for i in range(first, upto):
            pg = int(self.host_table[slot, i])
            if pg:
                self.free.append(pg)
                n += 1
            self.host_table[slot, i] = 0
        self.page_table[slot, first:upto].zero_()
        self.slot_first[slot] = upto
        return n

    def move_rows(self, slot: int, src_pos: list[int], dst_pos: list[int]) -> None:
        """Copy the cache rows of ``slot`` at positions ``src_pos`` to ``dst_pos`` in every layer (keys, values and
        their scales): what keeps the accepted branch of a verification tree and drops the rest. All sources are read
        before any destination is written."""
        pairs = [(s, d) for s, d in zip(src_pos, dst_pos) if s != d]
        if not pairs:
            return
        dev = self.k.device
        sp = torch.tensor([p for p, _ in pairs], dtype=torch.long)
        dp = torch.tensor([p for _, p in pairs], dtype=torch.long)
        tab = self.host_table[slot].long()
        s_page, s_off = tab[sp // PAGE].to(dev), (sp % PAGE).to(dev)
        d_page, d_off = tab[dp // PAGE].to(dev), (dp % PAGE).to(dev)
        for pool in (self.k, self.v, self.ks, self.vs):
            if pool is not None:
                rows = pool[:, s_page, :, s_off]              # gathered first: [pairs, layers, kv heads, width]
                pool[:, d_page, :, d_off] = rows

    def layer(self, i: int):
        k, v = self.k[i], self.v[i]
        if self.fmt >= 2:      # the ops read the format and the scale pools off the pool tensors
            k.kv_fmt = v.kv_fmt = self.fmt
            k.kv_scale, v.kv_scale = self.ks[i], self.vs[i]
            k.kv_hd, v.kv_hd = self.head_dim, self.v_head_dim
        return k, v

    # ---- snapshots (prefix cache): copy the rows [from_tok, to_tok) of a slot to / from host memory
    def save_rows(self, slot: int, from_tok: int, to_tok: int) -> dict:
        p0, p1 = from_tok // PAGE, self.pages_for(to_tok)
        pages = self.host_table[slot, p0:p1].long().to(self.device)
        snap = {"from": from_tok, "to": to_tok, "p0": p0,
                "k": self.k[:, pages].to("cpu", non_blocking=False),
                "v": self.v[:, pages].to("cpu", non_blocking=False)}
        if self.ks is not None:
            snap["ks"], snap["vs"] = self.ks[:, pages].to("cpu"), self.vs[:, pages].to("cpu")
        return snap

    def load_rows(self, slot: int, snap: dict) -> None:
        self.reserve(slot, snap["to"])
        p0 = snap["p0"]
        n = snap["k"].shape[1]
        pages = self.host_table[slot, p0:p0 + n].long().to(self.device)
        self.k[:, pages] = snap["k"].to(self.device)
        self.v[:, pages] = snap["v"].to(self.device)
        if self.ks is not None:
            self.ks[:, pages] = snap["ks"].to(self.device)
            self.vs[:, pages] = snap["vs"].to(self.device)

    def bytes_per_token(self) -> int:
        per = self.k.shape[-1] * self.k.element_size() + self.v.shape[-1] * self.v.element_size()
        if self.ks is not None:
            per += self.ks.shape[-1] + self.vs.shape[-1]
        return self.n_layers * self.n_kv * per
