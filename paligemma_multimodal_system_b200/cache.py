"""Sequence storage for the ragged-step engine: a shared pool of 64-token KV pages and a pool of recurrent-state slots.

The `KVCache` of modeling_gemma.py gives every batch row a fixed run of pages; here pages belong to whoever asks first.
A model describes what each of its layers keeps per sequence (`cache_layout()`):

    ("kv", key_width, value_width)      one key row and one value row per token  -> pages [num_pages, 64, width]
    ("latent", width)                   ONE row per token from which keys and values of every head are derived (latent
                                        attention: compressed kv vector + shared rotated key part) -> k_pages only
    ("state", shape)                    one fp32 tensor per sequence             -> [num_slots, *shape]
    None                                nothing

`SequenceStore` owns the device tensors and the host-side bookkeeping (free lists, per-request page lists and lengths).
Pages and slots go back to the free lists when a request is released and are handed out again, lowest id first, so a
second request really does land on memory a finished one used.  Nothing is cleared on reuse: a sequence's first step
starts from length zero (attention reads no stale key; recurrent layers start from a zero state when their context is empty).
"""
from typing import Dict, List, Optional, Sequence

import torch

from .modeling_gemma import PAGE


class PagePool:
    """Host-side free list of page ids (no tensors; CPU-testable)."""

    def __init__(self, num_pages: int):
        if num_pages <= 0:
            raise ValueError("a page pool needs at least one page")
        self.num_pages = int(num_pages)
        self.free: List[int] = list(range(self.num_pages))

    def take(self, n: int) -> List[int]:
        if n > len(self.free):
            raise MemoryError(f"KV page pool exhausted: {n} pages wanted, {len(self.free)} of {self.num_pages} free")
        self.free.sort()
        got, self.free = self.free[:n], self.free[n:]
        return got

    def give(self, pages: Sequence[int]):
        dup = set(pages) & set(self.free)
        if dup:
            raise RuntimeError(f"pages freed twice: {sorted(dup)[:4]}")
        self.free.extend(pages)


class SequenceRecord:
    __slots__ = ("rid", "slot", "pages", "length")

    def __init__(self, rid, slot):
        self.rid, self.slot, self.pages, self.length = rid, slot, [], 0


class SequenceStore:
    """Pages + state slots of the live requests of one engine."""

    def __init__(self, layout, max_tokens: int, num_slots: int, dtype: torch.dtype, device="cuda", allocate: bool = True):
        self.page = PAGE
        self.num_slots = int(num_slots)
        num_pages = (int(max_tokens) + PAGE - 1) // PAGE
        self.pool = PagePool(num_pages)
        self.free_slots: List[int] = list(range(self.num_slots))
        self.live: Dict[object, SequenceRecord] = {}
        self.layout = list(layout)
        self.k_pages: List[Optional[torch.Tensor]] = []
        self.v_pages: List[Optional[torch.Tensor]] = []
        self.state: List[Optional[torch.Tensor]] = []
        for spec in self.layout:
            k = v = s = None
            if allocate and spec is not None and spec[0] == "kv":
                k = torch.zeros(num_pages, PAGE, spec[1], device=device, dtype=dtype)
                v = torch.zeros(num_pages, PAGE, spec[2], device=device, dtype=dtype)
            elif allocate and spec is not None and spec[0] == "latent":
                k = torch.zeros(num_pages, PAGE, spec[1], device=device, dtype=dtype)
            elif allocate and spec is not None and spec[0] == "state":
                s = torch.zeros(self.num_slots, *spec[1], device=device, dtype=torch.float32)
            elif spec is not None and spec[0] not in ("kv", "latent", "state"):
                raise ValueError(f"unknown cache kind {spec[0]!r}")
            self.k_pages.append(k)
            self.v_pages.append(v)
            self.state.append(s)

    # -- bookkeeping ---------------------------------------------------------------------------------------------------
    def admit(self, rid) -> SequenceRecord:
        if rid in self.live:
            raise KeyError(f"request {rid!r} is already live")
        if not self.free_slots:
            raise MemoryError(f"all {self.num_slots} sequence slots are taken")
        self.free_slots.sort()
        rec = SequenceRecord(rid, self.free_slots.pop(0))
        self.live[rid] = rec
        return rec

    def reserve(self, rid, new_tokens: int) -> SequenceRecord:
        """Makes sure the request owns pages for `new_tokens` more tokens (its length is advanced by `commit`)."""
        rec = self.live[rid]
        need = (rec.length + new_tokens + PAGE - 1) // PAGE - len(rec.pages)
        if need > 0:
            rec.pages.extend(self.pool.take(need))
        return rec

    def commit(self, rid, new_tokens: int):
        self.live[rid].length += int(new_tokens)

    def release(self, rid):
        rec = self.live.pop(rid)
        self.pool.give(rec.pages)
        self.free_slots.append(rec.slot)

    def max_pages(self, rids) -> int:
        return max(1, max(len(self.live[r].pages) for r in rids))
