"""The cache of keys and values, and beside it per-sequence state of fixed size.

Storage is paged: a page holds PAGE consecutive positions of one sequence for
every kv head of one cache entry, laid out [n_kv][PAGE][head_dim], so the tile
(page, kv head) is contiguous. A cache ENTRY belongs to one run of a layer in
the model's schedule. Entries with the same needs (kv heads, head size, window)
form a GROUP with storage, page pool and page tables of its own: a group that
sees all keys keeps every page of a live sequence, a group with a window gives
pages back as soon as they fall out of every later query's sight.

A slot is one live sequence: its length, and per group its page table. Slots
are handed out when a batch starts and given back when a sequence ends.

The reference keeps one contiguous buffer [context, n_kv, d] per layer for its
single sequence (crates/aegisllm-cuda/src/executor/state.rs:747-819) and a
per-layer capacity min(window, context) (executor/full.rs:1259-1273); slots,
pages and groups are this library's own.
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import Dict, List, Optional, Tuple

import numpy as np
import torch

from ..csrc.build import page_size
from .slots import CacheError, CacheFull, PagePool, SlotAllocator

PAGE = page_size()      # tokens per page: LUMEN_PAGE of csrc/common.cuh
LAYOUT_LINEAR, LAYOUT_SW128 = 0, 1


def tile_layout(dtype, head_dim: int) -> int:
    """How a (page, kv head) tile is laid out: bfloat16 tiles whose head size is a
    multiple of 64 are kept in the 128-byte-swizzled form that the tensor-core kernels
    stage with plain bulk copies; everything else is [key][head_dim]."""
    return LAYOUT_SW128 if (dtype == torch.bfloat16 and head_dim % 64 == 0) else LAYOUT_LINEAR


def _aligned_zeros(shape, dtype, device, align=1024):
    """Zeros whose first byte lies on an `align`-byte boundary (tiles must)."""
    n = 1
    for s in shape:
        n *= s
    item = torch.empty((), dtype=dtype).element_size()
    raw = torch.zeros((n * item + align,), dtype=torch.uint8, device=device)
    off = (-raw.data_ptr()) % align
    return raw[off:off + n * item].view(dtype).view(shape)


@dataclass(frozen=True)
class CacheNeed:
    """What a mixer asks of the cache for one entry."""
    n_kv: int
    head_dim: int
    window: int = 0   # 0: all keys


def pages_for(n_tokens: int) -> int:
    return (n_tokens + PAGE - 1) // PAGE


class CacheGroup:
    def __init__(self, need: CacheNeed, entries: List[int], n_pages: int, max_slots: int,
                 max_pages_per_seq: int, dtype, device):
        self.need = need
        self.entries = list(entries)
        self.index_of = {e: i for i, e in enumerate(self.entries)}
        self.pool = PagePool(n_pages, reserved=1)
        total = n_pages + 1
        shape = (len(self.entries), total, need.n_kv, PAGE, need.head_dim)
        self.layout = tile_layout(dtype, need.head_dim)
        if device is not None:
            self.k = _aligned_zeros(shape, dtype, device)
            self.v = _aligned_zeros(shape, dtype, device)
        else:  # bookkeeping only (host tests)
            self.k = self.v = None
        self.table = np.zeros((max_slots, max_pages_per_seq), dtype=np.int32)
        self.first_page = np.zeros((max_slots,), dtype=np.int64)   # first page index still held
        self.n_held = np.zeros((max_slots,), dtype=np.int64)       # pages held: [first, first+n)

    def bytes_per_token(self, itemsize: int) -> int:
        return 2 * len(self.entries) * self.need.n_kv * self.need.head_dim * itemsize

    def reserve(self, slot: int, new_len: int) -> None:
        want_end = pages_for(new_len)
        have_end = int(self.first_page[slot] + self.n_held[slot])
        if want_end > self.table.shape[1]:
            raise CacheFull(f"slot {slot}: {new_len} tokens are beyond the longest sequence "
                            f"the cache was built for ({self.table.shape[1] * PAGE})")
        if want_end > have_end:
            try:
                got = self.pool.take(want_end - have_end)
            except CacheFull as e:
                raise CacheFull(f"slot {slot}: the cache is full ({e})") from None
            self.table[slot, have_end:want_end] = got
            self.n_held[slot] += want_end - have_end

    def trim(self, slot: int, length: int) -> None:
        """After a step: a group with a window gives back the pages that no later
        query can see (the next query sits at position `length`)."""
        w = self.need.window
        if w <= 0:
            return
        first_needed = max(0, length - w + 1) // PAGE
        first = int(self.first_page[slot])
        if first_needed > first:
            n = min(first_needed - first, int(self.n_held[slot]))
            self.pool.give_back(self.table[slot, first:first + n].tolist())
            self.table[slot, first:first + n] = 0
            self.first_page[slot] = first + n
            self.n_held[slot] -= n

    def release(self, slot: int) -> None:
        first, n = int(self.first_page[slot]), int(self.n_held[slot])
        if n:
            self.pool.give_back(self.table[slot, first:first + n].tolist())
        self.table[slot, :] = 0
        self.first_page[slot] = 0
        self.n_held[slot] = 0


class StateStore:
    """Per-sequence state of fixed size: for each entry that declares a shape, a
    tensor [max_slots + 1, *shape], zeroed when a slot is handed out. It is never
    indexed by position and never grows. Row `pad_row` (the last) belongs to no
    sequence: the padding rows of a captured step read and write it, as they write
    page 0 of the cache, so that a mixer which indexes its state by `seq_slot` on the
    device touches no live sequence's state for them. (The reference keeps such state
    per layer for its recurrent mixers: executor/state.rs:640-648.)"""

    def __init__(self, shapes: Dict[int, Tuple[Tuple[int, ...], torch.dtype]], max_slots: int, device):
        self.pad_row = max_slots
        self.tensors: Dict[int, torch.Tensor] = {}
        for entry, (shape, dtype) in shapes.items():
            self.tensors[entry] = torch.zeros((max_slots + 1, *shape), dtype=dtype, device=device)

    def zero_slot(self, slot: int) -> None:
        for t in self.tensors.values():
            t[slot].zero_()

    def of(self, entry: int) -> Optional[torch.Tensor]:
        return self.tensors.get(entry)


class KVCache:
    def __init__(self, needs: Dict[int, CacheNeed], max_tokens: int, max_slots: int,
                 max_positions: int, dtype=None, device=None,
                 state_shapes: Optional[Dict[int, Tuple[Tuple[int, ...], torch.dtype]]] = None):
        if max_tokens <= 0 or max_slots <= 0:
            raise CacheError("the cache needs room for at least one token and one slot")
        self.max_tokens = max_tokens
        self.max_slots = max_slots
        self.n_pages = pages_for(max_tokens)
        self.max_pages_per_seq = max(1, min(pages_for(max_positions), self.n_pages))
        self.dtype, self.device = dtype, device
        self.slots = SlotAllocator(max_slots)
        self.lengths = np.zeros((max_slots,), dtype=np.int64)
        by_need: Dict[CacheNeed, List[int]] = {}
        for entry in sorted(needs):
            by_need.setdefault(needs[entry], []).append(entry)
        self.groups: List[CacheGroup] = [
            CacheGroup(need, entries, self.n_pages, max_slots, self.max_pages_per_seq, dtype, device)
            for need, entries in by_need.items()]
        self.group_of: Dict[int, int] = {e: gi for gi, g in enumerate(self.groups) for e in g.entries}
        self.state = StateStore(state_shapes or {}, max_slots, device)

    # -------------------------------------------------- slots
    def alloc_slot(self) -> int:
        slot = self.slots.alloc()
        self.lengths[slot] = 0
        self.state.zero_slot(slot)
        return slot

    def free_slot(self, slot: int) -> None:
        self.slots.free(slot)       # raises if not held; nothing is touched then
        for g in self.groups:
            g.release(slot)
        self.lengths[slot] = 0

    def length(self, slot: int) -> int:
        self._live(slot)
        return int(self.lengths[slot])

    def _live(self, slot: int) -> None:
        if slot not in self.slots.held:
            raise CacheError(f"slot {slot} is not live")

    # -------------------------------------------------- growth
    def reserve(self, slot: int, n_new: int) -> int:
        """Makes room for n_new more tokens of the slot; returns its current length.
        On CacheFull the slot keeps what it had."""
        self._live(slot)
        cur = int(self.lengths[slot])
        for g in self.groups:
            g.reserve(slot, cur + n_new)
        return cur

    def commit(self, slot: int, n_new: int) -> None:
        self._live(slot)
        self.lengths[slot] += n_new
        for g in self.groups:
            g.trim(slot, int(self.lengths[slot]))

    def free_tokens(self) -> int:
        return min((g.pool.free_count for g in self.groups), default=self.n_pages) * PAGE

    # -------------------------------------------------- views
    def entry_storage(self, entry: int):
        g = self.groups[self.group_of[entry]]
        i = g.index_of[entry]
        return g.k[i], g.v[i], self.group_of[entry]

    def check(self) -> None:
        self.slots.check()
        for g in self.groups:
            g.pool.check()
            held = int(sum(g.n_held[s] for s in self.slots.held))
            if held != len(g.pool.held):
                raise CacheError(f"{len(g.pool.held)} pages are held but live slots account "
                                 f"for {held}")
