"""What one step hands to the parts: the batch's metadata on the device, and
views of the cache and of the per-sequence state for each run of a layer.

The vocabulary follows the reference's batch descriptors (`positions`,
`slot_mapping`, `cu_q`, `context_lens`: crates/aegisllm-cuda/src/executor/
prefill/batch/mod.rs:26-63), for B sequences that bring N tokens together:

  tokens[N], rope_pos[N] (position used for the rotation), cache_pos[N] (index
  of the token in its sequence's cache), tok_seq[N] (which of the B sequences),
  seq_slot[B], seq_start[B] (cached length before the step), seq_qlen[B],
  cu_q[B+1], want_rows[W] (rows whose logits are wanted), and per cache group a
  page table [B, pages].
"""
from __future__ import annotations

from dataclasses import dataclass, field
from typing import Dict, List, Optional

import torch


@dataclass
class StepContext:
    runtime: object
    B: int
    N: int
    q_lens: List[int]
    starts: List[int]
    slots: List[int]
    tokens: torch.Tensor
    rope_pos: torch.Tensor
    cache_pos: torch.Tensor
    tok_seq: torch.Tensor
    seq_slot: torch.Tensor
    seq_start: torch.Tensor
    seq_qlen: torch.Tensor
    cu_q: torch.Tensor
    want_rows: torch.Tensor
    block_tables: List[torch.Tensor]
    cache: object = None
    n_real: Optional[int] = None   # sequences that are not padding
    extras: Dict[str, object] = field(default_factory=dict)

    @property
    def is_decode(self) -> bool:
        return all(q == 1 for q in self.q_lens)

    @property
    def max_q(self) -> int:
        return max(self.q_lens)

    @property
    def max_len(self) -> int:
        return max(s + q for s, q in zip(self.starts, self.q_lens))


class EntryView:
    """One run of a layer as a mixer sees it."""

    def __init__(self, ctx: StepContext, entry: int, cache_entry: Optional[int], writes: bool):
        self.ctx = ctx
        self.entry = entry
        self.cache_entry = cache_entry
        self.writes_cache = writes

    def cache(self):
        """(keys, values, page table) of this run: [pages, n_kv, PAGE, d] twice and
        int32 [B, pages]."""
        if self.cache_entry is None:
            raise RuntimeError(f"entry {self.entry} has no cache (its mixer declared no need)")
        k, v, g = self.ctx.cache.entry_storage(self.cache_entry)
        return k, v, self.ctx.block_tables[g]

    def state(self):
        """Per-sequence state of fixed size: [max_slots, *shape]; row seq_slot[b] belongs
        to sequence b. None if the mixer declared none."""
        return self.ctx.cache.state.of(self.entry)
