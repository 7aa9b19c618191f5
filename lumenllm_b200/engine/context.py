"""What one step hands to the parts: the batch's metadata on the device, and
views of the cache and of the per-sequence state for each run of a layer.

The vocabulary follows the reference's batch descriptors (`positions`,
`slot_mapping`, `cu_q`, `context_lens`: crates/aegisllm-cuda/src/executor/
prefill/batch/mod.rs:26-63), for B sequences that bring N tokens together:

  tokens[N], rope_pos[N] (position used for the rotation), cache_pos[N] (index
  of the token in its sequence's cache), tok_seq[N] (which of the B sequences),
  seq_slot[B] (the state store's spare row for padding sequences), seq_start[B]
  (cached length before the step), seq_qlen[B],
  cu_q[B+1], want_rows[W] (rows whose logits are wanted), and per cache group a
  page table [B, pages].
"""
from __future__ import annotations

from dataclasses import dataclass, field
from typing import Dict, List, Optional, Sequence

import numpy as np
import torch

from ..cache.kv import pages_for


@dataclass
class StepEntry:
    """One sequence of a step: its slot, its next tokens, and the places among these
    tokens whose logits are wanted. `positions`, when given (one per token), are what the
    position encoding sees (`rope_pos`) instead of the tokens' indices in the cache; where
    a token's key is stored and which keys it sees still follow the cache index."""
    slot: int
    tokens: Sequence[int]
    want: Sequence[int] = ()
    positions: Optional[Sequence[int]] = None


def _pad4(n: int) -> int:
    return (n + 3) & ~3


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

    @property
    def layout(self) -> int:
        """Tile layout of this run's cache pages (cache.kv.LAYOUT_*)."""
        return self.ctx.cache.groups[self.ctx.cache.group_of[self.cache_entry]].layout

    def state(self):
        """Per-sequence state of fixed size: [max_slots + 1, *shape]; row seq_slot[b] belongs
        to sequence b (the last row to every padding sequence). None if the mixer declared
        none."""
        return self.ctx.cache.state.of(self.entry)


@dataclass
class StepLayout:
    """Where each array of a step lies in the one int32 buffer that carries them."""
    B: int
    N: int
    W: int
    width: int
    n_groups: int
    offs: List[int]
    total: int

    @classmethod
    def of(cls, B, N, W, width, n_groups) -> "StepLayout":
        sizes = [N, N, N, N, B, B, B, B + 1, W] + [B * width] * n_groups
        offs = [0]
        for s in sizes:
            offs.append(offs[-1] + _pad4(s))
        return cls(B, N, W, width, n_groups, offs, offs[-1])


def pack_step(cache, entries, pad_to: int = 0, table_width: int = 0, want_padding: bool = False,
              pad_lens: Optional[Sequence[int]] = None):
    """Reserves cache room for the entries and lays the step's metadata out on the host.
    With pad_to > len(entries), padding sequences are appended (of one token each, or of
    pad_lens[i] tokens, which may be none): they start at position 0, their page table is all zeros, so they
    write to the reserved page 0 and are read by nobody (with want_padding the logits at
    their first token are computed too, so that a captured step keeps its shapes)."""
    starts = [cache.reserve(e.slot, len(e.tokens)) for e in entries]
    B_real = len(entries)
    B = max(B_real, pad_to)
    pads = [1] * (B - B_real) if pad_lens is None else [int(x) for x in pad_lens]
    if len(pads) != B - B_real or any(x < 0 for x in pads):
        raise ValueError("pad_lens: one length for each padding sequence")
    q_lens = [len(e.tokens) for e in entries] + pads
    starts_all = starts + [0] * (B - B_real)
    # padding sequences point at the state store's spare row, as their writes go to page 0
    slots = [e.slot for e in entries] + [cache.state.pad_row] * (B - B_real)
    N = sum(q_lens)
    W = sum(len(e.want) for e in entries) + ((B - B_real) if want_padding else 0)
    n_groups = len(cache.groups)
    width = max(pages_for(s + q) for s, q in zip(starts_all, q_lens))
    width = max(width, table_width, 1)
    lay = StepLayout.of(B, N, W, width, n_groups)
    offs = lay.offs
    host = np.zeros((lay.total,), dtype=np.int32)
    tok = host[offs[0]:offs[0] + N]
    rpos = host[offs[1]:offs[1] + N]
    cpos = host[offs[2]:offs[2] + N]
    tseq = host[offs[3]:offs[3] + N]
    cu = host[offs[7]:offs[7] + B + 1]
    want = host[offs[8]:offs[8] + W]
    n = w = 0
    for b in range(B):
        q = q_lens[b]
        if b < B_real:
            tok[n:n + q] = np.asarray(entries[b].tokens, dtype=np.int64)
            for x in entries[b].want:
                want[w] = n + int(x)
                w += 1
        elif want_padding:
            want[w] = n if q > 0 else 0        # an empty padding sequence has no row of its own
            w += 1
        pos = np.arange(starts_all[b], starts_all[b] + q, dtype=np.int32)
        given = entries[b].positions if b < B_real else None
        rpos[n:n + q] = pos if given is None else np.asarray(given, dtype=np.int64)
        cpos[n:n + q] = pos
        tseq[n:n + q] = b
        cu[b] = n
        n += q
    cu[B] = n
    host[offs[4]:offs[4] + B] = slots
    host[offs[5]:offs[5] + B] = starts_all
    host[offs[6]:offs[6] + B] = q_lens
    for gi, g in enumerate(cache.groups):
        bt = host[offs[9 + gi]:offs[9 + gi] + B * width].reshape(B, width)
        wcols = min(width, g.table.shape[1])
        for b in range(B_real):
            bt[b, :wcols] = g.table[slots[b], :wcols]
    return host, lay, q_lens, starts_all, slots, B_real


def padding_twin(host: np.ndarray, lay: StepLayout, q_lens, pad_row: int) -> np.ndarray:
    """The metadata of a step with the same division of tokens in which EVERY sequence is a
    padding sequence (token 0, positions from 0, page table of zeros, the state store's spare
    row): what a captured step is run on once before its capture, so that this run changes
    nothing that belongs to a live sequence."""
    offs = lay.offs
    twin = host.copy()
    N, B = lay.N, lay.B
    twin[offs[0]:offs[0] + N] = 0
    pos = np.concatenate([np.arange(q, dtype=np.int32) for q in q_lens])
    twin[offs[1]:offs[1] + N] = pos
    twin[offs[2]:offs[2] + N] = pos
    twin[offs[4]:offs[4] + B] = pad_row
    twin[offs[5]:offs[5] + B] = 0
    for gi in range(lay.n_groups):
        twin[offs[9 + gi]:offs[9 + gi] + B * lay.width] = 0
    return twin


def context_on(dev: torch.Tensor, lay: StepLayout, q_lens, starts, slots, n_real, cache, runtime):
    """A StepContext whose arrays are views of `dev`, laid out as `lay` says."""
    offs = lay.offs
    sl = lambda i, n_: dev[offs[i]:offs[i] + n_]
    B, N = lay.B, lay.N
    return StepContext(
        runtime=runtime, B=B, N=N, q_lens=list(q_lens), starts=list(starts), slots=list(slots),
        tokens=sl(0, N), rope_pos=sl(1, N), cache_pos=sl(2, N), tok_seq=sl(3, N),
        seq_slot=sl(4, B), seq_start=sl(5, B), seq_qlen=sl(6, B), cu_q=sl(7, B + 1),
        want_rows=sl(8, lay.W),
        block_tables=[sl(9 + gi, B * lay.width).view(B, lay.width) for gi in range(lay.n_groups)],
        cache=cache, n_real=n_real)


def upload(host: np.ndarray, dev: torch.Tensor) -> None:
    """One asynchronous copy from pinned memory; the pinned block is not used again
    before the copy has run (the host allocator waits for it)."""
    dev[:host.size].copy_(torch.from_numpy(host).pin_memory(), non_blocking=True)


def build_context(cache, runtime, entries, meta_dev=None, pad_to: int = 0, table_width: int = 0):
    """pack_step + upload + context_on; returns the context and the (possibly regrown)
    device buffer."""
    host, lay, q_lens, starts, slots, n_real = pack_step(cache, entries, pad_to, table_width)
    if meta_dev is None or lay.total > meta_dev.numel():
        grow = max(lay.total, 2 * (0 if meta_dev is None else meta_dev.numel()), 1 << 14)
        meta_dev = torch.empty((grow,), dtype=torch.int32, device=runtime.device)
    upload(host, meta_dev)
    return context_on(meta_dev[:lay.total], lay, q_lens, starts, slots, n_real, cache, runtime), meta_dev
