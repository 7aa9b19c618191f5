"""The engine: a model on one GPU, its cache, and the step function.

`step` takes a batch of sequences with their next tokens (whole prompts of
unequal lengths, or one token each, or any mix), runs exactly those tokens as
one batch from the cache that earlier steps left, and returns the logits at the
wanted places. The reference has two separate paths for one sequence
(`prefill_prompt`, `forward_next_token`: crates/aegisllm-base/src/executor/
traits.rs:73-91) and `forward_logits` as its numerics entry point
(crates/aegisllm-cuda/src/executor/forward.rs:281-298); batches are this
library's own, checked before launch in the manner of
crates/aegisllm-cuda/src/executor/prefill/batch/builder.rs:15-36,441-469.
"""
from __future__ import annotations

from dataclasses import dataclass, field
from pathlib import Path
from typing import Dict, List, Optional, Sequence

import numpy as np
import torch

from ..cache.kv import PAGE, KVCache, pages_for
from ..cache.slots import CacheError, CacheFull
from ..config import ConfigError, ModelSpec, load_config
from ..parts.base import Runtime
from .context import StepContext
from .model import DecoderModel, expected_tensors

_DTYPES = {"bfloat16": torch.bfloat16, "float32": torch.float32,
           torch.bfloat16: torch.bfloat16, torch.float32: torch.float32}


class StepError(ValueError):
    """A step was refused before anything ran."""


@dataclass
class StepEntry:
    slot: int
    tokens: Sequence[int]
    want: Sequence[int] = ()


def _pad4(n: int) -> int:
    return (n + 3) & ~3


def require_gpu(device=None) -> torch.device:
    if not torch.cuda.is_available():
        raise RuntimeError("lumenllm_b200 computes on a CUDA device (sm_100a) only; none is visible "
                           "and there is no CPU path")
    return torch.device("cuda", torch.cuda.current_device() if device is None else int(device))


class Engine:
    def __init__(self, spec: ModelSpec, weights: Dict[str, torch.Tensor], dtype="bfloat16",
                 max_tokens: int = 8192, max_slots: Optional[int] = None, device=None,
                 config=None):
        if dtype not in _DTYPES:
            raise ConfigError(f"dtype {dtype!r}: bfloat16 or float32")
        self.device = require_gpu(device)
        torch.cuda.set_device(self.device)
        self.runtime = Runtime(self.device, _DTYPES[dtype])
        self.spec = spec
        self.config = config
        self.model = DecoderModel(spec, weights, self.runtime)
        n_pages = pages_for(max_tokens)
        if max_slots is None:
            max_slots = max(1, min(n_pages, 4096))
        self.cache = KVCache(self.model.cache_needs(), max_tokens, max_slots, spec.max_positions,
                             dtype=self.runtime.dtype, device=self.device,
                             state_shapes=self.model.state_shapes())
        self.vocab_size = spec.vocab_size
        self._meta_dev = torch.empty((1 << 16,), dtype=torch.int32, device=self.device)
        self.steps_run = 0

    # ------------------------------------------------------------ construction
    @classmethod
    def from_folder(cls, folder, dtype="bfloat16", max_tokens=8192, max_slots=None, device=None):
        """A folder with config.json and model.safetensors; config.json chooses the model."""
        from ..weights import load_weights
        dev = require_gpu(device)
        config = load_config(folder)
        spec = config.model_spec()
        exp = {n: shape for n, (shape, _) in expected_tensors(spec).items()}
        weights = load_weights(folder, exp, dev)
        return cls(spec, weights, dtype, max_tokens, max_slots, dev.index, config=config)

    @classmethod
    def from_random(cls, config, seed=0, std=0.02, norm_jitter=0.0, dtype="bfloat16",
                    max_tokens=8192, max_slots=None, device=None, weight_dtype="bfloat16"):
        """Random weights made on the device (large shapes need no file)."""
        from ..config import config_from_dict
        from ..weights import random_weights
        dev = require_gpu(device)
        if isinstance(config, dict):
            config = config_from_dict(config)
        spec = config.model_spec()
        weights = random_weights(expected_tensors(spec), seed, std, norm_jitter,
                                 _DTYPES[weight_dtype], device=dev)
        return cls(spec, weights, dtype, max_tokens, max_slots, dev.index, config=config)

    # ------------------------------------------------------------ slots
    def alloc_slot(self) -> int:
        return self.cache.alloc_slot()

    def free_slot(self, slot: int) -> None:
        self.cache.free_slot(slot)

    def length(self, slot: int) -> int:
        return self.cache.length(slot)

    # ------------------------------------------------------------ the step
    def _validate(self, entries: Sequence[StepEntry]) -> None:
        if not entries:
            raise StepError("a step needs at least one sequence")
        seen = set()
        V = self.vocab_size
        for e in entries:
            if e.slot in seen:
                raise StepError(f"slot {e.slot} appears twice in one step")
            seen.add(e.slot)
            if e.slot not in self.cache.slots.held:
                raise StepError(f"slot {e.slot} is not live")
            if len(e.tokens) == 0:
                raise StepError(f"slot {e.slot}: a sequence must bring at least one token")
            for t in e.tokens:
                if not 0 <= int(t) < V:
                    raise StepError(f"slot {e.slot}: token id {t} is outside the vocabulary "
                                    f"of {V}")
            for w in e.want:
                if not 0 <= int(w) < len(e.tokens):
                    raise StepError(f"slot {e.slot}: wanted place {w} is not among the "
                                    f"{len(e.tokens)} tokens of this step")
            if self.cache.length(e.slot) + len(e.tokens) > self.spec.max_positions:
                raise StepError(f"slot {e.slot}: {self.cache.length(e.slot) + len(e.tokens)} tokens "
                                f"exceed max_position_embeddings {self.spec.max_positions}")

    def build_context(self, entries: Sequence[StepEntry], pad_to: int = 0,
                      table_width: int = 0) -> StepContext:
        """Reserves cache room and puts the step's metadata on the device. With
        pad_to > len(entries), padding sequences of one token are appended; they
        write to the reserved page 0 and are read by nobody."""
        starts = [self.cache.reserve(e.slot, len(e.tokens)) for e in entries]
        B_real = len(entries)
        B = max(B_real, pad_to)
        q_lens = [len(e.tokens) for e in entries] + [1] * (B - B_real)
        starts_all = starts + [0] * (B - B_real)
        slots = [e.slot for e in entries] + [-1] * (B - B_real)
        N = sum(q_lens)
        W = sum(len(e.want) for e in entries)
        n_groups = len(self.cache.groups)
        width = max(pages_for(s + q) for s, q in zip(starts_all, q_lens))
        width = max(width, table_width, 1)
        sizes = [N, N, N, N, B, B, B, B + 1, W] + [B * width] * n_groups
        offs = np.cumsum([0] + [_pad4(s) for s in sizes])
        total = int(offs[-1])
        host = np.zeros((total,), dtype=np.int32)
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
            pos = np.arange(starts_all[b], starts_all[b] + q, dtype=np.int32)
            rpos[n:n + q] = pos
            cpos[n:n + q] = pos
            tseq[n:n + q] = b
            cu[b] = n
            n += q
        cu[B] = n
        host[offs[4]:offs[4] + B] = slots
        host[offs[5]:offs[5] + B] = starts_all
        host[offs[6]:offs[6] + B] = q_lens
        for gi, g in enumerate(self.cache.groups):
            bt = host[offs[9 + gi]:offs[9 + gi] + B * width].reshape(B, width)
            for b in range(B_real):
                wcols = min(width, g.table.shape[1])
                bt[b, :wcols] = g.table[slots[b], :wcols]
        if total > self._meta_dev.numel():
            self._meta_dev = torch.empty((max(total, 2 * self._meta_dev.numel()),),
                                         dtype=torch.int32, device=self.device)
        pinned = torch.from_numpy(host).pin_memory()
        dev = self._meta_dev[:total]
        dev.copy_(pinned, non_blocking=True)
        sl = lambda i, n_: dev[int(offs[i]):int(offs[i]) + n_]
        return StepContext(
            runtime=self.runtime, B=B, N=N, q_lens=q_lens, starts=starts_all, slots=slots,
            tokens=sl(0, N), rope_pos=sl(1, N), cache_pos=sl(2, N), tok_seq=sl(3, N),
            seq_slot=sl(4, B), seq_start=sl(5, B), seq_qlen=sl(6, B), cu_q=sl(7, B + 1),
            want_rows=sl(8, W),
            block_tables=[sl(9 + gi, B * width).view(B, width) for gi in range(n_groups)],
            cache=self.cache, n_real=B_real)

    def step(self, entries: Sequence[StepEntry]) -> torch.Tensor:
        """Runs the given tokens; returns float32 logits [wanted, vocab] on the device, in
        the order of the entries and of their `want`."""
        entries = list(entries)
        self._validate(entries)
        try:
            ctx = self.build_context(entries)
        except CacheFull as e:
            raise StepError(str(e)) from e
        logits = self.model.forward(ctx)
        for e in entries:
            self.cache.commit(e.slot, len(e.tokens))
        self.steps_run += 1
        return logits
