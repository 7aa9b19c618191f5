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

import warnings
from dataclasses import dataclass, field
from pathlib import Path
from typing import Dict, List, Optional, Sequence

import numpy as np
import torch

from ..cache.kv import PAGE, KVCache, pages_for
from ..cache.slots import CacheError, CacheFull
from ..config import ConfigError, ModelSpec, load_config
from ..ops import kernels as K
from ..ops.native import KernelError
from ..parts.base import Runtime
from .context import StepContext, StepEntry, build_context
from .model import DecoderModel, expected_tensors, tensor_fallbacks

_DTYPES = {"bfloat16": torch.bfloat16, "float32": torch.float32,
           torch.bfloat16: torch.bfloat16, torch.float32: torch.float32}


class _InFlight:
    """A launched step: its sampled tokens on the device (valid until the step after the next
    is launched), the pinned host copy under way, and the event that ends the copy."""
    __slots__ = ("dev", "host", "done", "n")

    def __init__(self, dev, host, done, n):
        self.dev, self.host, self.done, self.n = dev, host, done, n


class StepError(ValueError):
    """A step was refused before anything ran."""


def require_gpu(device=None) -> torch.device:
    if not torch.cuda.is_available():
        raise RuntimeError("lumenllm_b200 computes on a CUDA device (sm_100a) only; none is visible "
                           "and there is no CPU path")
    return torch.device("cuda", torch.cuda.current_device() if device is None else int(device))


class Engine:
    def __init__(self, spec: ModelSpec, weights: Dict[str, torch.Tensor], dtype="bfloat16",
                 max_tokens: int = 8192, max_slots: Optional[int] = None, device=None,
                 config=None, context_size: Optional[int] = None, max_step_tokens: int = 8192,
                 use_graphs: bool = True):
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
        self.max_seq_len = min(spec.max_positions, context_size or spec.max_positions)
        self.max_step_tokens = max(1, int(max_step_tokens))
        from ..sampling import DeviceSampler
        self.sampler = DeviceSampler(self.device)
        self._meta_dev = torch.empty((1 << 16,), dtype=torch.int32, device=self.device)
        self.steps_run = 0
        from .step_graph import StepGraphs
        self.graphs = StepGraphs(self)
        self.use_graphs = bool(use_graphs)

    # ------------------------------------------------------------ construction
    @classmethod
    def from_folder(cls, folder, dtype="bfloat16", max_tokens=8192, max_slots=None, device=None,
                    strict_weights: bool = True, **kw):
        """A folder with config.json and model.safetensors; config.json chooses the model.
        With strict_weights=False tensors that no part reads are warned about, not refused."""
        from ..weights import load_weights
        dev = require_gpu(device)
        config = load_config(folder)
        spec = config.model_spec()
        tensors = expected_tensors(spec)
        weights = load_weights(folder, {n: shape for n, (shape, _) in tensors.items()}, dev,
                               optional=[n for n, (_, kind) in tensors.items() if kind == "optional"],
                               fallbacks=tensor_fallbacks(spec), strict=strict_weights)
        for name, other in weights.stood_in.items():
            warnings.warn(f"{folder}: no tensor '{name}' is stored; '{other}' stands in for it")
        for name in weights.unexpected:
            warnings.warn(f"{folder}: tensor '{name}' is stored but no part of the model reads it")
        if _DTYPES.get(dtype) == torch.bfloat16:
            wide = [n for n, (_, kind) in tensors.items()
                    if kind != "norm" and n in weights and weights[n].dtype == torch.float32]
            if wide:
                # a tensor stored in 32-bit stays so, and its products then run in true 32-bit
                warnings.warn(f"{folder}: {len(wide)} matrices are stored in 32-bit (first: '{wide[0]}'); "
                              "they are kept so and multiplied by the 32-bit kernel, many times slower "
                              "than the tensor cores. Store the checkpoint in bfloat16 to serve it.")
        return cls(spec, weights, dtype, max_tokens, max_slots, dev.index, config=config, **kw)

    @classmethod
    def from_random(cls, config, seed=0, std=0.02, norm_jitter=0.0, dtype="bfloat16",
                    max_tokens=8192, max_slots=None, device=None, weight_dtype="bfloat16", **kw):
        """Random weights made on the device (large shapes need no file)."""
        from ..config import config_from_dict
        from ..weights import random_weights
        dev = require_gpu(device)
        if isinstance(config, dict):
            config = config_from_dict(config)
        spec = config.model_spec()
        weights = random_weights(expected_tensors(spec), seed, std, norm_jitter,
                                 _DTYPES[weight_dtype], device=dev)
        return cls(spec, weights, dtype, max_tokens, max_slots, dev.index, config=config, **kw)

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
            if e.positions is not None and (len(e.positions) != len(e.tokens)
                                            or any(int(x) < 0 for x in e.positions)):
                raise StepError(f"slot {e.slot}: positions must be one non-negative number "
                                "for each token")
            for w in e.want:
                if not 0 <= int(w) < len(e.tokens):
                    raise StepError(f"slot {e.slot}: wanted place {w} is not among the "
                                    f"{len(e.tokens)} tokens of this step")
            if self.cache.length(e.slot) + len(e.tokens) > self.max_seq_len:
                raise StepError(f"slot {e.slot}: kv cache context exhausted: "
                                f"{self.cache.length(e.slot) + len(e.tokens)} tokens exceed the "
                                f"context size {self.max_seq_len}")

    def build_context(self, entries: Sequence[StepEntry], pad_to: int = 0,
                      table_width: int = 0) -> StepContext:
        ctx, self._meta_dev = build_context(self.cache, self.runtime, entries, self._meta_dev,
                                            pad_to=pad_to, table_width=table_width)
        return ctx

    def step(self, entries: Sequence[StepEntry]) -> torch.Tensor:
        """Runs the given tokens; returns float32 logits [wanted, vocab] on the device, in
        the order of the entries and of their `want`."""
        entries = [e if isinstance(e, StepEntry) else StepEntry(*e) for e in entries]
        self._validate(entries)
        if sum(len(e.tokens) for e in entries) <= self.max_step_tokens:
            return self._forward(entries)
        # More tokens than one pass may hold in activations: the same work in several
        # passes over the same cache. Pieces of one sequence run in order, so every
        # token still sees exactly the keys before it.
        parts, origin = self._split(entries)
        out = [self._forward(p) for p in parts]
        logits = torch.cat(out, dim=0)
        if origin != sorted(origin):
            order = torch.tensor(sorted(range(len(origin)), key=origin.__getitem__),
                                 dtype=torch.long, device=logits.device)
            logits = logits.index_select(0, order)
        return logits

    def _forward(self, entries: List[StepEntry]) -> torch.Tensor:
        try:
            ctx = self.build_context(entries)
        except CacheFull as e:
            raise StepError(str(e)) from e
        logits = self.model.forward(ctx)
        for e in entries:
            self.cache.commit(e.slot, len(e.tokens))
        self.steps_run += 1
        return logits

    def _split(self, entries: List[StepEntry]):
        """Cuts a step into passes of at most max_step_tokens tokens. Returns the passes
        and, for every output row in pass order, its index in the caller's order."""
        budget = self.max_step_tokens
        row0, rows = 0, []
        for e in entries:
            rows.append({int(w): [] for w in e.want})
            for k, w in enumerate(e.want):
                rows[-1][int(w)].append(row0 + k)
            row0 += len(e.want)
        parts, origin, cur, room = [], [], [], budget
        for ei, e in enumerate(entries):
            toks = list(e.tokens)
            off = 0
            while off < len(toks):
                if room == 0:
                    parts.append(cur)
                    cur, room = [], budget
                n = min(room, len(toks) - off)
                want_here = sorted(w for w in rows[ei] if off <= w < off + n)
                wl = []
                for w in want_here:
                    for gi in rows[ei][w]:
                        wl.append(w - off)
                        origin.append(gi)
                cur.append(StepEntry(e.slot, toks[off:off + n], wl,
                                     None if e.positions is None else list(e.positions)[off:off + n]))
                off += n
                room -= n
                if off < len(toks):   # the rest of this sequence needs a later pass
                    parts.append(cur)
                    cur, room = [], budget
        if cur:
            parts.append(cur)
        return parts, origin

    # ------------------------------------------------------------ generation
    def check_kernels(self) -> None:
        """Raises KernelError if a kernel of an earlier step gave up on one of its bounded
        waits (its output is then not to be used); waits for the device. The engine stays
        usable: the flag and the kernels' shared counters are put back."""
        K.check_error_flags()

    def run(self, entries, configs, uniforms) -> List[int]:
        """Backend face of the generation loop: feeds each (slot, tokens), samples one
        token per sequence from the logits at its last token, returns them on the host."""
        toks = self.run_device(entries, configs, uniforms).tolist()
        self.check_kernels()
        return toks

    def run_device(self, entries, configs, uniforms, tokens_on_device=None) -> torch.Tensor:
        """As `run`, but the sampled tokens stay on the device (int32 [len(entries)])."""
        if self.use_graphs and self.model.graph_safe and all(t is not None and len(t) for _, t in entries) \
                and self.graphs.takes([len(t) for _, t in entries]):
            self._validate([StepEntry(s, t, [len(t) - 1]) for s, t in entries])
            try:
                return self.graphs.step(entries, configs, uniforms, tokens_on_device)
            except CacheFull as e:
                raise StepError(str(e)) from e
        if tokens_on_device is not None:
            toks = tokens_on_device.tolist()
            entries = [(s, [toks[i]]) for i, (s, _) in enumerate(entries)]
        logits = self.step([StepEntry(s, t, [len(t) - 1]) for s, t in entries])
        return self.sampler.pick(logits, configs, uniforms)

    def launch(self, entries, configs, uniforms, after=None, rows=None) -> "_InFlight":
        """Starts a step and returns without waiting for it: the generation loop's way to
        keep the device busy while the host reads the step before. With `after` (the handle
        of the step before) every entry's token is taken on the device from row rows[k] of
        that step's sampled tokens; the entries then carry no token of their own."""
        n = len(entries)
        if after is not None:
            fed = after.dev
            if list(rows) != list(range(fed.shape[0])):
                idx = torch.tensor(list(rows), dtype=torch.int64).to(self.device, non_blocking=True)
                fed = fed.index_select(0, idx)
            dev = self.run_device([(s, [0]) for s, _ in entries], configs, uniforms, tokens_on_device=fed)
        else:
            dev = self.run_device(entries, configs, uniforms)
        # two steps are alive at a time (the one being read and the one run ahead); four
        # pinned buffers in turn leave room to spare
        ring = self.__dict__.setdefault("_host_ring", [])
        if not ring:
            # the tokens, and behind them the kernels' error flag as it stands after the step
            ring.extend(torch.zeros((max(self.cache.max_slots, 1) + 1,), dtype=torch.int32).pin_memory()
                        for _ in range(4))
        self._launched = getattr(self, "_launched", 0) + 1
        host = ring[self._launched % len(ring)]
        host[:n].copy_(dev[:n], non_blocking=True)
        host[-1:].copy_(K.error_flag(self.device), non_blocking=True)
        done = torch.cuda.Event()
        done.record()
        return _InFlight(dev[:n], host, done, n)

    def collect(self, handle: "_InFlight") -> List[int]:
        """The sampled tokens of a launched step, on the host. Raises KernelError instead if
        a kernel of that step (or of one before it) gave up on a bounded wait."""
        handle.done.synchronize()
        if int(handle.host[-1]) != 0:
            torch.cuda.synchronize(self.device)      # the step run ahead is abandoned with it
            K.recover(self.device)
            raise KernelError(f"a kernel on {self.device} gave up waiting for its own copies; "
                              "the step's tokens are not valid")
        return handle.host[:handle.n].tolist()

    def generate(self, requests, eos_token_ids=None, max_batch: int = 64, on_token=None):
        """`requests`: one GenerateRequest or a list. Returns GenerateOutput(s)."""
        from .generate import GenerateRequest, generate
        single = isinstance(requests, GenerateRequest)
        reqs = [requests] if single else list(requests)
        eos = self.spec.eos_token_ids if eos_token_ids is None else eos_token_ids
        outs = generate(self, reqs, eos, max_batch=min(max_batch, self.cache.max_slots),
                        token_budget=self.cache.n_pages * PAGE, on_token=on_token)
        return outs[0] if single else outs
