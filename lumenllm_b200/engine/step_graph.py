"""Steps replayed from CUDA graphs.

A decode step (every live sequence brings one token) is some hundreds of short
kernels, and so is the step that takes a batch's prompts while these are short;
launched one by one the host cannot keep up with the device. Such steps are
therefore captured once per shape and replayed. The shape of a step is its
number of tokens, its number of sequences and the width of its page table, each
rounded up to a bucket; padding sequences make up the difference and change no
result: they start at position 0 with a page table of zeros, so they write to
the cache's spare page 0 and to the state store's spare row. How the tokens are
divided among the sequences is NOT part of the shape: the kernels read that from
the device (cu_q, seq_start), so one captured prompt step serves every batch of
prompts that fits its buckets. Everything that differs from step to step (tokens,
positions, page tables, sampling options and uniform numbers) lives in two small
device buffers at fixed addresses that one copy from pinned memory refreshes
before each replay. The reference does the same for the decode step of its single
sequence (crates/aegisllm-cuda/src/executor/forward.rs:439-503;
cuda/runtime/graph.rs:8-32).
"""
from __future__ import annotations

import gc
import weakref
from collections import OrderedDict
from typing import Dict, List, Sequence, Tuple

import numpy as np
import torch

from ..cache.kv import pages_for
from ..ops import kernels as K
from .context import StepEntry, StepLayout, context_on, pack_step, padding_twin, upload

# A prompt step of more tokens than this is launched kernel by kernel: the device then takes
# longer over it than the host does, and a bucket would waste more than the replay saves.
PROMPT_GRAPH_MAX_TOKENS = 1024
# Captured prompt steps kept (least recently used first out); decode steps are always kept.
PROMPT_GRAPHS_KEPT = 16


def _bucket(n: int, small=(1, 2, 4, 8, 16, 32, 64)) -> int:
    for b in small:
        if n <= b:
            return b
    return (n + 63) // 64 * 64


def _token_bucket(n: int) -> int:
    """Token count of a prompt step rounded up: to 32 up to 512 tokens (a step that short is a
    stream over the weights, and more rows cost next to nothing), then to 64."""
    g = 32 if n <= 512 else 64
    return (n + g - 1) // g * g


def _pow2(n: int) -> int:
    p = 1
    while p < n:
        p *= 2
    return p


class _Captured:
    def __init__(self, graph, meta, opts, top_k, logits, next_tok, ctx):
        self.graph, self.meta, self.opts, self.top_k = graph, meta, opts, top_k
        self.logits, self.next_tok, self.ctx = logits, next_tok, ctx


class StepGraphs:
    def __init__(self, engine):
        # no strong reference back to the engine: an engine that is dropped must free its
        # graphs at once, not whenever the cycle collector runs (which may be in the middle
        # of another engine's capture, where destroying a graph is not permitted)
        self._engine = weakref.ref(engine)
        # key: (tokens, sequences, page-table width, greedy), each a bucket; a decode step
        # has as many tokens as sequences
        self.captured: "OrderedDict[Tuple[int, int, int, bool], _Captured]" = OrderedDict()
        self.min_width = 1      # page-table width to capture for at least (saves re-captures)
        self._pool = None       # one memory pool for all graphs: they never run side by side

    @property
    def engine(self):
        eng = self._engine()
        if eng is None:
            raise RuntimeError("the engine of these graphs is gone")
        return eng

    def takes(self, lens: Sequence[int]) -> bool:
        """Whether a step whose sequences bring `lens` tokens is replayed from a graph."""
        n_tok = sum(lens)
        return n_tok == len(lens) or n_tok <= min(PROMPT_GRAPH_MAX_TOKENS, self.engine.max_step_tokens)

    @staticmethod
    def plan(lens: Sequence[int]):
        """(token bucket, sequence bucket, lengths of the padding sequences) for a step."""
        n, n_tok = len(lens), sum(lens)
        if n_tok == n:                                   # one token each
            Bb = _bucket(n)
            return Bb, Bb, [1] * (Bb - n)
        Bb = _bucket(n + 1)                              # the first padding sequence takes the
        Nb = _token_bucket(n_tok)                        # tokens that fill the bucket (maybe none),
        return Nb, Bb, [Nb - n_tok] + [0] * (Bb - n - 1)  # the others are empty

    def _capture(self, key, lay: StepLayout, lists, host) -> _Captured:
        eng = self.engine
        _, Bb, _, greedy = key
        dev = eng.device
        meta = torch.zeros((lay.total,), dtype=torch.int32, device=dev)
        opts = torch.zeros((Bb, 4), dtype=torch.float32, device=dev)
        top_k = torch.zeros((Bb,), dtype=torch.int32, device=dev)
        next_tok = torch.zeros((Bb,), dtype=torch.int32, device=dev)
        q_lens, starts, slots, n_real = lists
        ctx = context_on(meta, lay, q_lens, starts, slots, n_real, eng.cache, eng.runtime)
        ctx.extras["captured"] = True
        # The step is run once before it is captured (library workspaces, kernel attributes).
        # That run sees padding sequences only, so it changes no live sequence's cache or state;
        # the capture itself runs nothing, and the first replay is the step's one execution.
        upload(padding_twin(host, lay, q_lens, eng.cache.state.pad_row), meta)

        def body():
            logits = eng.model.forward(ctx)
            if greedy:
                K.argmax(logits, out=next_tok)
            else:
                K.sample(logits, opts, top_k, out=next_tok)
            return logits

        cur = torch.cuda.current_stream()
        side = torch.cuda.Stream()
        side.wait_stream(cur)
        with torch.cuda.stream(side):
            body()                       # warm-up: library workspaces, kernel attributes
        cur.wait_stream(side)
        torch.cuda.synchronize()
        from ..ops import native
        if self._pool is None:
            self._pool = torch.cuda.graph_pool_handle()
        graph = torch.cuda.CUDAGraph()
        before = native.launches
        gc.collect()
        was_enabled = gc.isenabled()
        gc.disable()          # no finaliser may touch CUDA while the stream is capturing
        try:
            with torch.cuda.graph(graph, pool=self._pool):
                logits = body()
        finally:
            if was_enabled:
                gc.enable()
        cap = _Captured(graph, meta, opts, top_k, logits, next_tok, ctx)
        cap.kernels_per_replay = native.launches - before
        return cap

    def step(self, entries: Sequence[Tuple[int, Sequence[int]]], configs, uniforms,
             tokens_on_device: torch.Tensor = None) -> torch.Tensor:
        """One step for (slot, tokens) entries, every one of which wants the token after its
        last; returns the next tokens, int32 [len(entries)], on the device. With
        tokens_on_device (int32 [len(entries)], one-token steps only) the fed tokens are taken
        from there instead of from the entries, without the host ever seeing them."""
        eng = self.engine
        n = len(entries)
        lens = [len(t) for _, t in entries]
        Nb, Bb, pad_lens = self.plan(lens)
        se = [StepEntry(s, t, [len(t) - 1]) for s, t in entries]
        need = max(eng.cache.length(e.slot) + len(e.tokens) for e in se)
        need = max(need, max(pad_lens, default=1), 1)
        Wb = min(_pow2(max(1, pages_for(need))), max(eng.cache.max_pages_per_seq, 1))
        Wb = max(Wb, pages_for(need), min(self.min_width, eng.cache.max_pages_per_seq))
        greedy = all(c.greedy for c in configs)
        key = (Nb, Bb, Wb, greedy)
        host, lay, q_lens, starts, slots, n_real = pack_step(eng.cache, se, pad_to=Bb, table_width=Wb,
                                                             want_padding=True, pad_lens=pad_lens)
        cap = self.captured.get(key)
        if cap is None:
            cap = self._capture(key, lay, (q_lens, starts, slots, n_real), host)
            self.captured[key] = cap
            prompts = [k for k in self.captured if k[0] != k[1]]
            for old in prompts[:max(0, len(prompts) - PROMPT_GRAPHS_KEPT)]:
                del self.captured[old]
        else:
            self.captured.move_to_end(key)
        upload(host, cap.meta)
        if tokens_on_device is not None:
            if Nb != Bb:
                raise ValueError("tokens on the device can only feed a step of one token each")
            cap.ctx.tokens[:n].copy_(tokens_on_device[:n])
        if not greedy:
            o = np.zeros((Bb, 4), dtype=np.float32)
            k = np.zeros((Bb,), dtype=np.int32)
            for i, (c, u) in enumerate(zip(configs, uniforms)):
                o[i] = (c.temperature, c.top_p, c.min_p, u)
                k[i] = c.top_k
            cap.opts.copy_(torch.from_numpy(o).pin_memory(), non_blocking=True)
            cap.top_k.copy_(torch.from_numpy(k).pin_memory(), non_blocking=True)
        cap.graph.replay()
        for e in se:
            eng.cache.commit(e.slot, len(e.tokens))
        eng.steps_run += 1
        self.last = cap
        return cap.next_tok[:n]

