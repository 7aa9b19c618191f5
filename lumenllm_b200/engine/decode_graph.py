"""Decode steps replayed from CUDA graphs.

A decode step (every live sequence brings one token) is some hundreds of short
kernels; launched one by one the host cannot keep up with the device. The step
is therefore captured once per shape (batch size and page-table width, both
rounded up to fixed buckets; padding rows make up the difference and change no
result) and replayed. Everything that differs from step to step (tokens,
positions, page tables, sampling options and uniform numbers) lives in two
small device buffers at fixed addresses that one copy from pinned memory
refreshes before each replay. The reference does the same for its single
sequence (crates/aegisllm-cuda/src/executor/forward.rs:439-503;
cuda/runtime/graph.rs:8-32).
"""
from __future__ import annotations

import gc
import weakref
from typing import Dict, List, Sequence, Tuple

import numpy as np
import torch

from ..cache.kv import pages_for
from ..ops import kernels as K
from .context import StepEntry, StepLayout, context_on, pack_step, upload


def _bucket(n: int, small=(1, 2, 4, 8, 16, 32, 64)) -> int:
    for b in small:
        if n <= b:
            return b
    return (n + 63) // 64 * 64


def _pow2(n: int) -> int:
    p = 1
    while p < n:
        p *= 2
    return p


class _Captured:
    def __init__(self, graph, meta, opts, top_k, logits, next_tok, ctx):
        self.graph, self.meta, self.opts, self.top_k = graph, meta, opts, top_k
        self.logits, self.next_tok, self.ctx = logits, next_tok, ctx


class DecodeGraphs:
    def __init__(self, engine):
        # no strong reference back to the engine: an engine that is dropped must free its
        # graphs at once, not whenever the cycle collector runs (which may be in the middle
        # of another engine's capture, where destroying a graph is not permitted)
        self._engine = weakref.ref(engine)
        self.captured: Dict[Tuple[int, int, bool], _Captured] = {}
        self.min_width = 1      # page-table width to capture for at least (saves re-captures)

    @property
    def engine(self):
        eng = self._engine()
        if eng is None:
            raise RuntimeError("the engine of these graphs is gone")
        return eng

    def _capture(self, key, lay: StepLayout, host, lists) -> _Captured:
        eng = self.engine
        Bb, _, greedy = key
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
        pad_host, pad_lay = pack_step(eng.cache, [], pad_to=Bb, table_width=lay.width,
                                      want_padding=True)[:2]
        assert pad_lay.total == lay.total and pad_lay.offs == lay.offs
        upload(pad_host, meta)

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
        graph = torch.cuda.CUDAGraph()
        before = native.launches
        gc.collect()
        was_enabled = gc.isenabled()
        gc.disable()          # no finaliser may touch CUDA while the stream is capturing
        try:
            with torch.cuda.graph(graph):
                logits = body()
        finally:
            if was_enabled:
                gc.enable()
        cap = _Captured(graph, meta, opts, top_k, logits, next_tok, ctx)
        cap.kernels_per_replay = native.launches - before
        return cap

    def step(self, entries: Sequence[Tuple[int, Sequence[int]]], configs, uniforms,
             tokens_on_device: torch.Tensor = None) -> torch.Tensor:
        """One decode step for (slot, [token]) entries; returns the next tokens, int32
        [len(entries)], on the device. With tokens_on_device (int32 [len(entries)]) the
        fed tokens are taken from there instead of from the entries, without the host
        ever seeing them."""
        eng = self.engine
        n = len(entries)
        Bb = _bucket(n)
        se = [StepEntry(s, t, [0]) for s, t in entries]
        need = max(eng.cache.length(e.slot) + 1 for e in se)
        Wb = min(_pow2(max(1, pages_for(need))), max(eng.cache.max_pages_per_seq, 1))
        Wb = max(Wb, pages_for(need), min(self.min_width, eng.cache.max_pages_per_seq))
        greedy = all(c.greedy for c in configs)
        key = (Bb, Wb, greedy)
        host, lay, q_lens, starts, slots, n_real = pack_step(eng.cache, se, pad_to=Bb, table_width=Wb,
                                                             want_padding=True)
        cap = self.captured.get(key)
        if cap is None:
            cap = self._capture(key, lay, host, (q_lens, starts, slots, n_real))
            self.captured[key] = cap
        upload(host, cap.meta)
        if tokens_on_device is not None:
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
            eng.cache.commit(e.slot, 1)
        eng.steps_run += 1
        self.last = cap
        return cap.next_tok[:n]
