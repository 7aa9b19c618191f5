"""A decoder put together from a ModelSpec: embedding, blocks run in the order of
the schedule, final norm on the wanted rows, head.
"""
from __future__ import annotations

from typing import Dict, Tuple

import torch

from ..cache.kv import CacheNeed
from ..config.spec import ModelSpec
from ..parts import build_part, part_class, part_tensors
from ..parts.base import Runtime
from .context import EntryView, StepContext


def expected_tensors(spec: ModelSpec) -> Dict[str, Tuple[Tuple[int, ...], str]]:
    """Every tensor the model reads, by name, with its shape and kind: "matrix", "norm", or
    "optional" (a matrix that is read if the file stores it and not missed if it does not)."""
    t = {}
    t.update(part_tensors("embedding", spec.embedding))
    for layer in spec.layers:
        t.update(part_class("block", layer.block).tensors(layer))
    t.update(part_tensors("norm", spec.final_norm))
    t.update(part_tensors("head", spec.head))
    return t


def tensor_fallbacks(spec: ModelSpec) -> Dict[str, str]:
    """{tensor: the stored tensor that may stand in when it is absent}, as parts declare."""
    f = getattr(part_class("head", spec.head.kind), "fallbacks", None)
    return dict(f(spec.head)) if f else {}


class DecoderModel:
    def __init__(self, spec: ModelSpec, weights: Dict[str, torch.Tensor], runtime: Runtime):
        spec.validate()
        self.spec = spec
        self.runtime = runtime
        self.embedding = build_part("embedding", spec.embedding, weights, runtime)
        self.blocks = [part_class("block", l.block)(l, weights, runtime) for l in spec.layers]
        self.final_norm = build_part("norm", spec.final_norm, weights, runtime)
        self.head = build_part("head", spec.head, weights, runtime)
        self.schedule = spec.schedule
        # a step can be captured in a CUDA graph only if no part looks at the step's
        # host-side lists; parts say so with `graph_safe = True`
        self.graph_safe = all(getattr(b.mixer, "graph_safe", False) and
                              getattr(b.ffn, "graph_safe", False) for b in self.blocks)

    # what the cache must hold, per schedule entry
    def cache_needs(self) -> Dict[int, CacheNeed]:
        needs = {}
        for i, e in enumerate(self.schedule):
            if e.cache_from is None:
                need = self.blocks[e.layer].mixer.cache_need()
                if need is not None:
                    needs[i] = need
        return needs

    def state_shapes(self):
        shapes = {}
        for i, e in enumerate(self.schedule):
            s = self.blocks[e.layer].mixer.state_shape()
            if s is not None:
                shapes[i] = s
        return shapes

    def forward(self, ctx: StepContext) -> torch.Tensor:
        """Logits float32 [W, V] at ctx.want_rows."""
        ctx.extras.pop("per_step", None)     # tables that parts share within ONE step
        h = self.embedding.forward(ctx.tokens)
        pending = None
        needs = ctx.cache.group_of
        for i, e in enumerate(self.schedule):
            src = i if e.cache_from is None else e.cache_from
            view = EntryView(ctx, i, src if src in needs else None, e.cache_from is None)
            h, pending = self.blocks[e.layer].forward(h, pending, ctx, view)
        if ctx.want_rows.numel() == 0:
            # nothing wanted: the stream still has to take its last update? No reader
            # follows, so the update is dropped with the stream.
            return torch.empty((0, self.spec.vocab_size), dtype=torch.float32,
                               device=self.runtime.device)
        y = self.final_norm.forward(h, pending, self.runtime.dtype, rows=ctx.want_rows,
                                    write_h=False)
        return self.head.forward(y)
