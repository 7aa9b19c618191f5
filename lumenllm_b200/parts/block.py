"""Arrangements of a mixer and a feed-forward around the residual stream.

"pre_norm": r = h + mixer(norm_mixer(h)); h' = r + ffn(norm_ffn(r))
(crates/aegisllm-cuda/src/executor/prefill/layer.rs:476-482,1090,1381-1439).
The adds are not done here: a block hands its last update on as `pending`, and
the next norm (the next block's, or the model's final one) adds it while it
reads the stream anyway.
"""
from __future__ import annotations

from .base import build_part, part_tensors, register_part


@register_part("block", "pre_norm")
class PreNormBlock:
    @classmethod
    def tensors(cls, layer_spec):
        t = {}
        t.update(part_tensors("norm", layer_spec.norms["mixer"]))
        t.update(part_tensors("mixer", layer_spec.mixer))
        t.update(part_tensors("norm", layer_spec.norms["ffn"]))
        t.update(part_tensors("ffn", layer_spec.ffn))
        return t

    def __init__(self, layer_spec, weights, runtime):
        self.runtime = runtime
        self.norm_mixer = build_part("norm", layer_spec.norms["mixer"], weights, runtime)
        self.mixer = build_part("mixer", layer_spec.mixer, weights, runtime)
        self.norm_ffn = build_part("norm", layer_spec.norms["ffn"], weights, runtime)
        self.ffn = build_part("ffn", layer_spec.ffn, weights, runtime)

    def forward(self, h, pending, ctx, entry):
        # A part that says `adds_residual` is offered the stream itself: it may add its update
        # there (a prompt-sized product does so in its epilogue) and return None, or return the
        # update as any part does. Either way the next norm sees the stream plus what is pending.
        y = self.norm_mixer.forward(h, pending, self.runtime.dtype)
        if getattr(self.mixer, "adds_residual", False):
            a = self.mixer.forward(y, ctx, entry, residual=h)
        else:
            a = self.mixer.forward(y, ctx, entry)
        y2 = self.norm_ffn.forward(h, a, self.runtime.dtype)
        if getattr(self.ffn, "adds_residual", False):
            m = self.ffn.forward(y2, ctx, residual=h)
        else:
            m = self.ffn.forward(y2, ctx)
        return h, m
