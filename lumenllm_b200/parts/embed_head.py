"""Token embedding and output head.

Embedding: h[t] = float32(E[token[t]]) (norm_rope_kv.cu:19-34), optionally times a
scale (none for Qwen: crates/aegisllm-base/src/model/mod.rs:128-130).
Head: logits = y W^T in float32, with W the embedding table when the head is tied
(crates/aegisllm-cuda/src/executor/full.rs:171-181; executor/forward.rs:288-297).
"""
from __future__ import annotations

from ..ops import kernels as K
from .base import need, register_part
from .linear import Linear, tiled_form


@register_part("embedding", "token_embedding")
class TokenEmbedding:
    @classmethod
    def tensors(cls, spec):
        return {f"{spec.prefix}.weight": ((int(need(spec.params, "vocab_size", "embedding")),
                                           int(need(spec.params, "hidden_size", "embedding"))),
                                          "matrix")}

    def __init__(self, spec, weights, runtime):
        self.table = weights[f"{spec.prefix}.weight"].contiguous()
        self.vocab_size = self.table.shape[0]
        # in a bfloat16 run the table is kept in the form an output head would read it in, so
        # that a head tied to it shares the one copy
        if not runtime.is_f32 and K.can_tile(self.table):
            self.table = tiled_form(self.table)
        self.scale = spec.params.get("scale")

    def forward(self, tokens):
        h = K.embed(tokens, self.table)
        if self.scale is not None:
            h.mul_(float(self.scale))
        return h


@register_part("head", "linear_head")
class LinearHead:
    """`tied_to` names the embedding table when config.json ties the head to it. Which matrix
    is used follows the reference, by presence (executor/full.rs:171-181): the head's own
    tensor when the file stores one, else the table named by `tied_to` or `falls_back_to`.
    So a tied checkpoint that also stores a head, and an untied one that stores none, both
    load; the loader reports the second case in its `stood_in`."""

    @classmethod
    def tensors(cls, spec):
        shape = (int(need(spec.params, "vocab_size", "head")), int(need(spec.params, "hidden_size", "head")))
        return {f"{spec.prefix}.weight": (shape, "optional" if spec.params.get("tied_to") else "matrix")}

    @classmethod
    def fallbacks(cls, spec):
        other = spec.params.get("falls_back_to")
        return {f"{spec.prefix}.weight": other} if other and not spec.params.get("tied_to") else {}

    def __init__(self, spec, weights, runtime):
        own = f"{spec.prefix}.weight"
        name = own if own in weights else spec.params.get("tied_to")
        if name is None or name not in weights:
            raise KeyError(f"the output head needs '{own}'")
        self.proj = Linear(weights[name], runtime)

    def forward(self, y):
        return self.proj(y)
