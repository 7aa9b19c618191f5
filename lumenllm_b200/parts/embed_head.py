"""Token embedding and output head.

Embedding: h[t] = float32(E[token[t]]) (norm_rope_kv.cu:19-34), optionally times a
scale (none for Qwen: crates/aegisllm-base/src/model/mod.rs:128-130).
Head: logits = y W^T in float32, with W the embedding table when the head is tied
(crates/aegisllm-cuda/src/executor/full.rs:171-181; executor/forward.rs:288-297).
"""
from __future__ import annotations

from ..ops import kernels as K
from .base import need, register_part
from .linear import Linear


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
        self.scale = spec.params.get("scale")

    def forward(self, tokens):
        h = K.embed(tokens, self.table)
        if self.scale is not None:
            h.mul_(float(self.scale))
        return h


@register_part("head", "linear_head")
class LinearHead:
    @classmethod
    def tensors(cls, spec):
        if spec.params.get("tied_to"):
            return {}
        return {f"{spec.prefix}.weight": ((int(need(spec.params, "vocab_size", "head")),
                                           int(need(spec.params, "hidden_size", "head"))), "matrix")}

    def __init__(self, spec, weights, runtime):
        name = spec.params.get("tied_to") or f"{spec.prefix}.weight"
        self.proj = Linear(weights[name], runtime)

    def forward(self, y):
        return self.proj(y)
