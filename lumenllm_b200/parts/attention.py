"""The attention mixer: grouped-query causal attention over the cache.

In order (crates/aegisllm-cuda/src/executor/attention.rs:139-202,241-250,341-352,
413-425; prompt twin executor/prefill/layer.rs:472-636,810-823,967-1047):
q, k, v = y Wq^T, y Wk^T, y Wv^T; optional per-head RMSNorm of q and k with a
weight of head_dim values; rotation of q and k; k, v appended to the cache at the
token's position; for query head h the kv head is h // (heads / kv_heads)
(attention_decode_common.cuh:112-115), scores scaled by `softmax_scale`, a query
at position p sees keys j <= p (and p - j < window if a window is set); o = ctx Wo^T.
Softmax, norms and angles are float32.
"""
from __future__ import annotations

import torch

from ..cache.kv import CacheNeed
from ..ops import kernels as K
from .base import build_part, need, part_tensors, register_part
from .linear import Linear


# Batches of a decode step for which the attention kernel does the rotary kernel's work itself
# (ops.kernels.attn_decode_qkv; the same bits either way). It saves a kernel and its wait on the
# step's path, and costs every block of a sequence's segments the making of its query heads:
# at the 8B shape 2,455 against 2,424 tokens/s at batch 8 and 4,428 against 4,372 at 16, but
# 6,985 against 7,083 at 32 and 10,290 against 10,600 at 64; at batch 1 338 against 340.
FUSED_DECODE_ROWS = (4, 16)


@register_part("mixer", "gqa_attention")
class GQAttention:
    graph_safe = True

    @classmethod
    def tensors(cls, spec):
        p = spec.params
        H, nq, nkv, d = (int(need(p, k, "gqa_attention")) for k in
                         ("hidden_size", "num_heads", "num_kv_heads", "head_dim"))
        t = {f"{spec.prefix}.q_proj.weight": ((nq * d, H), "matrix"),
             f"{spec.prefix}.o_proj.weight": ((H, nq * d), "matrix")}
        if not p.get("shares_cache", False):
            t[f"{spec.prefix}.k_proj.weight"] = ((nkv * d, H), "matrix")
            t[f"{spec.prefix}.v_proj.weight"] = ((nkv * d, H), "matrix")
        if p.get("qk_norm", False):
            t[f"{spec.prefix}.q_norm.weight"] = ((d,), "norm")
            if not p.get("shares_cache", False):
                t[f"{spec.prefix}.k_norm.weight"] = ((d,), "norm")
        t.update(part_tensors("position", p["position"]))
        return t

    def __init__(self, spec, weights, runtime):
        p = spec.params
        self.runtime = runtime
        self.H = int(p["hidden_size"])
        self.nq, self.nkv, self.d = int(p["num_heads"]), int(p["num_kv_heads"]), int(p["head_dim"])
        if self.nq % self.nkv:
            raise ValueError(f"{self.nq} heads are not a multiple of {self.nkv} kv heads")
        if self.d % 16 or self.d > 256:
            raise ValueError(f"head_dim {self.d}: the attention kernels take multiples of 16 up to 256")
        self.window = int(p.get("window", 0) or 0)
        self.scale = float(need(p, "softmax_scale", "gqa_attention"))
        self.shares_cache = bool(p.get("shares_cache", False))
        self.position = build_part("position", p["position"], weights, runtime)
        pre = spec.prefix
        mats = [weights[f"{pre}.q_proj.weight"]]
        if not self.shares_cache:
            mats += [weights[f"{pre}.k_proj.weight"], weights[f"{pre}.v_proj.weight"]]
        self.qkv = Linear.stacked(mats, runtime)
        # a run that reads another run's cache projects queries only
        self.q_only = self.qkv if self.shares_cache else self.qkv.first_rows(self.nq * self.d)
        self.o = Linear(weights[f"{pre}.o_proj.weight"], runtime)
        self.q_norm = self.k_norm = None
        self.qk_eps = float(p.get("qk_norm_eps", 0.0))
        if p.get("qk_norm", False):
            off = float(p.get("qk_norm_weight_offset", 0.0))
            f32 = lambda n: (weights[n].to(device=runtime.device, dtype=torch.float32) + off).contiguous()
            self.q_norm = f32(f"{pre}.q_norm.weight")
            if not self.shares_cache:
                self.k_norm = f32(f"{pre}.k_norm.weight")

    def cache_need(self):
        return CacheNeed(self.nkv, self.d, self.window)

    def state_shape(self):
        return None

    adds_residual = True      # forward takes `residual` and may add its update to it in place

    def forward(self, y, ctx, entry, residual=None):
        kc, vc, table = entry.cache()
        writes = entry.writes_cache and not self.shares_cache
        if (writes and not self.qkv.f32 and entry.layout == K.LAYOUT_SW128 and y.is_contiguous()
                and K.gemm_tc_qkv_takes(y.shape[0], self.qkv.out_features, self.qkv.in_features, self.nq,
                                        self.nkv, self.d, self.position.rotary_dim)):
            # a prompt with heads of 128: norm, rotation and cache write in the product's epilogue
            q = K.gemm_tc_qkv(y, self.qkv.weight, self.q_norm, self.k_norm, self.qk_eps,
                              self.position.angles(ctx), self.position.rotary_dim, ctx.cache_pos,
                              ctx.tok_seq, table, kc, vc, self.nq, self.nkv)
            out = self.attend(q, kc, vc, table, ctx, entry.layout)
            return self.o(out.view(-1, self.nq * self.d), split_ok=True, add_to=residual)
        # float32 [N, (nq + 2 nkv) d], possibly as S partial sums
        qkv = self.qkv(y, split_ok=True) if writes else self.q_only(y, split_ok=True)
        if (writes and ctx.is_decode and FUSED_DECODE_ROWS[0] <= ctx.B <= FUSED_DECODE_ROWS[1]
                and entry.layout == K.LAYOUT_SW128 and self.d == 128
                and self.nq // self.nkv <= 16 and self.position.rotary_dim in (0, 128)
                and kc.dtype == torch.bfloat16):
            # one token a sequence, heads of 128: the attention blocks make their query heads and
            # the new key and value themselves, from the projection's partial sums
            out = K.attn_decode_qkv(qkv, self.q_norm, self.k_norm, self.qk_eps, self.position.angles(ctx),
                                    self.position.rotary_dim, kc, vc, table, ctx.cache_pos, self.window,
                                    self.scale, self.nq, self.nkv)
            return self.o(out.view(-1, self.nq * self.d), split_ok=True, add_to=residual)
        nkv_new = self.nkv if writes else 0
        q = K.qk_norm_rope_store(qkv, self.q_norm, self.k_norm, self.qk_eps,
                                 self.position.angles(ctx), self.position.rotary_dim,
                                 ctx.cache_pos, ctx.tok_seq, table,
                                 kc if nkv_new else None, vc if nkv_new else None,
                                 self.nq, nkv_new, self.d, self.runtime.dtype, layout=entry.layout)
        out = self.attend(q, kc, vc, table, ctx, entry.layout)
        return self.o(out.view(-1, self.nq * self.d), split_ok=True, add_to=residual)

    def attend(self, q, kc, vc, table, ctx, layout):
        """Chooses the kernel by the step's shape: the split-KV kernel when every sequence
        brings one token, the flash kernel for prompts, and the general kernel for the
        32-bit path and for head sizes the fast kernels do not take. All agree within rounding."""
        fast = (layout == K.LAYOUT_SW128 and q.dtype == torch.bfloat16 and self.d in (64, 128)
                and self.nq // self.nkv <= 16)
        if fast and ctx.is_decode:
            return K.attn_decode(q, kc, vc, table, ctx.cache_pos, self.window, self.scale)
        if fast:
            # a captured step is replayed for other divisions of its tokens than the one it was
            # captured with: the kernel then takes the division from the device alone
            q_lens = None if ctx.extras.get("captured") else ctx.q_lens
            return K.attn_prefill(q, kc, vc, table, ctx.cu_q, ctx.seq_start, q_lens, self.window,
                                  self.scale, n_seqs=ctx.B)
        return K.attn_generic(q, kc, vc, table, ctx.tok_seq, ctx.cache_pos, self.window, self.scale,
                              layout=layout)
