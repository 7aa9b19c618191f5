"""Plain, slow Qwen3-dense decoder: whole sequences, no cache, one function per part.

This file is the oracle of the test-suite. It shares no code with the product
package: it reads a model folder with its own tiny safetensors parser, keeps
everything in float32 on the CPU and recomputes every sequence from its first
token.

It rests on the formulas of the reference project (demented484/LumenLLM), which
cannot be compiled or imported here (Rust + CUDA, no Rust toolchain, no GPU on
the build machine), so no golden vector from the reference's own code exists;
every function below cites the reference line that states its formula.
"""
from __future__ import annotations

import json
import math
import struct
from pathlib import Path

import torch

_DT = {
    "F32": (torch.float32, 4),
    "BF16": (torch.bfloat16, 2),
    "F16": (torch.float16, 2),
    "I32": (torch.int32, 4),
    "I64": (torch.int64, 8),
}


def read_safetensors(path):
    """[u64 LE header length][JSON header][payload]
    (crates/aegisllm-base/src/tensor/core.rs:86-181)."""
    raw = Path(path).read_bytes()
    (hlen,) = struct.unpack("<Q", raw[:8])
    header = json.loads(raw[8 : 8 + hlen])
    payload = memoryview(raw)[8 + hlen :]
    out = {}
    for name, info in header.items():
        if name == "__metadata__":
            continue
        dt, _ = _DT[info["dtype"]]
        b, e = info["data_offsets"]
        t = torch.frombuffer(bytearray(payload[b:e]), dtype=dt)
        out[name] = t.reshape(info["shape"]).clone()
    return out


def load_model(folder):
    """Returns (config dict, weights as float32 tensors by name)."""
    folder = Path(folder)
    cfg = json.loads((folder / "config.json").read_text())
    w = {k: v.to(torch.float32) for k, v in read_safetensors(folder / "model.safetensors").items()}
    return cfg, w


# ---------------------------------------------------------------- parts


def rms_norm(x, weight, eps):
    """y_i = x_i * 1/sqrt(mean(x^2) + eps) * w_i
    (crates/aegisllm-cpu/src/cpu/math.rs:4-8;
    crates/aegisllm-cuda/src/cuda/kernels/blackwell/norm_rope_kv.cu:36-62)."""
    x = x.to(torch.float32)
    ms = (x * x).mean(dim=-1, keepdim=True)
    return x * (1.0 / torch.sqrt(ms + eps)) * weight


def rope_inv_freq(head_dim, theta, rotary_dim=None):
    """inv_freq_i = 1 / theta^(2i/d), float32
    (crates/aegisllm-cpu/src/cpu/rope.rs:67-68; norm_rope_kv.cu:446)."""
    rd = head_dim if rotary_dim is None else rotary_dim
    i2 = torch.arange(0, rd, 2, dtype=torch.float32)
    return 1.0 / (torch.tensor(float(theta), dtype=torch.float32) ** (i2 / rd))


def apply_rope(x, positions, theta, rotary_dim=None):
    """Half-split pairs (i, i + d/2): x'_i = x_i cos - x_{i+d/2} sin,
    x'_{i+d/2} = x_i sin + x_{i+d/2} cos, angle = pos * inv_freq_i in float32
    (norm_rope_kv.cu:465-492; crates/aegisllm-cpu/src/cpu/rope.rs:34-63).
    x: [T, heads, d]; positions: [T]."""
    d = x.shape[-1]
    rd = d if rotary_dim is None else rotary_dim
    half = rd // 2
    inv = rope_inv_freq(d, theta, rotary_dim)
    ang = positions.to(torch.float32)[:, None] * inv[None, :]  # [T, half]
    cos = torch.cos(ang)[:, None, :]
    sin = torch.sin(ang)[:, None, :]
    x0 = x[..., :half]
    x1 = x[..., half:rd]
    out = x.clone()
    out[..., :half] = x0 * cos - x1 * sin
    out[..., half:rd] = x0 * sin + x1 * cos
    return out


def _same(t):
    return t


def rounded_to(dtype):
    """A function that rounds a float32 tensor to `dtype` and widens it again: the places
    where the serving path keeps activations in 16 bits (the inputs of matrix products, the
    cache, the softmax weights that multiply the values) are marked with it below. The
    reference rounds at the same places, to float16: activations of prompt products
    (crates/aegisllm-cuda/src/cuda/runtime/cublaslt.rs:99-164), the cache
    (norm_rope_kv.cu:623-651), the weights P of the prompt attention
    (attention_prefill_dense_wmma.cu:3013-3021)."""
    return lambda t: t.to(dtype).to(torch.float32)


def causal_attention(q, k, v, window=0, scale=None, rnd=_same):
    """Full [T, T] masked softmax. Query head h reads kv head h // (nq / nkv);
    scores scaled by 1/sqrt(d); a query at position p sees keys j <= p, and with
    a window W only those with p - j < W
    (crates/aegisllm-cpu/src/attention.rs:127-236;
    attention_decode_common.cuh:112-115). With `rnd` the weights exp(s - max) are rounded
    before they multiply the values while their sum is taken unrounded, as the reference's
    prompt kernel does (attention_prefill_dense_wmma.cu:2990-2994,3013-3021).
    q: [T, nq, d], k, v: [T, nkv, d] -> [T, nq, d]."""
    T, nq, d = q.shape
    nkv = k.shape[1]
    group = nq // nkv
    if scale is None:
        scale = 1.0 / math.sqrt(d)
    out = torch.empty_like(q)
    pos = torch.arange(T)
    visible = pos[None, :] <= pos[:, None]
    if window and window > 0:
        visible &= (pos[:, None] - pos[None, :]) < window
    for h in range(nq):
        kh = h // group
        s = (q[:, h, :] @ k[:, kh, :].T) * scale
        s = s.masked_fill(~visible, float("-inf"))
        if rnd is _same:
            p = torch.softmax(s, dim=-1)
            out[:, h, :] = p @ v[:, kh, :]
        else:
            e = torch.exp(s - s.max(dim=-1, keepdim=True).values)
            out[:, h, :] = (rnd(e) @ v[:, kh, :]) / e.sum(dim=-1, keepdim=True)
    return out


def swiglu(gate, up):
    """z = g / (1 + exp(-g)) * u (norm_rope_kv.cu:314-325;
    crates/aegisllm-cpu/src/cpu/simd.rs:196-206)."""
    return gate / (1.0 + torch.exp(-gate)) * up


def embed(tokens, table):
    """h[t] = E[token[t]] (norm_rope_kv.cu:19-34); no scale for Qwen
    (crates/aegisllm-base/src/model/mod.rs:128-130)."""
    return table[tokens]


def layer_window(cfg, i):
    """Key `use_sliding_window` with `sliding_window` and `max_window_layers` of
    config.json: layers from index max_window_layers on see a window."""
    types = cfg.get("layer_types")
    if types is not None:
        return int(cfg["sliding_window"]) if types[i] == "sliding_attention" else 0
    if cfg.get("use_sliding_window", False) and cfg.get("sliding_window"):
        if i >= int(cfg.get("max_window_layers", 0)):
            return int(cfg["sliding_window"])
    return 0


def attention_block(x, w, prefix, cfg, positions, window, rnd=_same):
    """norm -> q,k,v -> per-head q/k RMSNorm -> RoPE -> attention -> o_proj
    (crates/aegisllm-cuda/src/executor/attention.rs:139-202,241-250,413-425, with
    the Gemma-only V-norm and q*sqrt(d) of :203-219,262-269 off)."""
    nq = cfg["num_attention_heads"]
    nkv = cfg.get("num_key_value_heads", nq)
    d = cfg.get("head_dim") or cfg["hidden_size"] // nq
    eps = cfg.get("rms_norm_eps", 1e-5)
    theta = cfg.get("rope_theta", 10000.0)
    T = x.shape[0]
    q = (x @ w[prefix + "self_attn.q_proj.weight"].T).view(T, nq, d)
    k = (x @ w[prefix + "self_attn.k_proj.weight"].T).view(T, nkv, d)
    v = (x @ w[prefix + "self_attn.v_proj.weight"].T).view(T, nkv, d)
    q = rms_norm(q, w[prefix + "self_attn.q_norm.weight"], eps)
    k = rms_norm(k, w[prefix + "self_attn.k_norm.weight"], eps)
    q = rnd(apply_rope(q, positions, theta))
    k = rnd(apply_rope(k, positions, theta))
    ctx = rnd(causal_attention(q, k, rnd(v), window=window, rnd=rnd))
    return ctx.reshape(T, nq * d) @ w[prefix + "self_attn.o_proj.weight"].T


def mlp_block(x, w, prefix, rnd=_same):
    """gate, up -> SwiGLU -> down (crates/aegisllm-cuda/src/executor/mlp.rs:271-356)."""
    g = x @ w[prefix + "mlp.gate_proj.weight"].T
    u = x @ w[prefix + "mlp.up_proj.weight"].T
    return rnd(swiglu(g, u)) @ w[prefix + "mlp.down_proj.weight"].T


def decoder_layer(h, w, i, cfg, positions, rnd=_same):
    """Pre-norm residual block: r = h + attn(norm1(h)); h' = r + mlp(norm2(r))
    (crates/aegisllm-cuda/src/executor/prefill/layer.rs:476-482,1090,1381-1439)."""
    p = f"model.layers.{i}."
    eps = cfg.get("rms_norm_eps", 1e-5)
    y = rnd(rms_norm(h, w[p + "input_layernorm.weight"], eps))
    r = h + attention_block(y, w, p, cfg, positions, layer_window(cfg, i), rnd)
    y2 = rnd(rms_norm(r, w[p + "post_attention_layernorm.weight"], eps))
    return r + mlp_block(y2, w, p, rnd)


def forward_logits(cfg, w, tokens, positions=None, round_to=None):
    """Logits [T, V] at every position of one whole sequence
    (final norm + head: crates/aegisllm-cuda/src/executor/forward.rs:281-298;
    tied head when lm_head.weight is absent: executor/full.rs:171-181). `positions`
    (default 0, 1, 2, ...) are what the rotation sees; the causal mask follows the order of
    the tokens (prefill/mod.rs:136-141 keeps the two apart). With `round_to` the activations
    are rounded where a 16-bit serving path rounds them (see rounded_to); the residual
    stream, norms, softmax and every sum stay float32."""
    tokens = torch.as_tensor(tokens, dtype=torch.long)
    positions = torch.arange(tokens.numel()) if positions is None else torch.as_tensor(positions)
    rnd = _same if round_to is None else rounded_to(round_to)
    h = embed(tokens, w["model.embed_tokens.weight"])
    for i in range(cfg["num_hidden_layers"]):
        h = decoder_layer(h, w, i, cfg, positions, rnd)
    y = rnd(rms_norm(h, w["model.norm.weight"], cfg.get("rms_norm_eps", 1e-5)))
    head = w.get("lm_head.weight", w["model.embed_tokens.weight"])
    return y @ head.T


# ---------------------------------------------------------------- sampling


def argmax_lowest(logits):
    """Greedy pick; equal maxima resolve to the lowest index (sampling.cu:118-119,145)."""
    best, best_i = -math.inf, 0
    for i, x in enumerate(logits.tolist()):
        if x > best:
            best, best_i = x, i
    return best_i


def sample(logits, temperature=0.0, top_k=0, top_p=1.0, min_p=0.0, u=0.0):
    """temperature -> top-k -> top-p -> min-p -> draw with a given uniform u
    (crates/aegisllm-base/src/executor/generation.rs:193-273; device twin
    sampling.cu:275-375, which receives u from the host). Returns the token and
    the walk [(index, weight)] that the draw went over."""
    f32 = torch.float32
    logits = logits.to(f32)
    if temperature <= 0.0 or top_k == 1:
        return argmax_lowest(logits), []
    temp = max(float(temperature), 1e-6)
    cand = [(i, x) for i, x in enumerate(logits.tolist()) if math.isfinite(x)]
    if not cand:
        return argmax_lowest(logits), []
    cand.sort(key=lambda c: -c[1])  # stable: equal values keep index order
    if 0 < top_k < len(cand):
        cand = cand[:top_k]
    mx = cand[0][1]
    vals = torch.tensor([c[1] for c in cand], dtype=f32)
    wts = torch.exp((vals - torch.tensor(mx, dtype=f32)) / torch.tensor(temp, dtype=f32))
    weighted = [(c[0], float(x)) for c, x in zip(cand, wts.tolist()) if math.isfinite(x) and x > 0.0]
    if not weighted:
        return argmax_lowest(logits), []
    total = float(torch.tensor([x for _, x in weighted], dtype=f32).sum())
    if 0.0 < top_p < 1.0 and total > 0.0:
        cutoff = total * top_p
        cum, keep = 0.0, 0
        for _, x in weighted:
            cum += x
            keep += 1
            if cum >= cutoff:
                break
        weighted = weighted[: max(keep, 1)]
    if min_p > 0.0:
        cutoff = weighted[0][1] * min_p
        weighted = [(i, x) for i, x in weighted if x >= cutoff]
        if not weighted:
            return argmax_lowest(logits), []
    total = sum(x for _, x in weighted)
    if total <= 0.0:
        return argmax_lowest(logits), weighted
    draw = u * total
    for i, x in weighted:
        if draw <= x:
            return i, weighted
        draw -= x
    return argmax_lowest(logits), weighted


# ---------------------------------------------------------------- generation


def generate_greedy(cfg, w, prompt, max_tokens, eos=(), stop=()):
    """One request, recomputing the whole sequence for every token. Order of the
    checks per produced token: EOS ends without the token, a stop token is kept
    and ends, and no forward runs after the last allowed token
    (crates/aegisllm-base/src/executor/generation.rs:64-78)."""
    seq = list(prompt)
    out = []
    reason = "length"
    nxt = argmax_lowest(forward_logits(cfg, w, seq)[-1])
    for _ in range(max_tokens):
        if nxt in eos:
            reason = "eos_token"
            break
        if nxt in stop:
            out.append(nxt)
            reason = "stop"
            break
        out.append(nxt)
        seq.append(nxt)
        if len(out) < max_tokens:
            nxt = argmax_lowest(forward_logits(cfg, w, seq)[-1])
    return out, reason
