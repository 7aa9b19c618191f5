"""The plain implementation checked against hand-computed values and against itself."""
import math

import pytest
import torch

import plain_qwen3 as P
from conftest import TINY, seeded_tokens


def test_rms_norm_by_hand():
    x = torch.tensor([[3.0, 4.0]])
    w = torch.tensor([2.0, 0.5])
    y = P.rms_norm(x, w, 0.0)
    s = 1.0 / math.sqrt((9 + 16) / 2)
    assert torch.allclose(y, torch.tensor([[3 * s * 2, 4 * s * 0.5]]), atol=1e-6)
    assert float(P.rms_norm(torch.zeros(1, 4), torch.ones(4), 1e-6).abs().max()) == 0.0


def test_rope_pairs_and_angles():
    d, theta = 8, 100.0
    x = torch.arange(1.0, 9.0).view(1, 1, 8)
    y = P.apply_rope(x, torch.tensor([3]), theta)[0, 0]
    for i in range(4):
        ang = 3.0 * theta ** (-2 * i / d)
        a, b = float(i + 1), float(i + 5)
        assert abs(float(y[i]) - (a * math.cos(ang) - b * math.sin(ang))) < 1e-5
        assert abs(float(y[i + 4]) - (a * math.sin(ang) + b * math.cos(ang))) < 1e-5
    assert torch.equal(P.apply_rope(x, torch.tensor([0]), theta), x)
    part = P.apply_rope(x, torch.tensor([3]), theta, rotary_dim=4)[0, 0]
    assert torch.equal(part[4:], x[0, 0, 4:])


def test_swiglu_by_hand():
    g, u = torch.tensor([0.0, 1.0, -2.0]), torch.tensor([3.0, 2.0, 1.0])
    z = P.swiglu(g, u)
    assert torch.allclose(z, torch.tensor([0.0, 2 / (1 + math.exp(-1)), -2 / (1 + math.exp(2))]), atol=1e-6)


def test_attention_single_head_by_hand_and_group_map():
    q = torch.tensor([[[1.0, 0.0]], [[0.0, 2.0]]])        # T=2, one head, d=2
    k = torch.tensor([[[1.0, 0.0]], [[0.0, 1.0]]])
    v = torch.tensor([[[1.0, 10.0]], [[2.0, 20.0]]])
    o = P.causal_attention(q, k, v)
    assert torch.allclose(o[0, 0], v[0, 0])                # first token sees itself only
    s = torch.tensor([0.0, 2.0]) / math.sqrt(2)
    p = torch.softmax(s, 0)
    assert torch.allclose(o[1, 0], p[0] * v[0, 0] + p[1] * v[1, 0], atol=1e-6)
    # heads 0,1 read kv head 0; heads 2,3 kv head 1
    T, nq, nkv, d = 5, 4, 2, 4
    g = torch.Generator().manual_seed(0)
    q = torch.randn(T, nq, d, generator=g); k = torch.randn(T, nkv, d, generator=g)
    v = torch.randn(T, nkv, d, generator=g)
    o = P.causal_attention(q, k, v)
    for h in range(nq):
        one = P.causal_attention(q[:, h:h + 1], k[:, h // 2:h // 2 + 1], v[:, h // 2:h // 2 + 1])
        assert torch.allclose(o[:, h], one[:, 0], atol=1e-6)


def test_window_edge():
    T, d, W = 12, 4, 3
    q = torch.zeros(T, 1, d); k = torch.zeros(T, 1, d)
    v = torch.arange(T, dtype=torch.float32).view(T, 1, 1).expand(T, 1, d).clone()
    o = P.causal_attention(q, k, v, window=W)             # uniform weights over the visible keys
    for t in range(T):
        vis = list(range(max(0, t - W + 1), t + 1))
        assert abs(float(o[t, 0, 0]) - sum(vis) / len(vis)) < 1e-6


def test_prompt_rows_equal_shorter_prompts(tiny_models):
    """Row i of a whole prompt equals the last row of its first i+1 tokens (the
    identity crates/aegisllm-cpu/src/attention.rs:295-346 tests for attention)."""
    for name in ("A", "C"):
        cfg, w = P.load_model(tiny_models[name])
        toks = seeded_tokens(cfg["vocab_size"], [40], 3)[0]
        full = P.forward_logits(cfg, w, toks)
        for i in (0, 5, 23, 24, 25, 39):
            part = P.forward_logits(cfg, w, toks[: i + 1])
            assert torch.allclose(full[i], part[-1], atol=2e-5), (name, i)


def test_window_changes_results_only_past_its_edge(tiny_models):
    cfg, w = P.load_model(tiny_models["C"])
    toks = seeded_tokens(cfg["vocab_size"], [40], 4)[0]
    with_w = P.forward_logits(cfg, w, toks)
    no_w = P.forward_logits(dict(cfg, use_sliding_window=False), w, toks)
    assert torch.allclose(with_w[:24], no_w[:24], atol=1e-6)
    assert float((with_w[24:] - no_w[24:]).abs().max()) > 1e-4


def test_tied_and_untied_head(tiny_models):
    cfgA, wA = P.load_model(tiny_models["A"])
    assert "lm_head.weight" not in wA
    cfgB, wB = P.load_model(tiny_models["B"])
    assert wB["lm_head.weight"].shape == (384, 96)


def test_sampler_by_hand():
    lg = torch.tensor([1.0, 3.0, 3.0, 2.0, -1e30, float("nan")])
    assert P.sample(lg)[0] == 1                              # greedy: lowest index of equal maxima
    assert P.sample(lg, temperature=1.0, top_k=1)[0] == 1
    # temperature 1: weights e^0, e^0, e^-1, e^-2 in order (1, 2, 3, 0)
    tok, walk = P.sample(lg, temperature=1.0, u=0.0)
    assert tok == 1 and [i for i, _ in walk] == [1, 2, 3, 0, 4][:len(walk)]
    total = 2 + math.exp(-1) + math.exp(-2)
    assert P.sample(lg, temperature=1.0, u=1.5 / total)[0] == 2
    assert P.sample(lg, temperature=1.0, u=2.2 / total)[0] == 3
    assert P.sample(lg, temperature=1.0, u=0.9999)[0] == 0
    assert P.sample(lg, temperature=1.0, top_k=2, u=0.9999)[0] == 2
    assert P.sample(lg, temperature=1.0, top_p=0.5, u=0.9999)[0] == 2     # prefix reaching half
    assert P.sample(lg, temperature=1.0, min_p=0.5, u=0.9999)[0] == 2     # e^-1 < 0.5
    assert P.sample(lg, temperature=0.5, min_p=0.1, u=0.9999)[0] == 3     # e^-2 >= 0.1 > e^-4


def test_generate_greedy_rules(tiny_models):
    cfg, w = P.load_model(tiny_models["A"])
    prompt = seeded_tokens(cfg["vocab_size"], [6], 5)[0]
    toks, reason = P.generate_greedy(cfg, w, prompt, 5)
    assert len(toks) == 5 and reason == "length"
    t2, r2 = P.generate_greedy(cfg, w, prompt, 5, eos=[toks[2]])
    assert t2 == toks[:toks.index(toks[2])] and r2 == "eos_token"
    t3, r3 = P.generate_greedy(cfg, w, prompt, 5, stop=[toks[1]])
    assert t3 == toks[:toks.index(toks[1]) + 1] and r3 == "stop"
