import os
import sys
from pathlib import Path

import pytest
import torch

ROOT = Path(__file__).resolve().parent.parent
sys.path.insert(0, str(ROOT))
sys.path.insert(0, str(ROOT / "tests"))


def pytest_configure(config):
    config.addinivalue_line("markers", "gpu: needs a CUDA device (NVIDIA B200)")


def pytest_collection_modifyitems(config, items):
    if torch.cuda.is_available():
        return
    skip = pytest.mark.skip(reason="no CUDA device")
    for item in items:
        if "gpu" in item.keywords:
            item.add_marker(skip)


# Tiny configurations of the architecture that differ in every size and option:
# layers, width, heads, groups (ratio 2 / 4 / 1), head size (16 / 32 / 48, so heads x size is
# equal to, larger than and different from the width), feed-forward width, vocabulary (a power
# of two, a multiple of 128, a prime), theta, eps, tied or untied head, and window (none, none,
# 24 keys on the layers from index 1 on). D and E have the head sizes (64, 128) that the
# tensor-core attention kernels take, with groups of 2 and 4 and, for D, a window of 40 keys on
# its second layer, so that the engine's tests run through those kernels too.
TINY = {
    "A": dict(architectures=["Qwen3ForCausalLM"], model_type="qwen3", hidden_size=64,
              num_hidden_layers=2, num_attention_heads=4, num_key_value_heads=2, head_dim=16,
              intermediate_size=128, vocab_size=256, rope_theta=10000.0, rms_norm_eps=1e-6,
              max_position_embeddings=1024, tie_word_embeddings=True, attention_bias=False,
              use_sliding_window=False, hidden_act="silu"),
    "B": dict(architectures=["Qwen3ForCausalLM"], model_type="qwen3", hidden_size=96,
              num_hidden_layers=3, num_attention_heads=8, num_key_value_heads=2, head_dim=32,
              intermediate_size=224, vocab_size=384, rope_theta=1000000.0, rms_norm_eps=1e-5,
              max_position_embeddings=2048, tie_word_embeddings=False, attention_bias=False,
              use_sliding_window=False, hidden_act="silu"),
    "C": dict(architectures=["Qwen3ForCausalLM"], model_type="qwen3", hidden_size=80,
              num_hidden_layers=4, num_attention_heads=5, num_key_value_heads=5, head_dim=48,
              intermediate_size=176, vocab_size=311, rope_theta=50000.0, rms_norm_eps=3e-6,
              max_position_embeddings=1536, tie_word_embeddings=False, attention_bias=False,
              use_sliding_window=True, sliding_window=24, max_window_layers=1, hidden_act="silu"),
    "D": dict(architectures=["Qwen3ForCausalLM"], model_type="qwen3", hidden_size=128,
              num_hidden_layers=2, num_attention_heads=4, num_key_value_heads=2, head_dim=64,
              intermediate_size=192, vocab_size=500, rope_theta=100000.0, rms_norm_eps=1e-6,
              max_position_embeddings=1024, tie_word_embeddings=False, attention_bias=False,
              use_sliding_window=True, sliding_window=40, max_window_layers=1, hidden_act="silu"),
    "E": dict(architectures=["Qwen3ForCausalLM"], model_type="qwen3", hidden_size=128,
              num_hidden_layers=2, num_attention_heads=4, num_key_value_heads=1, head_dim=128,
              intermediate_size=160, vocab_size=272, rope_theta=1000000.0, rms_norm_eps=1e-5,
              max_position_embeddings=1024, tie_word_embeddings=True, attention_bias=False,
              use_sliding_window=False, hidden_act="silu"),
}


@pytest.fixture(scope="session")
def tiny_models(tmp_path_factory):
    """name -> folder of a random-weights model (bfloat16 tensors, seeded)."""
    from lumenllm_b200.config import config_from_dict
    from lumenllm_b200.weights import write_random_model
    out = {}
    for i, (name, cfg) in enumerate(TINY.items()):
        d = tmp_path_factory.mktemp(f"tiny{name}")
        write_random_model(config_from_dict(cfg), d, seed=11 + i, std=0.05, norm_jitter=0.1)
        out[name] = d
    return out


def seeded_tokens(vocab, lengths, seed):
    g = torch.Generator().manual_seed(seed)
    return [torch.randint(0, vocab, (n,), generator=g).tolist() for n in lengths]


def tolerance(dtype, ref):
    """float32: float32 rounding over a few hundred terms. bfloat16: activations are
    rounded to 8 bits of mantissa about six times a layer; the bound is 3 % of the
    logits' scale."""
    scale = max(1.0, float(ref.abs().max()))
    return 2e-5 * scale if dtype == "float32" else 3e-2 * scale
