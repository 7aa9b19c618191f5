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
    """Bound on |engine - plain float32| for logits. float32: float32 rounding over a few
    hundred terms (worst seen on a B200: 6e-6 of the logits' scale). bfloat16: what rounding
    the activations to 8 bits of mantissa at nine places a layer does to a tiny model's
    logits; the worst seen is 1.0e-2 of the scale, and the plain implementation with the same
    roundings alone differs from the plain float32 one by up to 0.8e-2 on these models."""
    scale = max(1.0, float(ref.abs().max()))
    return 2e-5 * scale if dtype == "float32" else 2e-2 * scale


# |engine bfloat16 - plain implementation with the same roundings|, as a fraction of the
# logits' scale (max |logit|, at least 1); worst seen 1.0e-2. It is not far below the bound
# above: at widths of 64 to 128 a single 16-bit rounding that falls the other way (because
# a float32 sum was taken in another order) moves every output of the next product enough to
# turn some of ITS roundings, so the two computations drift apart as two roundings of the
# same numbers would. Stage by stage (tests of the parts and kernels) they agree to a few
# units in the last place of bfloat16.
BF16_VS_ROUNDED = 1.5e-2

_observed = {}


def record_error(kind, dtype, err, scale, what=""):
    model = what.split(" ")[0] if what.split(" ")[0] in TINY else "-"
    k = (f"{kind} [{model}]", dtype)
    worst = _observed.get(k, (0.0, 1.0, 0))
    _observed[k] = (max(worst[0], err / scale), scale if err / scale > worst[0] else worst[1], worst[2] + 1)


def pytest_terminal_summary(terminalreporter):
    if not _observed:
        return
    terminalreporter.write_line("worst observed |engine - plain| / max(1, max|logit|):")
    for (kind, dtype), (rel, scale, n) in sorted(_observed.items()):
        terminalreporter.write_line(f"  {dtype:9s} {kind:34s} {rel:.3e}  (scale {scale:.2f}, {n} comparisons)")
    path = os.environ.get("LUMEN_TEST_ERRORS")
    if path:
        import json
        with open(path, "w") as f:
            json.dump({f"{d}:{k}": v[0] for (k, d), v in _observed.items()}, f, indent=1)


class Ref:
    """Plain logits of a sequence twice: all float32, and with activations rounded to
    bfloat16 where the serving path rounds them. Indexing takes the same rows of both."""

    def __init__(self, f32, b16):
        self.f32, self.b16 = f32, b16

    def __getitem__(self, idx):
        return Ref(self.f32[idx], self.b16[idx])

    @property
    def shape(self):
        return self.f32.shape

    @staticmethod
    def cat(refs):
        return Ref(torch.cat([r.f32 for r in refs]), torch.cat([r.b16 for r in refs]))

    @staticmethod
    def stack(refs):
        return Ref(torch.stack([r.f32 for r in refs]), torch.stack([r.b16 for r in refs]))


def plain_ref(cfg, w, tokens, **kw):
    import plain_qwen3 as P
    return Ref(P.forward_logits(cfg, w, tokens, **kw),
               P.forward_logits(cfg, w, tokens, round_to=torch.bfloat16, **kw))


def check(got, ref, dtype, what):
    """Engine logits against the plain implementation: float32 against the float32 plain
    logits; bfloat16 against those (wide bound) and, tightly, against the plain logits made
    with the same roundings."""
    r32 = ref.f32 if isinstance(ref, Ref) else ref
    assert got.shape == r32.shape, what
    assert torch.isfinite(got).all(), what

    def one(r, tol, kind):
        scale = max(1.0, float(r.abs().max()))
        err = float((got - r).abs().max())
        record_error(kind, dtype, err, scale, what)
        if err > tol * scale:
            bad = int((got - r).abs().max(dim=1).values.argmax())
            raise AssertionError(f"{what}: max abs error {err:.3e} > {tol * scale:.3e} ({kind}); "
                                 f"worst position {bad} of {got.shape[0]}")
    if dtype == "float32":
        one(r32, 2e-5, "vs plain float32")
    else:
        one(r32, 2e-2, "vs plain float32")
        if isinstance(ref, Ref):
            one(ref.b16, BF16_VS_ROUNDED, "vs plain with bf16 roundings")
