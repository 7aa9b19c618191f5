"""Typed configuration of Qwen3 dense (`Qwen3ForCausalLM`, model_type "qwen3").

Every size and constant comes from config.json; defaults for absent keys are the
reference's: num_key_value_heads = num_attention_heads
(crates/aegisllm-base/src/graph.rs:356-358), head_dim = hidden_size / heads
(crates/aegisllm-base/src/artifact.rs:560-564), rope_theta = 10000
(crates/aegisllm-base/src/model/llama.rs:49), rms_norm_eps = 1e-5
(crates/aegisllm-cuda/src/executor/full.rs:672). Keys that would change the
arithmetic in a way this library does not compute are refused, never ignored.
"""
from __future__ import annotations

from dataclasses import dataclass, field
from typing import Any, Dict, Optional, Tuple

from .registry import eos_ids_of, register_architecture
from .spec import ConfigError, LayerSpec, ModelSpec, PartSpec, ScheduleEntry

_REQUIRED = ("hidden_size", "num_hidden_layers", "num_attention_heads", "vocab_size",
             "intermediate_size")


def _pos_int(d, key, default=None):
    v = d.get(key, default)
    if v is None:
        raise ConfigError(f"config.json: missing key '{key}'")
    if isinstance(v, bool) or not isinstance(v, int) or v <= 0:
        raise ConfigError(f"config.json: '{key}' must be a positive integer, got {v!r}")
    return v


def _number(d, key, default):
    v = d.get(key, default)
    if isinstance(v, bool) or not isinstance(v, (int, float)):
        raise ConfigError(f"config.json: '{key}' must be a number, got {v!r}")
    return float(v)


@register_architecture("Qwen3ForCausalLM", model_type="qwen3")
@dataclass(frozen=True)
class Qwen3Config:
    vocab_size: int
    hidden_size: int
    intermediate_size: int
    num_hidden_layers: int
    num_attention_heads: int
    num_key_value_heads: int
    head_dim: int
    max_position_embeddings: int
    rope_theta: float
    rms_norm_eps: float
    tie_word_embeddings: bool = False
    attention_bias: bool = False
    hidden_act: str = "silu"
    use_sliding_window: bool = False
    sliding_window: Optional[int] = None
    max_window_layers: int = 0
    layer_types: Optional[Tuple[str, ...]] = None
    torch_dtype: str = "bfloat16"
    eos_token_ids: Tuple[int, ...] = ()
    architectures: Tuple[str, ...] = ("Qwen3ForCausalLM",)
    model_type: str = "qwen3"
    extra: Dict[str, Any] = field(default_factory=dict, compare=False)

    # ------------------------------------------------------------ parsing
    @classmethod
    def from_dict(cls, d: dict) -> "Qwen3Config":
        for k in _REQUIRED:
            if k not in d:
                raise ConfigError(f"config.json: missing key '{k}'")
        H = _pos_int(d, "hidden_size")
        nq = _pos_int(d, "num_attention_heads")
        nkv = _pos_int(d, "num_key_value_heads", nq)
        if d.get("head_dim") is None:
            if H % nq:
                raise ConfigError(f"config.json: no 'head_dim', and hidden_size {H} is not a "
                                  f"multiple of num_attention_heads {nq}")
            hd = H // nq
        else:
            hd = _pos_int(d, "head_dim")
        if nq % nkv:
            raise ConfigError(f"config.json: num_attention_heads {nq} is not a multiple of "
                              f"num_key_value_heads {nkv}")
        if hd % 2:
            raise ConfigError(f"config.json: head_dim {hd} must be even for rotary pairs")
        if d.get("attention_bias", False):
            raise ConfigError("config.json: attention_bias=true is not supported (the projections "
                              "of this architecture carry no bias here)")
        act = d.get("hidden_act", d.get("hidden_activation", "silu"))
        if act not in ("silu", "swiglu"):
            raise ConfigError(f"config.json: hidden_act {act!r} is not supported (silu only)")
        scaling = d.get("rope_scaling")
        if scaling is None and isinstance(d.get("rope_parameters"), dict):
            rp = d["rope_parameters"]
            if rp.get("rope_type", "default") not in ("default", None):
                scaling = rp
        if scaling is not None and scaling.get("rope_type", scaling.get("type", "default")) != "default":
            raise ConfigError(f"config.json: rope_scaling {scaling!r} is not supported")
        theta = d.get("rope_theta")
        if theta is None and isinstance(d.get("rope_parameters"), dict):
            theta = d["rope_parameters"].get("rope_theta")  # hoisted as artifact.rs:703-829 does
        theta = _number({"rope_theta": 10000.0 if theta is None else theta}, "rope_theta", 10000.0)
        if theta <= 0:
            raise ConfigError("config.json: rope_theta must be positive")
        eps = _number(d, "rms_norm_eps", 1e-5)
        if eps < 0:
            raise ConfigError("config.json: rms_norm_eps must not be negative")
        L = _pos_int(d, "num_hidden_layers")
        use_win = bool(d.get("use_sliding_window", False))
        win = d.get("sliding_window")
        lt = d.get("layer_types")
        if lt is not None:
            if len(lt) != L or any(t not in ("full_attention", "sliding_attention") for t in lt):
                raise ConfigError("config.json: layer_types must name 'full_attention' or "
                                  f"'sliding_attention' for each of the {L} layers")
            lt = tuple(lt)
        needs_win = use_win or (lt is not None and "sliding_attention" in lt)
        if needs_win:
            if isinstance(win, bool) or not isinstance(win, int) or win <= 0:
                raise ConfigError("config.json: a sliding window is switched on but "
                                  f"'sliding_window' is {win!r}")
            if lt is None and d.get("max_window_layers") is None:
                # which layers get the window is the file's to say; the reference ignores
                # windows for this family (crates/aegisllm-base/src/model/qwen3.rs:55-61),
                # so there is no default of its own to take
                raise ConfigError("config.json: use_sliding_window is on, but neither "
                                  "'layer_types' nor 'max_window_layers' says which layers "
                                  "have the window")
        eos_ids: Tuple[int, ...] = eos_ids_of(d.get("eos_token_id"), "config.json")
        dtype = d.get("torch_dtype", d.get("dtype", "bfloat16"))
        known = set(cls.__dataclass_fields__) | {"eos_token_id", "dtype", "hidden_activation",
                                                  "rope_scaling", "rope_parameters"}
        return cls(
            vocab_size=_pos_int(d, "vocab_size"), hidden_size=H,
            intermediate_size=_pos_int(d, "intermediate_size"), num_hidden_layers=L,
            num_attention_heads=nq, num_key_value_heads=nkv, head_dim=hd,
            max_position_embeddings=_pos_int(d, "max_position_embeddings", 32768),
            rope_theta=theta, rms_norm_eps=eps,
            tie_word_embeddings=bool(d.get("tie_word_embeddings", False)),
            attention_bias=False, hidden_act="silu", use_sliding_window=use_win,
            sliding_window=win if needs_win else (win if isinstance(win, int) else None),
            max_window_layers=int(d.get("max_window_layers", 0) or 0), layer_types=lt,
            torch_dtype=str(dtype), eos_token_ids=eos_ids,
            architectures=tuple(d.get("architectures") or ("Qwen3ForCausalLM",)),
            model_type=str(d.get("model_type", "qwen3")),
            extra={k: v for k, v in d.items() if k not in known},
        )

    def to_dict(self) -> dict:
        d = {
            "architectures": list(self.architectures), "model_type": self.model_type,
            "vocab_size": self.vocab_size, "hidden_size": self.hidden_size,
            "intermediate_size": self.intermediate_size,
            "num_hidden_layers": self.num_hidden_layers,
            "num_attention_heads": self.num_attention_heads,
            "num_key_value_heads": self.num_key_value_heads, "head_dim": self.head_dim,
            "max_position_embeddings": self.max_position_embeddings,
            "rope_theta": self.rope_theta, "rope_scaling": None,
            "rms_norm_eps": self.rms_norm_eps, "hidden_act": self.hidden_act,
            "tie_word_embeddings": self.tie_word_embeddings,
            "attention_bias": self.attention_bias,
            "use_sliding_window": self.use_sliding_window, "sliding_window": self.sliding_window,
            "max_window_layers": self.max_window_layers, "torch_dtype": self.torch_dtype,
        }
        if self.layer_types is not None:
            d["layer_types"] = list(self.layer_types)
        if self.eos_token_ids:
            d["eos_token_id"] = list(self.eos_token_ids) if len(self.eos_token_ids) > 1 \
                else self.eos_token_ids[0]
        return d

    # ------------------------------------------------------------ meaning
    def window_of_layer(self, i: int) -> int:
        """0 = all keys. With `layer_types` the list decides; else
        `use_sliding_window` gives layers from `max_window_layers` on a window of
        `sliding_window` keys (the query's own position included)."""
        if self.layer_types is not None:
            return int(self.sliding_window) if self.layer_types[i] == "sliding_attention" else 0
        if self.use_sliding_window and self.sliding_window and i >= self.max_window_layers:
            return int(self.sliding_window)
        return 0

    def model_spec(self) -> ModelSpec:
        """The layer formulas, in order, are those of the reference's dense decoder
        (crates/aegisllm-cuda/src/executor/attention.rs:139-202,241-250,341-352,413-425;
        executor/mlp.rs:271-356) with the Gemma-only steps (weightless V norm,
        q*sqrt(d): attention.rs:203-219,262-269) and the Qwen3-Next-only ones
        ((1+w) norm weights, output gate, partial rotary: loader.rs:189-194,212-215)
        switched off by parameters."""
        H = self.hidden_size
        layers = []
        for i in range(self.num_hidden_layers):
            p = f"model.layers.{i}"
            position = PartSpec("rotary", {"head_dim": self.head_dim, "theta": self.rope_theta,
                                           "rotary_dim": self.head_dim})
            mixer = PartSpec("gqa_attention", {
                "hidden_size": H, "num_heads": self.num_attention_heads,
                "num_kv_heads": self.num_key_value_heads, "head_dim": self.head_dim,
                "qk_norm": True, "qk_norm_eps": self.rms_norm_eps, "qk_norm_weight_offset": 0.0,
                "softmax_scale": float(self.head_dim) ** -0.5,
                "window": self.window_of_layer(i), "position": position,
            }, prefix=f"{p}.self_attn")
            ffn = PartSpec("swiglu", {"hidden_size": H, "intermediate_size": self.intermediate_size},
                           prefix=f"{p}.mlp")
            norm = lambda name: PartSpec("rmsnorm", {"size": H, "eps": self.rms_norm_eps,
                                                     "weight_offset": 0.0}, prefix=f"{p}.{name}")
            layers.append(LayerSpec("pre_norm", mixer, ffn,
                                    {"mixer": norm("input_layernorm"),
                                     "ffn": norm("post_attention_layernorm")}, prefix=p))
        spec = ModelSpec(
            architecture="Qwen3ForCausalLM", vocab_size=self.vocab_size, hidden_size=H,
            max_positions=self.max_position_embeddings,
            embedding=PartSpec("token_embedding", {"vocab_size": self.vocab_size, "hidden_size": H,
                                                   "scale": None}, prefix="model.embed_tokens"),
            layers=tuple(layers),
            schedule=tuple(ScheduleEntry(i) for i in range(self.num_hidden_layers)),
            final_norm=PartSpec("rmsnorm", {"size": H, "eps": self.rms_norm_eps,
                                            "weight_offset": 0.0}, prefix="model.norm"),
            head=PartSpec("linear_head", {"vocab_size": self.vocab_size, "hidden_size": H,
                                          "tied_to": "model.embed_tokens.weight"
                                          if self.tie_word_embeddings else None,
                                          "falls_back_to": "model.embed_tokens.weight"},
                          prefix="lm_head"),
            eos_token_ids=self.eos_token_ids,
        )
        spec.validate()
        return spec
