"""The Python entry point, named after the reference's Rust one
(`AegisEngine::build(EngineConfig)`, `.generate(GenerateRequest) -> GenerateOutput`,
`.generate_timed`: crates/aegisllm/src/engine.rs:78-193).

    from lumenllm_b200 import EngineConfig, GenerateRequest, SamplingConfig, build
    engine = build(EngineConfig(model_path="/models/x"))
    out = engine.generate(GenerateRequest(prompt_tokens=[1, 2, 3], max_tokens=16))
"""
from __future__ import annotations

from dataclasses import dataclass, field
from typing import Optional

from ..config import ConfigError, ParametersFile, SamplingDefaults
from ..sampling import SamplingConfig
from .engine import Engine

DEFAULT_CTX_SIZE = 8192   # the reference's --ctx-size default (crates/aegisllm/src/cli/flags.rs:44)


@dataclass
class EngineConfig:
    model_path: Optional[str] = None        # folder with config.json and safetensors
    parameters: Optional[str] = None        # a parameters.json; explicit fields below override it
    random_config: Optional[dict] = None    # config.json keys of a random-weights model
    random_seed: int = 0
    dtype: Optional[str] = None             # "bfloat16" (default) or "float32"
    context_size: Optional[int] = None      # longest sequence
    max_tokens: Optional[int] = None        # tokens the cache holds; default context x batch
    max_batch: Optional[int] = None
    device: Optional[int] = None
    sampling: Optional[SamplingDefaults] = None
    strict_weights: bool = True             # False: stored tensors that no part reads are warned about


@dataclass
class BuiltEngine:
    engine: Engine
    sampling: SamplingDefaults
    max_batch: int

    def default_sampling(self, **override) -> SamplingConfig:
        s = self.sampling
        base = dict(temperature=s.temperature, top_k=s.top_k, top_p=s.top_p, min_p=s.min_p,
                    seed=s.seed)
        base.update({k: v for k, v in override.items() if v is not None})
        return SamplingConfig(**base)

    def generate(self, requests, **kw):
        kw.setdefault("max_batch", self.max_batch)
        return self.engine.generate(requests, **kw)

    def generate_timed(self, requests, **kw):
        """Same as generate; every GenerateOutput carries prefill_s and decode_s."""
        return self.generate(requests, **kw)

    def __getattr__(self, name):
        return getattr(self.engine, name)


def build(cfg: EngineConfig) -> BuiltEngine:
    pf = ParametersFile.from_path(cfg.parameters) if cfg.parameters else ParametersFile()
    model_path = cfg.model_path or pf.model_path
    random_config = cfg.random_config or (None if cfg.model_path else pf.random_config)
    if (model_path is None) == (random_config is None):
        raise ConfigError("engine command requires --model <path> or --config <path> "
                          "(exactly one of a model folder and a random-weights shape)")
    dtype = cfg.dtype or pf.dtype or "bfloat16"
    ctx = cfg.context_size or pf.context_size or DEFAULT_CTX_SIZE
    max_batch = cfg.max_batch or pf.batch_size or 8
    max_tokens = cfg.max_tokens or pf.max_tokens or ctx * max_batch
    device = cfg.device if cfg.device is not None else pf.device
    common = dict(dtype=dtype, max_tokens=max_tokens, device=device, context_size=ctx)
    if model_path is not None:
        eng = Engine.from_folder(model_path, strict_weights=cfg.strict_weights, **common)
    else:
        seed = cfg.random_seed if cfg.random_config else pf.random_seed
        eng = Engine.from_random(random_config, seed=seed, **common)
    return BuiltEngine(eng, cfg.sampling or pf.sampling, max_batch)
