"""The run-parameters file, in the manner of the reference's `parameters.json`
(kebab-case keys, unknown keys refused: crates/aegisllm/src/params/file.rs:34-337).

    {"model": {"path": "/models/x",            # or "random": {"config": {...}, "seed": 0}
               "compute": "cuda:0", "store": "vram", "dtype": "bfloat16",
               "hidden-layers": {"kv-cache": {"context-size": 4096, "max-tokens": 65536,
                                              "type-k": "bf16", "type-v": "bf16"}},
               "other-parameters": {"temperature": 0.7, "top-p": 0.95, "top-k": 50,
                                    "min-p": 0.05, "seed": 1, "batch-size": 8}},
     "cuda": {"device": 0}}

Only what a single-GPU library computes is accepted: `compute` must name a CUDA
device, `store` must be "vram", cache types must equal the run dtype.
"""
from __future__ import annotations

import json
import re
from dataclasses import dataclass
from pathlib import Path
from typing import Optional

from .spec import ConfigError


@dataclass(frozen=True)
class SamplingDefaults:
    """Defaults 0 / 0 / 1.0 / 0.0 as crates/aegisllm-base/src/generation.rs:166-175."""
    temperature: float = 0.0
    top_k: int = 0
    top_p: float = 1.0
    min_p: float = 0.0
    seed: Optional[int] = None


def _only(d, allowed, where):
    if not isinstance(d, dict):
        raise ConfigError(f"parameters: '{where}' must be an object")
    extra = sorted(set(d) - set(allowed))
    if extra:
        raise ConfigError(f"parameters: unknown key(s) {extra} in '{where}' "
                          f"(allowed: {sorted(allowed)})")


def _strip_comments(text: str) -> str:
    # .jsonc files of the reference carry // comments
    return re.sub(r"(^|\s)//[^\n]*", r"\1", text)


@dataclass(frozen=True)
class ParametersFile:
    model_path: Optional[str] = None
    random_config: Optional[dict] = None
    random_seed: int = 0
    dtype: Optional[str] = None
    device: int = 0
    context_size: Optional[int] = None
    max_tokens: Optional[int] = None
    batch_size: Optional[int] = None
    sampling: SamplingDefaults = SamplingDefaults()

    @classmethod
    def from_path(cls, path) -> "ParametersFile":
        p = Path(path)
        if not p.exists():
            raise ConfigError(f"missing file: {p}")
        try:
            d = json.loads(_strip_comments(p.read_text()))
        except json.JSONDecodeError as e:
            raise ConfigError(f"{p}: not valid JSON ({e})") from e
        return cls.from_dict(d, base=p.parent)

    @classmethod
    def from_dict(cls, d: dict, base: Path | None = None) -> "ParametersFile":
        _only(d, {"model", "cuda"}, "<top level>")
        if "model" not in d:
            raise ConfigError("parameters: missing section 'model'")
        m = d["model"]
        _only(m, {"path", "random", "compute", "store", "dtype", "hidden-layers",
                  "other-parameters"}, "model")
        if ("path" in m) == ("random" in m):
            raise ConfigError("parameters: 'model' needs exactly one of 'path' and 'random'")
        device = 0
        cuda = d.get("cuda", {})
        _only(cuda, {"device"}, "cuda")
        if "device" in cuda:
            device = int(cuda["device"])
        compute = m.get("compute")
        if compute is not None:
            mt = re.fullmatch(r"cuda(?::(\d+))?", str(compute))
            if not mt:
                raise ConfigError(f"parameters: model.compute={compute!r}: only a CUDA device "
                                  "computes here (cuda or cuda:N)")
            if mt.group(1) is not None:
                device = int(mt.group(1))
        if m.get("store", "vram") != "vram":
            raise ConfigError(f"parameters: model.store={m['store']!r}: weights live in GPU "
                              "memory only ('vram')")
        dtype = m.get("dtype")
        if dtype is not None and dtype not in ("bfloat16", "float32"):
            raise ConfigError(f"parameters: model.dtype={dtype!r}: bfloat16 or float32")
        model_path, rnd_cfg, seed = None, None, 0
        if "path" in m:
            model_path = str(m["path"])
            if base is not None and not Path(model_path).is_absolute():
                model_path = str((base / model_path))
        else:
            r = m["random"]
            _only(r, {"config", "seed"}, "model.random")
            cfg = r.get("config")
            if isinstance(cfg, str):
                cp = Path(cfg)
                if base is not None and not cp.is_absolute():
                    cp = base / cp
                cfg = json.loads(cp.read_text())
            if not isinstance(cfg, dict):
                raise ConfigError("parameters: model.random.config must be an object or a path")
            rnd_cfg, seed = cfg, int(r.get("seed", 0))
        ctx = mx = None
        hl = m.get("hidden-layers", {})
        _only(hl, {"kv-cache", "compute", "store"}, "model.hidden-layers")
        kv = hl.get("kv-cache", {})
        _only(kv, {"context-size", "max-tokens", "store", "type-k", "type-v"},
              "model.hidden-layers.kv-cache")
        if "context-size" in kv:
            ctx = int(kv["context-size"])
            if ctx <= 0:
                raise ConfigError("parameters: kv-cache.context-size must be positive")
        if "max-tokens" in kv:
            mx = int(kv["max-tokens"])
            if mx <= 0:
                raise ConfigError("parameters: kv-cache.max-tokens must be positive")
        for key in ("type-k", "type-v"):
            if key in kv and kv[key] not in ("bf16", "bfloat16", "f32", "float32"):
                raise ConfigError(f"parameters: kv-cache.{key}={kv[key]!r}: the cache is kept "
                                  "in the run dtype (bf16 or f32); quantized caches are not built")
        o = m.get("other-parameters", {})
        _only(o, {"temperature", "top-p", "top-k", "min-p", "seed", "batch-size"},
              "model.other-parameters")
        sampling = SamplingDefaults(
            temperature=float(o.get("temperature", 0.0)), top_k=int(o.get("top-k", 0)),
            top_p=float(o.get("top-p", 1.0)), min_p=float(o.get("min-p", 0.0)),
            seed=None if o.get("seed") is None else int(o["seed"]))
        bs = o.get("batch-size")
        return cls(model_path=model_path, random_config=rnd_cfg, random_seed=seed, dtype=dtype,
                   device=device, context_size=ctx, max_tokens=mx,
                   batch_size=None if bs is None else int(bs), sampling=sampling)
