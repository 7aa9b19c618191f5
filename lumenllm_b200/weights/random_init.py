"""Random-weights mode: from a configuration and a seed, either a model folder
(config.json + model.safetensors, read back by the by-name loader like any
checkpoint) or tensors made directly on the device for large shapes.

A tensor's values depend on (seed, tensor name) only, not on the order in which
tensors are made. Matrices are N(0, std); norm weights are 1 + U(-jitter, jitter)
(jitter 0 gives exactly 1). The reference has no such mode.
"""
from __future__ import annotations

import hashlib
import json
from pathlib import Path
from typing import Dict, Tuple

import torch

from .safetensors_io import write_file


def _seed_for(seed: int, name: str) -> int:
    h = hashlib.sha256(f"{seed}:{name}".encode()).digest()
    return int.from_bytes(h[:8], "little") & 0x7FFFFFFFFFFFFFFF


def random_tensor(name: str, shape, kind: str, seed: int, std: float, norm_jitter: float,
                  dtype, device="cpu") -> torch.Tensor:
    g = torch.Generator(device=device)
    g.manual_seed(_seed_for(seed, name))
    if kind == "norm":
        t = torch.rand(shape, generator=g, device=device, dtype=torch.float32)
        t = 1.0 + (t * 2.0 - 1.0) * norm_jitter
    else:
        t = torch.randn(shape, generator=g, device=device, dtype=torch.float32) * std
    return t.to(dtype)


def random_weights(expected: Dict[str, Tuple[Tuple[int, ...], str]], seed: int, std=0.02,
                   norm_jitter=0.0, dtype=torch.bfloat16, device="cpu") -> Dict[str, torch.Tensor]:
    """expected: name -> (shape, kind) with kind "matrix" or "norm"; "optional" tensors are
    not made."""
    return {n: random_tensor(n, shape, kind, seed, std, norm_jitter, dtype, device)
            for n, (shape, kind) in expected.items() if kind != "optional"}


def write_random_model(config, folder, seed: int = 0, std: float = 0.02, norm_jitter: float = 0.0,
                       dtype: str = "bfloat16") -> Path:
    """`config` is a configuration object (or a dict of config.json keys)."""
    from ..config import config_from_dict
    from ..engine.model import expected_tensors
    if isinstance(config, dict):
        config = config_from_dict(config)
    tdt = {"bfloat16": torch.bfloat16, "float32": torch.float32}[dtype]
    folder = Path(folder)
    folder.mkdir(parents=True, exist_ok=True)
    exp = expected_tensors(config.model_spec())
    tensors = random_weights(exp, seed, std, norm_jitter, tdt)
    d = config.to_dict()
    d["torch_dtype"] = dtype
    (folder / "config.json").write_text(json.dumps(d, indent=1))
    write_file(folder / "model.safetensors", tensors,
               metadata={"format": "pt", "seed": seed, "std": std, "norm_jitter": norm_jitter})
    return folder
