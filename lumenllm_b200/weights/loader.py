"""Weights by tensor name.

`open_checkpoint(folder)` indexes `model.safetensors` (or the shards named by
`model.safetensors.index.json`: crates/aegisllm-base/src/artifact.rs:567-645).
`load_weights` compares the names and shapes the model expects with what the
files hold and raises ONE WeightError that lists every missing tensor, every
unexpected tensor and every wrong shape; then it copies the tensors to the
device. bfloat16 stays bfloat16, a tensor stored in 32-bit float stays so,
float16 is widened to float32 (exact), integer tables become int32.

Three things soften the comparison, each named by the caller. `optional` tensors
are loaded when stored and not missed when absent. `fallbacks` {name: other}
let a missing tensor stand for another one that is stored: the reference takes
the output head from `lm_head.weight` when the file has it and from the
embedding when not, whatever config.json says
(crates/aegisllm-cuda/src/executor/full.rs:171-181). Names in IGNORED_SUFFIXES
(tables that older exporters store and no model reads) are never unexpected.
With strict=False other unexpected tensors are reported in the result's
`unexpected` list instead of raising.
"""
from __future__ import annotations

import json
from pathlib import Path
from typing import Dict, Tuple

import torch

from .safetensors_io import MappedFile, SafetensorsError, TensorInfo, read_header


class WeightError(ValueError):
    def __init__(self, message, missing=(), unexpected=(), wrong_shape=(), wrong_dtype=()):
        super().__init__(message)
        self.missing = list(missing)
        self.unexpected = list(unexpected)
        self.wrong_shape = list(wrong_shape)
        self.wrong_dtype = list(wrong_dtype)


def open_checkpoint(folder) -> Dict[str, TensorInfo]:
    folder = Path(folder)
    index = folder / "model.safetensors.index.json"
    single = folder / "model.safetensors"
    try:
        if index.exists():
            wm = json.loads(index.read_text()).get("weight_map", {})
            infos: Dict[str, TensorInfo] = {}
            headers = {}
            for name, shard in wm.items():
                if shard not in headers:
                    sp = folder / shard
                    if not sp.exists():
                        raise WeightError(f"missing file: {sp} (named by {index.name})")
                    headers[shard] = read_header(sp)
                if name not in headers[shard]:
                    raise WeightError(f"{index.name} places '{name}' in {shard}, "
                                      "which does not hold it")
                infos[name] = headers[shard][name]
            return infos
        if single.exists():
            return read_header(single)
    except SafetensorsError as e:
        raise WeightError(str(e)) from e
    raise WeightError(f"missing file: {single} (and no model.safetensors.index.json)")


def _kept_dtype(stored: str):
    if stored == "BF16":
        return torch.bfloat16
    if stored in ("F32", "F16"):
        return torch.float32
    if stored in ("I64", "I32", "I16", "I8", "U8"):
        return torch.int32
    return None


IGNORED_SUFFIXES = ("rotary_emb.inv_freq",)


class LoadedWeights(dict):
    """name -> tensor, with what the comparison let pass: `unexpected` (stored, read by
    nobody; only with strict=False) and `stood_in` {missing name: the stored tensor used}."""
    unexpected: list = []
    stood_in: dict = {}


def check_against(expected: Dict[str, Tuple[int, ...]], infos: Dict[str, TensorInfo],
                  where: str = "checkpoint", optional=(), fallbacks=None, strict: bool = True):
    """Raises the one WeightError, or returns (unexpected names, {missing: stand-in})."""
    optional, fallbacks = set(optional), dict(fallbacks or {})
    stood_in = {n: fallbacks[n] for n in expected
                if n not in infos and n in fallbacks and fallbacks[n] in infos
                and tuple(infos[fallbacks[n]].shape) == tuple(expected[n])}
    missing = sorted(n for n in expected if n not in infos and n not in optional
                     and n not in stood_in)
    unexpected = sorted(n for n in infos if n not in expected and not n.endswith(IGNORED_SUFFIXES))
    wrong = [(n, tuple(expected[n]), infos[n].shape) for n in sorted(expected)
             if n in infos and tuple(infos[n].shape) != tuple(expected[n])]
    bad_dtype = [(n, infos[n].dtype) for n in sorted(expected)
                 if n in infos and _kept_dtype(infos[n].dtype) is None]
    if not strict:
        passed, unexpected = unexpected, []
    else:
        passed = []
    if not (missing or unexpected or wrong or bad_dtype):
        return passed, stood_in
    lines = [f"{where} does not match the model:"]
    if missing:
        lines.append(f"  missing tensors ({len(missing)}):")
        lines += [f"    {n}  expected shape {list(expected[n])}" for n in missing]
    if unexpected:
        lines.append(f"  unexpected tensors ({len(unexpected)}):")
        lines += [f"    {n}  shape {list(infos[n].shape)}" for n in unexpected]
    if wrong:
        lines.append(f"  wrong shapes ({len(wrong)}):")
        lines += [f"    {n}  expected {list(e)}, got {list(g)}" for n, e, g in wrong]
    if bad_dtype:
        lines.append(f"  unsupported dtypes ({len(bad_dtype)}):")
        lines += [f"    {n}  stored as {d}" for n, d in bad_dtype]
    raise WeightError("\n".join(lines), missing, unexpected, wrong, bad_dtype)


def load_weights(folder, expected: Dict[str, Tuple[int, ...]], device, optional=(),
                 fallbacks=None, strict: bool = True) -> LoadedWeights:
    infos = open_checkpoint(folder)
    passed, stood_in = check_against(expected, infos, where=str(folder), optional=optional,
                                     fallbacks=fallbacks, strict=strict)
    files: Dict[Path, MappedFile] = {}
    out = LoadedWeights()
    out.unexpected, out.stood_in = list(passed), dict(stood_in)
    try:
        for name in expected:
            if name not in infos:
                continue                  # optional and absent, or stood in for below
            info = infos[name]
            mf = files.get(info.file)
            if mf is None:
                mf = files[info.file] = MappedFile(info.file)
            t = mf.tensor(info)
            keep = _kept_dtype(info.dtype)
            if keep == torch.int32 and t.dtype == torch.int64 and t.numel():
                if int(t.max()) > 2**31 - 1 or int(t.min()) < -2**31:
                    raise WeightError(f"{name}: integer table does not fit int32")
            out[name] = t.to(device=device, dtype=keep, copy=True)
            del t
    finally:
        for mf in files.values():
            mf.close()
    for name, other in stood_in.items():
        out[name] = out[other]
    return out
