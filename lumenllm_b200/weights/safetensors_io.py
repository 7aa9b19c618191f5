"""Reader and writer of the safetensors container:
[u64 little-endian header length][JSON header][payload]; per tensor `dtype`,
`shape`, `data_offsets` relative to the payload. The checks are those of the
reference (crates/aegisllm-base/src/tensor/core.rs:86-181: byte size equals
shape x dtype size, the range ends inside the payload;
crates/aegisllm-base/src/artifact.rs:651-674: header length guard).
"""
from __future__ import annotations

import json
import mmap
import struct
from dataclasses import dataclass
from pathlib import Path
from typing import Dict, Tuple

import torch

_DTYPES = {
    "F32": (torch.float32, 4), "BF16": (torch.bfloat16, 2), "F16": (torch.float16, 2),
    "F64": (torch.float64, 8), "I64": (torch.int64, 8), "I32": (torch.int32, 4),
    "I16": (torch.int16, 2), "I8": (torch.int8, 1), "U8": (torch.uint8, 1), "BOOL": (torch.bool, 1),
}
_NAMES = {v[0]: k for k, v in _DTYPES.items()}
_MAX_HEADER = 256 << 20


class SafetensorsError(ValueError):
    pass


@dataclass(frozen=True)
class TensorInfo:
    name: str
    dtype: str
    shape: Tuple[int, ...]
    begin: int   # absolute file offsets
    end: int
    file: Path


def read_header(path) -> Dict[str, TensorInfo]:
    path = Path(path)
    size = path.stat().st_size
    with open(path, "rb") as f:
        head = f.read(8)
        if len(head) < 8:
            raise SafetensorsError(f"{path}: too short to be a safetensors file")
        if head.startswith(b"version "):
            raise SafetensorsError(f"{path}: this is a git-lfs pointer, not the weights")
        (hlen,) = struct.unpack("<Q", head)
        if hlen > _MAX_HEADER or 8 + hlen > size:
            raise SafetensorsError(f"{path}: header length {hlen} is beyond the file")
        try:
            header = json.loads(f.read(hlen))
        except (json.JSONDecodeError, UnicodeDecodeError) as e:
            raise SafetensorsError(f"{path}: header is not valid JSON ({e})") from e
    payload0 = 8 + hlen
    payload_len = size - payload0
    out = {}
    for name, info in header.items():
        if name == "__metadata__":
            continue
        dt = info.get("dtype")
        if dt not in _DTYPES:
            raise SafetensorsError(f"{path}: tensor '{name}' has unsupported dtype {dt!r}")
        shape = tuple(int(x) for x in info["shape"])
        b, e = (int(x) for x in info["data_offsets"])
        n = 1
        for s in shape:
            n *= s
        if e - b != n * _DTYPES[dt][1]:
            raise SafetensorsError(f"{path}: tensor '{name}' holds {e - b} bytes, but shape "
                                   f"{list(shape)} of {dt} needs {n * _DTYPES[dt][1]}")
        if b < 0 or e > payload_len:
            raise SafetensorsError(f"{path}: tensor '{name}' ends at byte {e} of a payload of "
                                   f"{payload_len} (file truncated?)")
        out[name] = TensorInfo(name, dt, shape, payload0 + b, payload0 + e, path)
    return out


class MappedFile:
    """One mmap per shard; tensors are views of it until copied."""

    def __init__(self, path):
        self._f = open(path, "rb")
        self._mm = mmap.mmap(self._f.fileno(), 0, access=mmap.ACCESS_READ)

    def tensor(self, info: TensorInfo) -> torch.Tensor:
        dt, _ = _DTYPES[info.dtype]
        if info.end == info.begin:
            return torch.empty(info.shape, dtype=dt)
        buf = memoryview(self._mm)[info.begin:info.end]
        import warnings
        with warnings.catch_warnings():
            warnings.simplefilter("ignore")  # the view is read-only; it is copied before use
            t = torch.frombuffer(buf, dtype=dt)
        return t.reshape(info.shape)

    def close(self):
        try:
            self._mm.close()
        except BufferError:
            pass
        self._f.close()


def write_file(path, tensors: Dict[str, torch.Tensor], metadata=None) -> None:
    header, offset, blobs = {}, 0, []
    for name, t in tensors.items():
        t = t.detach().cpu().contiguous()
        if t.dtype not in _NAMES:
            raise SafetensorsError(f"cannot store dtype {t.dtype}")
        raw = t.view(torch.uint8).reshape(-1).numpy().tobytes() if t.numel() else b""
        header[name] = {"dtype": _NAMES[t.dtype], "shape": list(t.shape),
                        "data_offsets": [offset, offset + len(raw)]}
        offset += len(raw)
        blobs.append(raw)
    if metadata:
        header["__metadata__"] = {str(k): str(v) for k, v in metadata.items()}
    hj = json.dumps(header, separators=(",", ":")).encode()
    hj += b" " * ((8 - len(hj) % 8) % 8)
    with open(path, "wb") as f:
        f.write(struct.pack("<Q", len(hj)))
        f.write(hj)
        for raw in blobs:
            f.write(raw)
