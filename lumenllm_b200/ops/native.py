"""Loads the compiled kernel modules and calls their C entry points.

There is no fallback: if a module cannot be built or loaded, or a launch
reports an error, an exception says so.
"""
from __future__ import annotations

import ctypes
import threading

import torch

from ..csrc import build as _build

ERR_UNSUPPORTED = 100001
ERR_BAD_ARGUMENT = 100002
ERR_NOT_READY = 100003


class KernelError(RuntimeError):
    pass


_libs: dict = {}
_lock = threading.Lock()


def library(module: str) -> ctypes.CDLL:
    lib = _libs.get(module)
    if lib is None:
        with _lock:
            lib = _libs.get(module)
            if lib is None:
                path = _build.ensure_built([module])[module]
                try:
                    lib = ctypes.CDLL(str(path))
                except OSError as e:  # pragma: no cover
                    raise KernelError(f"cannot load kernel module '{module}' from {path}: {e}") from e
                _libs[module] = lib
    return lib


def preload(modules) -> None:
    """Builds (in parallel) and loads the given modules."""
    _build.ensure_built(list(modules))
    for m in modules:
        library(m)


def set_dependent_launch(on: bool, modules=None) -> None:
    """Measurement switch: programmatic dependent launch on or off for the given modules (all
    that are loaded when none are named). The product never calls this; it is on."""
    for m in (list(_libs) if modules is None else modules):
        f = library(m).lumen_set_pdl
        f.restype, f.argtypes = None, [ctypes.c_int]
        f(1 if on else 0)


_fn_cache: dict = {}


_probe = None


def _raw_fn(module: str, name: str, argtypes):
    key = (module, name)
    f = _fn_cache.get(key)
    if f is None:
        f = getattr(library(module), name)
        f.restype = ctypes.c_int
        f.argtypes = list(argtypes)
        _fn_cache[key] = f
    return f


def fn(module: str, name: str, argtypes):
    """The C entry point `name` of a module (one that launches kernels)."""
    f = _raw_fn(module, name, argtypes)
    return f if _probe is None else _bracketed(name, f)


def instrument(probe) -> None:
    """Measurement hook: with `probe(name, args) -> (label, start event, end event)` every
    kernel entry point called from now on records the two events around its launch; None
    switches it off again. The product never sets it."""
    global _probe
    _probe = probe


def _bracketed(name, f):
    def call(*args):
        _, e0, e1 = _probe(name, args)
        e0.record()
        rc = f(*args)
        e1.record()
        return rc
    return call


launches = 0   # kernels of this library launched (or recorded into a graph) so far


def check(code: int, what: str) -> None:
    global launches
    if code == 0:
        launches += 1
        return
    if code == ERR_UNSUPPORTED:
        raise KernelError(f"{what}: this kernel does not take these sizes")
    if code == ERR_BAD_ARGUMENT:
        raise KernelError(f"{what}: bad argument")
    if code == ERR_NOT_READY:
        raise KernelError(f"{what}: the kernel's set-up failed on this device")
    raise KernelError(f"{what}: CUDA error {code}")


_raw_stream = getattr(torch._C, "_cuda_getCurrentRawStream", None)


def stream_ptr() -> int:
    """The current stream of the current device as the raw handle the C entry points take.
    Asked for at every launch (a capture or a `torch.cuda.stream` block changes it), so it goes
    the short way where torch offers one: hundreds of launches make a step, and the host's time
    per launch is what a short prompt waits for."""
    if _raw_stream is not None:
        return _raw_stream(torch.cuda.current_device())
    return torch.cuda.current_stream().cuda_stream


def int_fn(module: str, name: str, argtypes):
    """A C function of a module that returns a plain number (no launch, no error code)."""
    return _raw_fn(module, name, argtypes)


def ptr(t):
    return 0 if t is None else t.data_ptr()


def require(t: torch.Tensor, dtype, name: str, *, contiguous=True):
    if not t.is_cuda:
        raise KernelError(f"{name}: tensor is not on a CUDA device (no CPU path exists)")
    if t.dtype != dtype:
        raise KernelError(f"{name}: expected {dtype}, got {t.dtype}")
    if contiguous and not t.is_contiguous():
        raise KernelError(f"{name}: tensor must be contiguous")
    return t
