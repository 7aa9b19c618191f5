"""Builds the sm_100a kernel library, one shared object per source file.

Each module is compiled by a direct nvcc call (no JIT cache in the home
directory) into ``lumen_<module>.<hash of its sources>.so`` beside the sources,
so a checkout that has been built once needs no compiler again, a changed
source is rebuilt under a new name, and two processes that build at the same
time cannot see a half-written file (the result is renamed into place). If the
package folder cannot be written, a per-user folder under the temporary
directory is used. While nvcc runs a line is printed to stderr every few
seconds.
"""
from __future__ import annotations

import hashlib
import os
import shutil
import subprocess
import sys
import tempfile
import threading
import time
from concurrent.futures import ThreadPoolExecutor
from pathlib import Path

CSRC = Path(__file__).resolve().parent

# module -> (sources compiled into it, headers it depends on)
MODULES = {
    "core": (["core.cu"], ["common.cuh", "qk_head.cuh"]),
    "gemm_f32": (["gemm_f32.cu"], ["common.cuh"]),
    "gemm_tc": (["gemm_tc.cu"], ["common.cuh", "mma_utils.cuh"]),
    "attn_generic": (["attn_generic.cu"], ["common.cuh"]),
    "sample": (["sample.cu"], ["common.cuh"]),
    "attn_decode": (["attn_decode.cu"], ["common.cuh", "mma_utils.cuh", "qk_head.cuh", "attn_decode_noalloc.h"]),
    "attn_prefill": (["attn_prefill.cu"], ["common.cuh", "mma_utils.cuh"]),
    "attn_prefill_tc": (["attn_prefill_tc.cu"], ["common.cuh", "mma_utils.cuh"]),
    "stream_probe": (["stream_probe.cu"], ["common.cuh", "mma_utils.cuh"]),     # a measurement (kbench stream)
}

NVCC_FLAGS = [
    "-gencode", "arch=compute_100a,code=sm_100a",
    "-lineinfo", "-O3", "-std=c++17",
    "-Xcompiler", "-fPIC", "-shared",
]


class BuildError(RuntimeError):
    pass


def page_size() -> int:
    """Tokens per cache page: the value of LUMEN_PAGE in common.cuh, the one place where the
    number is written. The Python side (cache, generation loop, metadata) reads it here."""
    import re
    m = re.search(r"^#define\s+LUMEN_PAGE\s+(\d+)\s*$", (CSRC / "common.cuh").read_text(), re.M)
    if not m:
        raise BuildError("common.cuh does not define LUMEN_PAGE")
    return int(m.group(1))


def _nvcc() -> str:
    for cand in (os.environ.get("NVCC"), shutil.which("nvcc"), "/usr/local/cuda/bin/nvcc"):
        if cand and Path(cand).exists():
            return cand
    raise BuildError("nvcc not found: the CUDA kernels of lumenllm_b200 cannot be built "
                     "(looked at $NVCC, PATH and /usr/local/cuda/bin/nvcc)")


def _digest(module: str) -> str:
    srcs, hdrs = MODULES[module]
    h = hashlib.sha256()
    for name in list(srcs) + list(hdrs):
        h.update(name.encode())
        h.update((CSRC / name).read_bytes())
    h.update(" ".join(NVCC_FLAGS).encode())
    return h.hexdigest()[:12]


def _out_dirs():
    yield CSRC
    uid = os.getuid() if hasattr(os, "getuid") else 0
    yield Path(tempfile.gettempdir()) / f"lumenllm_b200-{uid}"


def _find_built(module: str):
    name = f"lumen_{module}.{_digest(module)}.so"
    for d in _out_dirs():
        p = d / name
        if p.exists():
            return p
    return None


def _writable_dir() -> Path:
    for d in _out_dirs():
        try:
            d.mkdir(parents=True, exist_ok=True)
            probe = d / f".w{os.getpid()}"
            probe.write_bytes(b"")
            probe.unlink()
            return d
        except OSError:
            continue
    raise BuildError("no writable folder for the compiled kernels")


def _compile(module: str, out_dir: Path) -> Path:
    srcs, _ = MODULES[module]
    final = out_dir / f"lumen_{module}.{_digest(module)}.so"
    tmp = out_dir / f".lumen_{module}.{os.getpid()}.{threading.get_ident()}.tmp.so"
    cmd = [_nvcc(), *NVCC_FLAGS, "-I", str(CSRC), "-o", str(tmp)] + [str(CSRC / s) for s in srcs]
    env = dict(os.environ)
    env.setdefault("TMPDIR", tempfile.gettempdir())
    proc = subprocess.run(cmd, stdout=subprocess.PIPE, stderr=subprocess.STDOUT, text=True, env=env)
    if proc.returncode != 0:
        try:
            tmp.unlink()
        except OSError:
            pass
        raise BuildError(f"nvcc failed for kernel module '{module}':\n{' '.join(cmd)}\n{proc.stdout}")
    os.replace(tmp, final)
    for old in out_dir.glob(f"lumen_{module}.*.so"):  # stale builds of older sources
        if old != final:
            try:
                old.unlink()
            except OSError:
                pass
    return final


def ensure_built(modules=None, verbose=True) -> dict:
    """Returns {module: path of its shared object}, compiling what is missing."""
    modules = list(MODULES) if modules is None else list(modules)
    for m in modules:
        if m not in MODULES:
            raise BuildError(f"unknown kernel module '{m}'")
    paths, todo = {}, []
    for m in modules:
        p = _find_built(m)
        if p is None:
            todo.append(m)
        else:
            paths[m] = p
    if not todo:
        return paths
    out_dir = _writable_dir()
    t0 = time.time()
    if verbose:
        print(f"[lumenllm_b200] compiling CUDA kernels for sm_100a: {', '.join(todo)}",
              file=sys.stderr, flush=True)
    done = threading.Event()

    def ticker():
        while not done.wait(8.0):
            print(f"[lumenllm_b200] still compiling ({time.time() - t0:.0f} s) ...",
                  file=sys.stderr, flush=True)

    th = threading.Thread(target=ticker, daemon=True)
    if verbose:
        th.start()
    try:
        with ThreadPoolExecutor(max_workers=min(len(todo), os.cpu_count() or 4)) as ex:
            for m, p in zip(todo, ex.map(lambda mod: _compile(mod, out_dir), todo)):
                paths[m] = p
    finally:
        done.set()
    if verbose:
        print(f"[lumenllm_b200] kernels built in {time.time() - t0:.0f} s", file=sys.stderr, flush=True)
    return paths


if __name__ == "__main__":
    for mod, path in ensure_built(sys.argv[1:] or None).items():
        print(mod, path)
