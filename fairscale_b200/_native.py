"""Build and load the native sm_100a library (``fairscale_b200/lib/libfsb200.so``).

The kernels are plain CUDA with a C ABI (no torch headers), compiled file by file with
``nvcc -gencode arch=compute_100a,code=sm_100a`` and linked into one shared object that
lives inside the package directory.  Python talks to it through :mod:`ctypes`; tensors are
passed as raw device pointers plus the current CUDA stream.

On a machine with a GPU the library is mandatory: :func:`lib` raises if it is missing so a
silent fallback to framework ops cannot happen.  Without a GPU (CPU test tier) callers use
their PyTorch reference implementations and never ask for the library.
"""

from __future__ import annotations

import ctypes
import os
import shutil
import subprocess
import sys
import threading
from concurrent.futures import ThreadPoolExecutor
from typing import Any, List, Optional

_PKG_DIR = os.path.dirname(os.path.abspath(__file__))
CSRC_DIR = os.path.join(_PKG_DIR, "csrc")
OBJ_DIR = os.path.join(_PKG_DIR, "_obj")
LIB_DIR = os.path.join(_PKG_DIR, "lib")
LIB_PATH = os.path.join(LIB_DIR, "libfsb200.so")

NVCC_FLAGS = [
    "-gencode",
    "arch=compute_100a,code=sm_100a",
    "-lineinfo",
    "-O3",
    "-std=c++17",
    "--expt-relaxed-constexpr",
    "-Xcompiler",
    "-fPIC",
    "-Xcompiler",
    "-fvisibility=hidden",
]

_lock = threading.Lock()
_lib: Optional[ctypes.CDLL] = None


def _nvcc() -> str:
    for cand in (os.environ.get("NVCC"), shutil.which("nvcc"), "/usr/local/cuda/bin/nvcc"):
        if cand and os.path.exists(cand):
            return cand
    raise RuntimeError("nvcc not found; set NVCC or install the CUDA toolkit")


def sources() -> List[str]:
    return sorted(os.path.join(CSRC_DIR, f) for f in os.listdir(CSRC_DIR) if f.endswith(".cu"))


def _headers_mtime() -> float:
    return max(os.path.getmtime(os.path.join(CSRC_DIR, f)) for f in os.listdir(CSRC_DIR) if f.endswith((".cuh", ".h")))


def _compile_one(src: str, verbose: bool, ptxas_info: bool) -> str:
    obj = os.path.join(OBJ_DIR, os.path.basename(src)[:-3] + ".o")
    stale = (
        not os.path.exists(obj)
        or os.path.getmtime(obj) < os.path.getmtime(src)
        or os.path.getmtime(obj) < _headers_mtime()
    )
    if stale:
        cmd = [_nvcc()] + NVCC_FLAGS + (["-Xptxas", "-v"] if ptxas_info else []) + ["-I", CSRC_DIR, "-c", src, "-o", obj]
        if verbose:
            print(" ".join(cmd), flush=True)
        res = subprocess.run(cmd, capture_output=True, text=True)
        if res.returncode != 0:
            raise RuntimeError(f"nvcc failed for {src}:\n{res.stdout}\n{res.stderr}")
        if ptxas_info or verbose:
            sys.stderr.write(res.stderr)
    return obj


def build(force: bool = False, verbose: bool = False, ptxas_info: bool = False) -> str:
    """Compile every ``csrc/*.cu`` for sm_100a and link ``libfsb200.so``; returns its path.

    Only stale objects are rebuilt unless ``force``.  Works without a GPU (nvcc cross-compiles).
    """
    global _lib
    with _lock:
        os.makedirs(OBJ_DIR, exist_ok=True)
        os.makedirs(LIB_DIR, exist_ok=True)
        if force:
            for f in os.listdir(OBJ_DIR):
                os.remove(os.path.join(OBJ_DIR, f))
        srcs = sources()
        with ThreadPoolExecutor(max_workers=min(8, len(srcs))) as pool:
            objs = list(pool.map(lambda s: _compile_one(s, verbose, ptxas_info), srcs))
        relink = not os.path.exists(LIB_PATH) or any(os.path.getmtime(o) > os.path.getmtime(LIB_PATH) for o in objs)
        if relink:
            tmp = LIB_PATH + ".tmp"
            cmd = [_nvcc(), "-shared", "-o", tmp] + objs + ["-gencode", "arch=compute_100a,code=sm_100a", "-lcudart"]
            if verbose:
                print(" ".join(cmd), flush=True)
            res = subprocess.run(cmd, capture_output=True, text=True)
            if res.returncode != 0:
                raise RuntimeError(f"link failed:\n{res.stdout}\n{res.stderr}")
            os.replace(tmp, LIB_PATH)
            _lib = None
    return LIB_PATH


def available() -> bool:
    """True if the shared object exists (it may still be unusable without a CUDA device)."""
    return os.path.exists(LIB_PATH)


def lib() -> ctypes.CDLL:
    """The loaded native library.  Raises if it has not been built."""
    global _lib
    if _lib is None:
        with _lock:
            if _lib is None:
                if not os.path.exists(LIB_PATH):
                    raise RuntimeError(
                        f"native library {LIB_PATH} is missing: run `python -m fairscale_b200._native` "
                        "(or call fairscale_b200._native.build()) before using CUDA ops"
                    )
                _lib = ctypes.CDLL(LIB_PATH)
    return _lib


def use_native(*tensors: Any) -> bool:
    """Decide between the native kernel and the PyTorch reference for an op.

    CUDA tensors always take the native path (and fail loudly if the library is absent);
    CPU tensors take the reference path.
    """
    return len(tensors) > 0 and all(getattr(t, "is_cuda", False) for t in tensors if t is not None)


def check(code: int, what: str) -> None:
    if code != 0:
        raise RuntimeError(f"{what} failed with code {code}")


_status_tensors: dict = {}


def status_word(device: Any) -> Any:
    """Per-device int32 status word that kernels with bounded waits write on timeout."""
    import torch

    key = torch.device(device).index if torch.device(device).index is not None else torch.cuda.current_device()
    if key not in _status_tensors:
        _status_tensors[key] = torch.zeros(1, dtype=torch.int32, device=f"cuda:{key}")
    return _status_tensors[key]


def read_status(device: Any = None) -> int:
    """Synchronously read (and clear) the status word; 0 means no kernel reported an error."""
    import torch

    dev = torch.device("cuda", torch.cuda.current_device()) if device is None else torch.device(device)
    t = status_word(dev)
    val = int(t.item())
    if val != 0:
        t.zero_()
    return val


if __name__ == "__main__":
    print(build(force="--force" in sys.argv, verbose=True, ptxas_info="--ptxas" in sys.argv))
