"""Build and load ``libhi_b200_kernels.so`` from ``hi_b200/csrc/*.cu`` with nvcc for sm_100a.

The library is built in-tree (``hi_b200/csrc/_build/``) on first use and rebuilt when a
source changes (content hash). Nothing outside the checkout is written, so it works for
an ordinary user with an empty HOME. While nvcc runs, a line is printed every few seconds.
There is no fallback: if the library cannot be built or loaded, :func:`library` raises.
"""
from __future__ import annotations

import ctypes
import hashlib
import os
import shutil
import subprocess
import sys
import threading
import time
from concurrent.futures import ThreadPoolExecutor
from typing import List, Optional

CSRC = os.path.normpath(os.path.join(os.path.dirname(os.path.abspath(__file__)), "..", "csrc"))
BUILD_DIR = os.path.join(CSRC, "_build")
LIB_NAME = "libhi_b200_kernels.so"
ARCH_FLAGS = ["-gencode", "arch=compute_100a,code=sm_100a"]
NVCC_FLAGS = ["-O3", "-std=c++17", "-lineinfo", "-Xcompiler", "-fPIC", "--expt-relaxed-constexpr"]

_lock = threading.Lock()
_lib: Optional[ctypes.CDLL] = None


class KernelBuildError(RuntimeError):
    pass


def _nvcc() -> str:
    for cand in (os.environ.get("HI_B200_NVCC"), shutil.which("nvcc"), "/usr/local/cuda/bin/nvcc"):
        if cand and os.path.isfile(cand):
            return cand
    raise KernelBuildError("nvcc not found (looked at $HI_B200_NVCC, PATH and /usr/local/cuda/bin)")


def sources() -> List[str]:
    return sorted(os.path.join(CSRC, f) for f in os.listdir(CSRC) if f.endswith(".cu"))


def _headers() -> List[str]:
    return sorted(os.path.join(CSRC, f) for f in os.listdir(CSRC) if f.endswith((".h", ".cuh")))


def _digest() -> str:
    h = hashlib.sha256()
    for path in sources() + _headers():
        h.update(os.path.basename(path).encode())
        with open(path, "rb") as f:
            h.update(f.read())
    h.update(" ".join(ARCH_FLAGS + NVCC_FLAGS).encode())
    return h.hexdigest()[:16]


def _run(cmd: List[str]) -> None:
    proc = subprocess.run(cmd, stdout=subprocess.PIPE, stderr=subprocess.STDOUT, text=True)
    if proc.returncode != 0:
        raise KernelBuildError("command failed: " + " ".join(cmd) + "\n" + proc.stdout)


def build(verbose: bool = True, force: bool = False) -> str:
    """Compile every .cu file (in parallel) and link the shared library. Returns its path."""
    os.makedirs(BUILD_DIR, exist_ok=True)
    digest = _digest()
    lib_path = os.path.join(BUILD_DIR, LIB_NAME)
    stamp = os.path.join(BUILD_DIR, "digest.txt")
    if not force and os.path.isfile(lib_path) and os.path.isfile(stamp):
        with open(stamp) as f:
            if f.read().strip() == digest:
                return lib_path
    nvcc = _nvcc()
    srcs = sources()
    t0 = time.time()
    done = threading.Event()

    def ticker():
        while not done.wait(5.0):
            print(f"[hi_b200] compiling CUDA kernels for sm_100a ... {time.time() - t0:.0f}s",
                  file=sys.stderr, flush=True)

    if verbose:
        print(f"[hi_b200] building {LIB_NAME} from {len(srcs)} sources with {nvcc}", file=sys.stderr, flush=True)
        threading.Thread(target=ticker, daemon=True).start()
    try:
        objs = [os.path.join(BUILD_DIR, os.path.basename(s)[:-3] + f".{digest}.o") for s in srcs]

        def compile_one(pair):
            src, obj = pair
            if not os.path.isfile(obj):
                _run([nvcc, *ARCH_FLAGS, *NVCC_FLAGS, "-I", CSRC, "-c", src, "-o", obj + ".tmp"])
                os.replace(obj + ".tmp", obj)

        with ThreadPoolExecutor(max_workers=min(8, len(srcs))) as pool:
            list(pool.map(compile_one, zip(srcs, objs)))
        tmp = lib_path + f".{os.getpid()}.tmp"
        _run([nvcc, *ARCH_FLAGS, "-shared", "-o", tmp, *objs, "-lcudart"])
        os.replace(tmp, lib_path)
        with open(stamp, "w") as f:
            f.write(digest)
        for name in os.listdir(BUILD_DIR):  # objects of older source states
            if name.endswith(".o") and f".{digest}." not in name:
                try:
                    os.remove(os.path.join(BUILD_DIR, name))
                except OSError:
                    pass
    finally:
        done.set()
    if verbose:
        print(f"[hi_b200] built in {time.time() - t0:.1f}s", file=sys.stderr, flush=True)
    return lib_path


def library() -> ctypes.CDLL:
    """The loaded kernel library; builds it first if needed. Raises if that fails."""
    global _lib
    with _lock:
        if _lib is None:
            path = build()
            try:
                _lib = ctypes.CDLL(path)
            except OSError as e:
                raise KernelBuildError(f"cannot load {path}: {e}") from e
        return _lib
