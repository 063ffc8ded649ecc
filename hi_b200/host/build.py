"""Build and load ``libhi_b200_host.so``: the host runtime (cache manager, step packing,
scheduler) from ``hi_b200/csrc/host/*.cpp`` with the C++ compiler. No CUDA in it, so it
builds and runs on a machine without a GPU.

Built in-tree (``hi_b200/csrc/_build/``) on first use and rebuilt when a source changes
(content hash); nothing outside the checkout is written. There is no Python stand-in: if the
library cannot be built or loaded, :func:`library` raises.
"""
from __future__ import annotations

import ctypes
import hashlib
import os
import shutil
import subprocess
import sys
import threading
from typing import List, Optional

HOST_SRC = os.path.normpath(os.path.join(os.path.dirname(os.path.abspath(__file__)), "..", "csrc", "host"))
BUILD_DIR = os.path.normpath(os.path.join(HOST_SRC, "..", "_build"))
LIB_NAME = "libhi_b200_host.so"
CXX_FLAGS = ["-O2", "-std=c++17", "-fPIC", "-Wall"]

_lock = threading.Lock()
_lib: Optional[ctypes.CDLL] = None


class HostBuildError(RuntimeError):
    pass


def _cxx() -> str:
    for cand in (os.environ.get("HI_B200_CXX"), os.environ.get("CXX"), "g++", "c++", "clang++"):
        if cand:
            path = cand if os.path.isfile(cand) else shutil.which(cand)
            if path:
                return path
    raise HostBuildError("no C++ compiler found (looked at $HI_B200_CXX, $CXX, g++, c++, clang++)")


def sources() -> List[str]:
    return sorted(os.path.join(HOST_SRC, f) for f in os.listdir(HOST_SRC) if f.endswith(".cpp"))


def _digest() -> str:
    h = hashlib.sha256()
    for name in sorted(os.listdir(HOST_SRC)):
        if name.endswith((".cpp", ".h")):
            h.update(name.encode())
            with open(os.path.join(HOST_SRC, name), "rb") as f:
                h.update(f.read())
    h.update(" ".join(CXX_FLAGS).encode())
    return h.hexdigest()[:16]


def build(verbose: bool = True, force: bool = False) -> str:
    """Compile and link the host library. Returns its path."""
    os.makedirs(BUILD_DIR, exist_ok=True)
    digest = _digest()
    lib_path = os.path.join(BUILD_DIR, LIB_NAME)
    stamp = os.path.join(BUILD_DIR, "host_digest.txt")
    if not force and os.path.isfile(lib_path) and os.path.isfile(stamp):
        with open(stamp) as f:
            if f.read().strip() == digest:
                return lib_path
    cxx = _cxx()
    if verbose:
        print(f"[hi_b200] building {LIB_NAME} with {cxx}", file=sys.stderr, flush=True)
    tmp = lib_path + f".{os.getpid()}.tmp"
    cmd = [cxx, *CXX_FLAGS, "-shared", "-I", HOST_SRC, "-o", tmp, *sources()]
    proc = subprocess.run(cmd, stdout=subprocess.PIPE, stderr=subprocess.STDOUT, text=True)
    if proc.returncode != 0:
        raise HostBuildError("command failed: " + " ".join(cmd) + "\n" + proc.stdout)
    os.replace(tmp, lib_path)
    with open(stamp, "w") as f:
        f.write(digest)
    return lib_path


I, L, P = ctypes.c_int, ctypes.c_int64, ctypes.c_void_p
_SIGNATURES = {
    "hbh_pool_create": (P, [I]), "hbh_pool_destroy": (None, [P]), "hbh_pool_take": (I, [P, L, P]),
    "hbh_pool_give": (I, [P, I, L]), "hbh_pool_owner": (I, [P, I, P, P]), "hbh_pool_stat": (L, [P, I]),
    "hbh_cache_create": (P, [I, P, P, P, I, I]), "hbh_cache_destroy": (None, [P]),
    "hbh_cache_error": (ctypes.c_char_p, [P]), "hbh_cache_pool": (P, [P, I]), "hbh_cache_open": (I, [P, L, P]),
    "hbh_cache_close": (I, [P, L]), "hbh_cache_is_open": (I, [P, L]), "hbh_cache_free_slots": (I, [P]),
    "hbh_cache_open_requests": (I, [P, P, I]), "hbh_cache_request_stat": (L, [P, L, I]),
    "hbh_cache_pages_needed": (I, [P, L, I, L, P]), "hbh_cache_reserve": (I, [P, L, I, P]),
    "hbh_cache_unreserve": (I, [P, L, P]), "hbh_cache_commit": (I, [P, L, I]), "hbh_cache_returned": (I, [P, P, I]),
    "hbh_cache_table_length": (I, [P, I, L]), "hbh_cache_table": (I, [P, I, L, P, I]), "hbh_cache_check": (I, [P]),
    "hbh_step_widths": (I, [P, I, P, P]), "hbh_pack_step": (I, [P, I, P, P, P, P, P, P, P, P, P, P, P, P]),
    "hbh_sched_create": (P, [P, I, I, I, I, L]), "hbh_sched_destroy": (None, [P]),
    "hbh_sched_error": (ctypes.c_char_p, [P]), "hbh_sched_set_release": (None, [P, P, P]),
    "hbh_sched_add": (I, [P, L, I, I]), "hbh_sched_abort": (I, [P, L]), "hbh_sched_has_work": (I, [P]), "hbh_sched_assume_running": (I, [P, L, L]),
    "hbh_sched_plan": (I, [P, P, P, I, P, P, I, P, P, I, P]), "hbh_sched_commit": (I, [P, L, P, I, P, I, P]),
    "hbh_sched_request_stat": (L, [P, L, I]), "hbh_sched_queue": (I, [P, I, P, I]), "hbh_sched_counter": (L, [P, I]),
    "hbh_sched_forget": (None, [P, L]),
    "hbh_random_normal": (I, [P, L, L, ctypes.c_uint64, ctypes.c_float]),
    "hbh_cpu_forward": (I, [P, P, P, I, P, I, P, I, P, P]),
}

# the C interface's codes (hi_b200/csrc/host/runtime.h)
OK, ERR_ARG, ERR_NOT_OPEN, ERR_ALREADY_OPEN, ERR_NO_SLOT, ERR_NO_PAGES = 0, -1, -2, -3, -4, -5
ERR_BAD_PAGE, ERR_DOUBLE_FREE, ERR_NOT_OWNER, ERR_INVARIANT, ERR_CONTEXT_LENGTH, ERR_NEVER_FITS = -6, -7, -8, -9, -10, -11
ERR_CAPACITY = -12
RELEASE_FN = ctypes.CFUNCTYPE(None, ctypes.c_void_p, ctypes.c_int64)


def library() -> ctypes.CDLL:
    """The loaded host library; builds it first if needed. Raises if that fails."""
    global _lib
    with _lock:
        if _lib is None:
            path = build()
            try:
                lib = ctypes.CDLL(path)
            except OSError as e:
                raise HostBuildError(f"cannot load {path}: {e}") from e
            for name, (res, args) in _SIGNATURES.items():
                fn = getattr(lib, name)
                fn.restype, fn.argtypes = res, args
            _lib = lib
        return _lib
