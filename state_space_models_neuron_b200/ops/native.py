"""Build and load the native sm_100a library.

`build()` compiles every `csrc/*.cu` with nvcc for `compute_100a/sm_100a` into
`ops/_native/libssm_b200.so` (in-tree, next to the sources; the kernels expose a plain C ABI so no
PyTorch headers are involved and a full build takes seconds).  `lib()` loads it with ctypes and
declares argument types; if the library is missing it is built on the spot, and if that is impossible
the error is raised: GPU ops never fall back silently.
"""
from __future__ import annotations

import ctypes
import hashlib
import os
import shutil
import subprocess
import threading
from concurrent.futures import ThreadPoolExecutor

_HERE = os.path.dirname(os.path.abspath(__file__))
CSRC = os.path.join(_HERE, "csrc")
OUT_DIR = os.path.join(_HERE, "_native")
LIB_PATH = os.path.join(OUT_DIR, "libssm_b200.so")
NVCC_FLAGS = ["-gencode", "arch=compute_100a,code=sm_100a", "-lineinfo", "-O3", "-std=c++17",
              "--use_fast_math", "-Xcompiler", "-fPIC", "-Xcompiler", "-fvisibility=default"]
_lock = threading.Lock()
_lib = None


def _nvcc() -> str:
    for cand in (os.environ.get("NVCC"), shutil.which("nvcc"), "/usr/local/cuda/bin/nvcc"):
        if cand and os.path.exists(cand):
            return cand
    raise RuntimeError("nvcc not found; cannot build the sm_100a kernels")


def _sources():
    return sorted(f for f in os.listdir(CSRC) if f.endswith(".cu"))


def _source_hash() -> str:
    h = hashlib.sha256()
    for f in sorted(os.listdir(CSRC)):
        if f.endswith((".cu", ".cuh", ".h")):
            with open(os.path.join(CSRC, f), "rb") as fh:
                h.update(f.encode())
                h.update(fh.read())
    h.update(" ".join(NVCC_FLAGS).encode())
    return h.hexdigest()


def is_current() -> bool:
    stamp = os.path.join(OUT_DIR, "build.hash")
    if not (os.path.exists(LIB_PATH) and os.path.exists(stamp)):
        return False
    with open(stamp) as f:
        return f.read().strip() == _source_hash()


def build(force: bool = False, verbose: bool = False) -> str:
    """Compile all kernels (parallel over files) and link the shared library.  Returns its path."""
    import fcntl
    os.makedirs(OUT_DIR, exist_ok=True)
    # one builder at a time, across threads and across processes (several ranks may find a stale library at once)
    with _lock, open(os.path.join(OUT_DIR, "build.lock"), "w") as lockf:
        fcntl.flock(lockf, fcntl.LOCK_EX)
        if not force and is_current():
            return LIB_PATH
        nvcc = _nvcc()
        tag = f".{os.getpid()}"

        def compile_one(src):
            obj = os.path.join(OUT_DIR, src[:-3] + tag + ".o")
            cmd = [nvcc, *NVCC_FLAGS, "-I", CSRC, "-c", os.path.join(CSRC, src), "-o", obj]
            if verbose:
                cmd.insert(1, "-Xptxas=-v")
            r = subprocess.run(cmd, capture_output=True, text=True)
            if r.returncode != 0:
                raise RuntimeError(f"nvcc failed for {src}:\n{r.stdout}\n{r.stderr}")
            if verbose:
                print(r.stderr)
            return obj

        with ThreadPoolExecutor(max_workers=min(8, os.cpu_count() or 1)) as ex:
            objs = list(ex.map(compile_one, _sources()))
        tmp = LIB_PATH + tag + ".tmp"
        r = subprocess.run([nvcc, "-shared", "-o", tmp, *objs, "-gencode", "arch=compute_100a,code=sm_100a"],
                           capture_output=True, text=True)
        if r.returncode != 0:
            raise RuntimeError(f"link failed:\n{r.stdout}\n{r.stderr}")
        os.replace(tmp, LIB_PATH)
        for o in objs:
            os.remove(o)
        with open(os.path.join(OUT_DIR, "build.hash"), "w") as f:
            f.write(_source_hash())
        return LIB_PATH


def lib() -> ctypes.CDLL:
    global _lib
    if _lib is None:
        if not is_current():
            build()
        _lib = ctypes.CDLL(LIB_PATH)
    return _lib


def check(code: int, what: str) -> None:
    if code != 0:
        raise RuntimeError(f"{what} failed with code {code} (negative: argument check; positive: cudaError)")
