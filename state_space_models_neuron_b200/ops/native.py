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
DEBUG_LIB_PATH = os.path.join(OUT_DIR, "libssm_b200_debug.so")       # same sources with -DSSM_DEBUG_BOUNDS
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


def is_current(debug: bool = False) -> bool:
    stamp = os.path.join(OUT_DIR, "build_debug.hash" if debug else "build.hash")
    if not (os.path.exists(DEBUG_LIB_PATH if debug else LIB_PATH) and os.path.exists(stamp)):
        return False
    with open(stamp) as f:
        return f.read().strip() == _source_hash()


def build(force: bool = False, verbose: bool = False, debug: bool = False) -> str:
    """Compile all kernels (parallel over files) and link the shared library.  Returns its path.
    `debug=True` builds a second library, `libssm_b200_debug.so`, from the same sources with -DSSM_DEBUG_BOUNDS:
    device-side index checks that record the first violation in a status array and skip the access (no trap);
    `debug_bounds(lib)` reads the record."""
    import fcntl
    os.makedirs(OUT_DIR, exist_ok=True)
    lib_path = DEBUG_LIB_PATH if debug else LIB_PATH
    # one builder at a time, across threads and across processes (several ranks may find a stale library at once)
    with _lock, open(os.path.join(OUT_DIR, "build.lock"), "w") as lockf:
        fcntl.flock(lockf, fcntl.LOCK_EX)
        if not force and is_current(debug):
            return lib_path
        nvcc = _nvcc()
        tag = f".{os.getpid()}" + (".dbg" if debug else "")
        extra = ["-DSSM_DEBUG_BOUNDS"] if debug else []

        def compile_one(src):
            obj = os.path.join(OUT_DIR, src[:-3] + tag + ".o")
            cmd = [nvcc, *NVCC_FLAGS, *extra, "-I", CSRC, "-c", os.path.join(CSRC, src), "-o", obj]
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
        tmp = lib_path + tag + ".tmp"
        r = subprocess.run([nvcc, "-shared", "-o", tmp, *objs, "-gencode", "arch=compute_100a,code=sm_100a"],
                           capture_output=True, text=True)
        if r.returncode != 0:
            raise RuntimeError(f"link failed:\n{r.stdout}\n{r.stderr}")
        os.replace(tmp, lib_path)
        for o in objs:
            os.remove(o)
        with open(os.path.join(OUT_DIR, "build_debug.hash" if debug else "build.hash"), "w") as f:
            f.write(_source_hash())
        return lib_path


def lib() -> ctypes.CDLL:
    global _lib
    if _lib is None:
        if not is_current():
            build()
        _lib = ctypes.CDLL(LIB_PATH)
    return _lib


_debug_lib = None


def debug_lib() -> ctypes.CDLL:
    """The -DSSM_DEBUG_BOUNDS build (built on first use), for tests and for chasing a suspected bad index."""
    global _debug_lib
    if _debug_lib is None:
        if not is_current(debug=True):
            build(debug=True)
        _debug_lib = ctypes.CDLL(DEBUG_LIB_PATH)
    return _debug_lib


def debug_bounds(library: ctypes.CDLL, reset: bool = True):
    """First failed index check of each source file since the last reset: {file: (code, line, index, limit)} for the
    files that recorded one (empty dict: all checks passed; always empty for the regular build)."""
    out = {}
    for name in ("elementwise", "comm", "decode"):
        rec = (ctypes.c_int * 4)()
        fn = getattr(library, f"ssm_debug_bounds_{name}")
        fn.restype = ctypes.c_int
        code = fn(rec, int(reset))
        if code != 0:
            raise RuntimeError(f"reading the debug record of {name} failed with cudaError {code}")
        if rec[0] != 0:
            out[name] = tuple(rec)
    return out


def check(code: int, what: str) -> None:
    if code != 0:
        raise RuntimeError(f"{what} failed with code {code} (negative: argument check; positive: cudaError)")
