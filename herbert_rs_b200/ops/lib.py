"""Building and loading the kernel library (`libherbert_b200.so`).

The CUDA sources under `csrc/` are compiled for sm_100a with nvcc into one shared library
that is loaded through ctypes.  The library is built in-tree (`herbert_rs_b200/_build/`) the
first time it is needed and again whenever a source or a flag changes.  There is no fallback:
if the library cannot be built or loaded, every op raises `BackendError`.
"""

from __future__ import annotations

import concurrent.futures
import ctypes
import hashlib
import os
import shutil
import subprocess
import sys
import tempfile
import threading
import time

from ..errors import BackendError

_HERE = os.path.dirname(os.path.abspath(__file__))
CSRC = os.path.join(os.path.dirname(_HERE), "csrc")
LIB_NAME = "libherbert_b200.so"
NVCC_FLAGS = [
    "-std=c++17", "-O3", "-gencode", "arch=compute_100a,code=sm_100a", "-lineinfo",
    "-Xcompiler", "-fPIC",
]

_lock = threading.Lock()
_lib = None


def _log(msg: str) -> None:
    print(f"[herbert-b200] {msg}", file=sys.stderr, flush=True)


def _sources() -> list:
    return sorted(f for f in os.listdir(CSRC) if f.endswith(".cu"))


def _build_key() -> str:
    h = hashlib.sha256()
    for f in sorted(os.listdir(CSRC)):
        if f.endswith((".cu", ".cuh", ".h")):
            h.update(f.encode())
            with open(os.path.join(CSRC, f), "rb") as fh:
                h.update(fh.read())
    h.update(" ".join(NVCC_FLAGS).encode())
    return h.hexdigest()[:20]


def _find_nvcc() -> str:
    for cand in (os.environ.get("NVCC"), shutil.which("nvcc"), "/usr/local/cuda/bin/nvcc"):
        if cand and os.path.exists(cand):
            return cand
    raise BackendError("nvcc not found: the sm_100a kernel library cannot be built")


def _build_dirs() -> list:
    dirs = [os.path.join(os.path.dirname(_HERE), "_build")]
    uid = os.getuid() if hasattr(os, "getuid") else 0
    dirs.append(os.path.join(tempfile.gettempdir(), f"herbert_b200_build_{uid}"))
    return dirs


def _compile_one(nvcc: str, src: str, obj: str) -> None:
    cmd = [nvcc, *NVCC_FLAGS, "-I", CSRC, "-c", os.path.join(CSRC, src), "-o", obj]
    r = subprocess.run(cmd, stdout=subprocess.PIPE, stderr=subprocess.STDOUT, text=True)
    if r.returncode != 0:
        raise BackendError(f"nvcc failed on {src}:\n{r.stdout}")


def build(verbose: bool = True) -> str:
    """Compile every kernel for sm_100a (if not already built for these sources); return the path."""
    key = _build_key()
    last_err = None
    for d in _build_dirs():
        lib = os.path.join(d, LIB_NAME)
        keyfile = os.path.join(d, "build_key.txt")
        try:
            if os.path.exists(lib) and os.path.exists(keyfile) and open(keyfile).read().strip() == key:
                return lib
        except OSError:
            pass
        try:
            os.makedirs(d, exist_ok=True)
            probe = os.path.join(d, f".w{os.getpid()}")
            open(probe, "w").close()
            os.remove(probe)
        except OSError as e:
            last_err = e
            continue
        nvcc = _find_nvcc()
        srcs = _sources()
        if verbose:
            _log(f"compiling {len(srcs)} CUDA sources for sm_100a into {d} (first call only)")
        t0 = time.time()
        objs = [os.path.join(d, s[:-3] + f".{key}.o") for s in srcs]
        done = 0
        with concurrent.futures.ThreadPoolExecutor(max_workers=min(8, os.cpu_count() or 2)) as pool:
            futs = {pool.submit(_compile_one, nvcc, s, o): s for s, o in zip(srcs, objs)}
            pending = set(futs)
            while pending:
                finished, pending = concurrent.futures.wait(pending, timeout=10.0)
                for f in finished:
                    f.result()
                    done += 1
                    if verbose:
                        _log(f"compiled {futs[f]} ({done}/{len(srcs)}, {time.time() - t0:.0f} s)")
                if pending and not finished and verbose:
                    _log(f"still compiling ({done}/{len(srcs)} done, {time.time() - t0:.0f} s)")
        tmp = lib + f".tmp{os.getpid()}"
        r = subprocess.run([nvcc, "-shared", "-o", tmp, *objs, "-lcudart"],
                           stdout=subprocess.PIPE, stderr=subprocess.STDOUT, text=True)
        if r.returncode != 0:
            raise BackendError(f"linking {LIB_NAME} failed:\n{r.stdout}")
        os.replace(tmp, lib)
        with open(keyfile, "w") as f:
            f.write(key)
        for o in objs:
            try:
                os.remove(o)
            except OSError:
                pass
        if verbose:
            _log(f"built {lib} in {time.time() - t0:.0f} s")
        return lib
    raise BackendError(f"no writable place to build the kernel library: {last_err}")


def load():
    """The loaded library (built first if needed).  Raises BackendError; never falls back."""
    global _lib
    if _lib is not None:
        return _lib
    with _lock:
        if _lib is not None:
            return _lib
        path = build()
        try:
            lib = ctypes.CDLL(path)
        except OSError as e:
            raise BackendError(f"cannot load {path}: {e}") from e
        lib.hb_last_error.restype = ctypes.c_char_p
        _lib = lib
        return _lib


def last_error() -> str:
    return load().hb_last_error().decode("utf-8", "replace")
