"""Builds and loads the library of hand-written sm_100a kernels (csrc/*.cu).

The kernels are compiled with nvcc for ``sm_100a`` into one shared library with C entry
points and loaded with ctypes: no Python binding code is compiled, so a first call in a fresh
checkout takes about a minute. The library is kept inside the package (``_lib/``) when that
folder can be written, else under the user's temporary folder; it is rebuilt when a source file
or a flag changes. There is no fallback: without nvcc, or if compilation fails, loading raises.
Environment: ``PTB200_NVCC`` (the compiler), ``PTB200_BUILD_DIR`` (where the library goes),
``PTB200_NVCC_EXTRA`` (more flags, a ``-D`` for a trial build; they are part of the fingerprint).
"""
from __future__ import annotations

import ctypes
import hashlib
import os
import shutil
import subprocess
import sys
import tempfile
import threading
import time
from concurrent.futures import ThreadPoolExecutor
from typing import List, Optional

from .utils import logging as log

_logger = log.get_logger(__name__)
_HERE = os.path.dirname(os.path.abspath(__file__))
CSRC = os.path.join(_HERE, "csrc")
LIB_NAME = "libptb200_kernels.so"
# precise math (no --use_fast_math): float32 paths must round as IEEE says
NVCC_FLAGS = ["-gencode", "arch=compute_100a,code=sm_100a", "-O3", "-std=c++17", "-lineinfo",
              "-Xcompiler", "-fPIC", "-Xcompiler", "-fvisibility=hidden"]

# more flags for nvcc from the environment (a -D for a trial build, say); part of the fingerprint
NVCC_FLAGS += [f for f in os.environ.get("PTB200_NVCC_EXTRA", "").split() if f]

_lock = threading.Lock()
_lib: Optional[ctypes.CDLL] = None


class NativeBuildError(RuntimeError):
    """The kernel library could not be compiled or loaded."""


def _sources() -> List[str]:
    return sorted(os.path.join(CSRC, f) for f in os.listdir(CSRC) if f.endswith(".cu"))


def _headers() -> List[str]:
    return sorted(os.path.join(CSRC, f) for f in os.listdir(CSRC) if f.endswith((".cuh", ".h")))


def _find_nvcc() -> str:
    for cand in (os.environ.get("PTB200_NVCC"), shutil.which("nvcc"), "/usr/local/cuda/bin/nvcc"):
        if cand and os.path.isfile(cand):
            return cand
    raise NativeBuildError("nvcc was not found (looked at $PTB200_NVCC, PATH and /usr/local/cuda/bin): the "
                           "sm_100a kernels cannot be compiled and there is no other code path")


def _fingerprint() -> str:
    h = hashlib.sha256()
    h.update(" ".join(NVCC_FLAGS).encode())
    for path in _sources() + _headers():
        h.update(os.path.basename(path).encode())
        with open(path, "rb") as f:
            h.update(f.read())
    return h.hexdigest()[:16]


def _writable_dir() -> str:
    cands = [os.environ.get("PTB200_BUILD_DIR"), os.path.join(_HERE, "_lib"),
             os.path.join(tempfile.gettempdir(), f"ptb200_kernels_{os.getuid()}")]
    for d in cands:
        if not d:
            continue
        try:
            os.makedirs(d, exist_ok=True)
            probe = os.path.join(d, f".probe_{os.getpid()}")
            with open(probe, "w") as f:
                f.write("x")
            os.remove(probe)
            return d
        except OSError:
            continue
    raise NativeBuildError("no writable folder for the compiled kernel library (tried: " + ", ".join(
        c for c in cands if c) + ")")


def _say(msg: str) -> None:
    # progress of a compilation that may take a minute: shown at the default verbosity too
    log.always(_logger, msg)


def _compile_one(nvcc: str, src: str, obj: str, verbose_ptxas: bool) -> str:
    cmd = [nvcc] + NVCC_FLAGS + (["-Xptxas", "-v"] if verbose_ptxas else []) + ["-I", CSRC, "-c", src, "-o", obj]
    t0 = time.time()
    proc = subprocess.run(cmd, capture_output=True, text=True)
    if proc.returncode != 0:
        raise NativeBuildError(f"nvcc failed on {os.path.basename(src)}:\n{proc.stdout}\n{proc.stderr}")
    _say(f"compiled {os.path.basename(src)} in {time.time() - t0:.0f} s")
    return proc.stderr


def build(force: bool = False, verbose_ptxas: bool = False) -> str:
    """Compile the library if it is missing or stale; returns its path."""
    fp = _fingerprint()
    for d in (os.environ.get("PTB200_BUILD_DIR"), os.path.join(_HERE, "_lib"),
              os.path.join(tempfile.gettempdir(), f"ptb200_kernels_{os.getuid()}")):
        if d and not force:
            lib, stamp = os.path.join(d, LIB_NAME), os.path.join(d, "fingerprint.txt")
            try:
                if os.path.isfile(lib) and open(stamp).read().strip() == fp:
                    return lib
            except OSError:
                pass
    out_dir = _writable_dir()
    nvcc = _find_nvcc()
    srcs = _sources()
    _say(f"compiling {len(srcs)} CUDA files for sm_100a into {out_dir} (first use; about a minute)")
    obj_dir = os.path.join(out_dir, f"obj_{os.getpid()}")
    os.makedirs(obj_dir, exist_ok=True)
    logs = []
    try:
        objs = [os.path.join(obj_dir, os.path.basename(s)[:-3] + ".o") for s in srcs]
        with ThreadPoolExecutor(max_workers=min(8, len(srcs))) as pool:
            futs = [pool.submit(_compile_one, nvcc, s, o, verbose_ptxas) for s, o in zip(srcs, objs)]
            for f in futs:
                logs.append(f.result())
        tmp_lib = os.path.join(obj_dir, LIB_NAME)
        link = [nvcc, "-shared", "-gencode", "arch=compute_100a,code=sm_100a", "-o", tmp_lib] + objs
        proc = subprocess.run(link, capture_output=True, text=True)
        if proc.returncode != 0:
            raise NativeBuildError(f"linking the kernel library failed:\n{proc.stdout}\n{proc.stderr}")
        lib = os.path.join(out_dir, LIB_NAME)
        os.replace(tmp_lib, lib)
        with open(os.path.join(out_dir, "fingerprint.txt"), "w") as f:
            f.write(fp + "\n")
        if verbose_ptxas:
            with open(os.path.join(out_dir, "ptxas.log"), "w") as f:
                f.write("\n".join(logs))
        _say("kernel library ready")
        return lib
    finally:
        shutil.rmtree(obj_dir, ignore_errors=True)


def library() -> ctypes.CDLL:
    """The loaded kernel library (built on first use)."""
    global _lib
    if _lib is None:
        with _lock:
            if _lib is None:
                path = build()
                try:
                    _lib = ctypes.CDLL(path)
                except OSError as e:
                    raise NativeBuildError(f"could not load {path}: {e}") from e
    return _lib
