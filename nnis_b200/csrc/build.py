"""Builds the CUDA kernels for sm_100a into one shared library and loads it.

The sources are plain ``.cu`` files with C entry points; they include no torch
header, so each compiles in seconds.  ``nvcc`` writes objects and the library
into ``_build/`` beside the sources; a stamp of the sources' content decides
whether the library on disk is current.  Nothing is compiled when it is.  While
compiling, a line goes to stderr for every finished file and every few seconds
in between.

NNIS compiles its kernels at run time as well, with NVRTC for the device it
finds (crates/nnis-jit/src/program.rs:27-66); here the target is fixed.
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

HERE = os.path.dirname(os.path.abspath(__file__))
BUILD_DIR = os.path.join(HERE, "_build")
LIB_NAME = "libnnis_b200_kernels.so"
ARCH_FLAGS = ["-gencode", "arch=compute_100a,code=sm_100a"]
NVCC_FLAGS = ["-O3", "-std=c++17", "-lineinfo", "-Xcompiler", "-fPIC", "-Xcompiler",
              "-fvisibility=hidden", "--expt-relaxed-constexpr"]


class KernelBuildError(RuntimeError):
    pass


def sources() -> List[str]:
    return sorted(f for f in os.listdir(HERE) if f.endswith(".cu"))


def _headers() -> List[str]:
    return sorted(f for f in os.listdir(HERE) if f.endswith((".cuh", ".h")))


def _stamp() -> str:
    h = hashlib.sha256()
    h.update(" ".join(ARCH_FLAGS + NVCC_FLAGS).encode())
    for name in sources() + _headers():
        h.update(name.encode())
        with open(os.path.join(HERE, name), "rb") as f:
            h.update(f.read())
    return h.hexdigest()


def find_nvcc() -> str:
    for candidate in (os.environ.get("NNIS_NVCC"), shutil.which("nvcc"),
                      os.path.join(os.environ.get("CUDA_HOME", "/usr/local/cuda"), "bin", "nvcc"),
                      "/usr/local/cuda/bin/nvcc"):
        if candidate and os.path.isfile(candidate) and os.access(candidate, os.X_OK):
            return candidate
    raise KernelBuildError("nvcc not found (set NNIS_NVCC or CUDA_HOME); the kernels cannot be "
                           "compiled and there is no fallback")


def _say(text: str) -> None:
    print(f"[nnis_b200] {text}", file=sys.stderr, flush=True)


def library_path() -> str:
    return os.path.join(BUILD_DIR, LIB_NAME)


def is_current() -> bool:
    stamp_file = os.path.join(BUILD_DIR, "stamp")
    if not (os.path.isfile(library_path()) and os.path.isfile(stamp_file)):
        return False
    with open(stamp_file) as f:
        return f.read().strip() == _stamp()


def build(force: bool = False, verbose_ptxas: bool = False) -> str:
    """Compile what is out of date; returns the library's path."""
    if not force and is_current():
        return library_path()
    nvcc = find_nvcc()
    try:
        os.makedirs(BUILD_DIR, exist_ok=True)
        probe = os.path.join(BUILD_DIR, f".probe{os.getpid()}")
        open(probe, "w").close()
        os.remove(probe)
    except OSError as e:
        raise KernelBuildError(f"cannot write the build folder {BUILD_DIR}: {e}") from None
    names = sources()
    _say(f"compiling {len(names)} CUDA files for sm_100a with {nvcc} (first use only)")
    started = time.time()
    done = threading.Event()

    def heartbeat():
        while not done.wait(10.0):
            _say(f"still compiling ({time.time() - started:.0f} s)")

    beat = threading.Thread(target=heartbeat, daemon=True)
    beat.start()

    def compile_one(name: str) -> str:
        obj = os.path.join(BUILD_DIR, name[:-3] + f".{os.getpid()}.o")
        cmd = [nvcc, *ARCH_FLAGS, *NVCC_FLAGS, "-I", HERE, "-c", os.path.join(HERE, name), "-o", obj]
        if verbose_ptxas:
            cmd.insert(1, "-Xptxas=-v")
        r = subprocess.run(cmd, stdout=subprocess.PIPE, stderr=subprocess.STDOUT, text=True)
        if r.returncode != 0:
            raise KernelBuildError(f"nvcc failed on {name}:\n{r.stdout}")
        if verbose_ptxas:
            sys.stderr.write(r.stdout)
        _say(f"compiled {name} ({time.time() - started:.0f} s)")
        return obj

    objects: List[str] = []
    try:
        with ThreadPoolExecutor(max_workers=min(8, os.cpu_count() or 2)) as pool:
            objects = list(pool.map(compile_one, names))
        tmp_lib = library_path() + f".{os.getpid()}.tmp"
        cmd = [nvcc, *ARCH_FLAGS, "-shared", "-o", tmp_lib, *objects]
        r = subprocess.run(cmd, stdout=subprocess.PIPE, stderr=subprocess.STDOUT, text=True)
        if r.returncode != 0:
            raise KernelBuildError(f"linking the kernels failed:\n{r.stdout}")
        os.replace(tmp_lib, library_path())
        with open(os.path.join(BUILD_DIR, "stamp"), "w") as f:
            f.write(_stamp())
    finally:
        done.set()
        for obj in objects:
            try:
                os.remove(obj)
            except OSError:
                pass
    _say(f"kernels built in {time.time() - started:.0f} s")
    return library_path()


_lib: Optional[ctypes.CDLL] = None
_lock = threading.Lock()


def load() -> ctypes.CDLL:
    """The loaded kernel library; builds it first when needed.  Fails loudly:
    there is no other implementation to fall back to."""
    global _lib
    with _lock:
        if _lib is None:
            path = build()
            try:
                _lib = ctypes.CDLL(path)
            except OSError as e:
                raise KernelBuildError(f"cannot load {path}: {e}") from None
        return _lib
