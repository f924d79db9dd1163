"""Compiles the CUDA sources of this folder for sm_100a and loads them with ctypes.

Each `<name>.cu` becomes one shared library `_build/<name>.so`, built with plain nvcc
(no Python or torch headers are involved, so a file compiles in seconds) and exporting
`extern "C"` entry points that take raw device pointers and a stream.  A library is built
the first time something needs it, so a run compiles only what its model and dtype use.
A stamp file beside each library records a hash of the sources and flags it was built
from; a stale or missing library is rebuilt.  While nvcc runs, a progress line goes to
stderr every few seconds.

The build folder is `_build/` beside the sources when that is writable, otherwise a
per-user folder under the system's temporary directory (a read-only install).

There is no fallback: if nvcc is missing or a compile fails, loading raises
KernelBuildError, and every op of the engine fails with it.
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
from typing import Dict, List, Optional

CSRC_DIR = os.path.dirname(os.path.abspath(__file__))
ARCH_FLAGS = ["-gencode", "arch=compute_100a,code=sm_100a"]
NVCC_FLAGS = ["-O3", "-std=c++17", "-lineinfo", "--shared", "-Xcompiler", "-fPIC",
              "-Xcompiler", "-fvisibility=hidden", "--expt-relaxed-constexpr"]
# Libraries of this folder, with the extra libraries each links against.
LIBRARIES: Dict[str, List[str]] = {
    "embed": [],
    "norm": [],
    "gemm_simt": [],
    "gemm_tc": [],
    "gemm_tc2": [],
    "gemm_skinny": [],
    "attention": [],
    "attention_decode": [],
    "attention_decode_bulk": [],
    "attention_prefill": [],
    "attention_prefill_tc": [],
    "sampling": [],
}


class KernelBuildError(RuntimeError):
    pass


_loaded: Dict[str, ctypes.CDLL] = {}
_lock = threading.Lock()


def _find_nvcc() -> str:
    for cand in (os.environ.get("SANDYRT_NVCC"), shutil.which("nvcc"), "/usr/local/cuda/bin/nvcc"):
        if cand and os.path.isfile(cand) and os.access(cand, os.X_OK):
            return cand
    raise KernelBuildError("nvcc not found (looked at $SANDYRT_NVCC, PATH and /usr/local/cuda/bin); "
                           "the CUDA kernels cannot be built and there is no other path")


def _headers() -> List[str]:
    return sorted(f for f in os.listdir(CSRC_DIR) if f.endswith((".cuh", ".h")))


def _source_hash(name: str) -> str:
    h = hashlib.sha256()
    for fname in [name + ".cu"] + _headers():
        with open(os.path.join(CSRC_DIR, fname), "rb") as f:
            h.update(fname.encode())
            h.update(f.read())
    h.update(" ".join(ARCH_FLAGS + NVCC_FLAGS + LIBRARIES.get(name, [])).encode())
    return h.hexdigest()


def _build_dir() -> str:
    env = os.environ.get("SANDYRT_BUILD_DIR")
    if env:
        os.makedirs(env, exist_ok=True)
        return env
    local = os.path.join(CSRC_DIR, "_build")
    try:
        os.makedirs(local, exist_ok=True)
        probe = os.path.join(local, f".probe{os.getpid()}")
        with open(probe, "w"):
            pass
        os.remove(probe)
        return local
    except OSError:
        d = os.path.join(tempfile.gettempdir(), f"sandyrt_b200_build_{os.getuid()}")
        os.makedirs(d, exist_ok=True)
        return d


def library_path(name: str) -> str:
    return os.path.join(_build_dir(), name + ".so")


def is_current(name: str) -> bool:
    so = library_path(name)
    stamp = so + ".stamp"
    if not (os.path.isfile(so) and os.path.isfile(stamp)):
        return False
    with open(stamp) as f:
        return f.read().strip() == _source_hash(name)


def compile_library(name: str, verbose: bool = True) -> str:
    """Build `<name>.cu` into its shared library (unconditionally) and return the path."""
    if name not in LIBRARIES:
        raise KernelBuildError(f"no such kernel library: {name}")
    nvcc = _find_nvcc()
    so = library_path(name)
    tmp = f"{so}.{os.getpid()}.tmp"
    cmd = [nvcc] + ARCH_FLAGS + NVCC_FLAGS + ["-o", tmp, os.path.join(CSRC_DIR, name + ".cu")] + LIBRARIES[name]
    env = dict(os.environ)
    # nvcc writes its intermediates to TMPDIR; keep it somewhere that surely exists
    env.setdefault("TMPDIR", tempfile.gettempdir())
    t0 = time.time()
    if verbose:
        print(f"[sandyrt_b200] compiling {name}.cu for sm_100a ...", file=sys.stderr, flush=True)
    proc = subprocess.Popen(cmd, stdout=subprocess.PIPE, stderr=subprocess.STDOUT, env=env, cwd=CSRC_DIR)
    out_chunks: List[bytes] = []
    reader = threading.Thread(target=lambda: out_chunks.append(proc.stdout.read()), daemon=True)
    reader.start()
    while True:
        try:
            proc.wait(timeout=5.0)
            break
        except subprocess.TimeoutExpired:
            if verbose:
                print(f"[sandyrt_b200]   still compiling {name}.cu ({time.time() - t0:.0f} s)",
                      file=sys.stderr, flush=True)
    reader.join()
    output = b"".join(out_chunks).decode("utf-8", "replace")
    if proc.returncode != 0:
        try:
            os.remove(tmp)
        except OSError:
            pass
        raise KernelBuildError(f"nvcc failed for {name}.cu (exit {proc.returncode}):\n{output}")
    os.replace(tmp, so)
    with open(so + ".stamp", "w") as f:
        f.write(_source_hash(name))
    if verbose:
        print(f"[sandyrt_b200] built {name}.so in {time.time() - t0:.1f} s", file=sys.stderr, flush=True)
    return so


def load_library(name: str) -> ctypes.CDLL:
    """The loaded library `name`, building it first if it is missing or stale."""
    with _lock:
        lib = _loaded.get(name)
        if lib is not None:
            return lib
        if not is_current(name):
            compile_library(name)
        try:
            lib = ctypes.CDLL(library_path(name))
        except OSError as e:
            raise KernelBuildError(f"cannot load {library_path(name)}: {e}") from e
        _loaded[name] = lib
        return lib


def build_all(verbose: bool = True, names: Optional[List[str]] = None) -> List[str]:
    """Build every library that is missing or stale (in parallel); return their paths."""
    names = [n for n in (names or list(LIBRARIES)) if os.path.isfile(os.path.join(CSRC_DIR, n + ".cu"))]
    todo = [n for n in names if not is_current(n)]
    errors: List[str] = []

    def work(n):
        try:
            compile_library(n, verbose)
        except KernelBuildError as e:  # collected, raised together below
            errors.append(str(e))

    threads = [threading.Thread(target=work, args=(n,)) for n in todo]
    for t in threads:
        t.start()
    for t in threads:
        t.join()
    if errors:
        raise KernelBuildError("\n".join(errors))
    return [library_path(n) for n in names]
