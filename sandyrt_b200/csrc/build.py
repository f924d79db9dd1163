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
    "gemm_small": [],
    "attention": [],
    "attention_decode": [],
    "attention_decode_bulk": [],
    "attention_decode_mma": [],
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
    """Headers the kernel sources include (sandy_kernels.h only declares their entry points for the host library)."""
    return sorted(f for f in os.listdir(CSRC_DIR) if f.endswith((".cuh", ".h")) and f != "sandy_kernels.h")


def _source_hash(name: str) -> str:
    h = hashlib.sha256()
    for fname in [name + ".cu"] + _headers():
        with open(os.path.join(CSRC_DIR, fname), "rb") as f:
            h.update(fname.encode())
            h.update(f.read())
    h.update(" ".join(ARCH_FLAGS + NVCC_FLAGS + LIBRARIES.get(name, [])).encode())
    return h.hexdigest()


_build_dir_cache: Optional[str] = None
_build_dir_lock = threading.Lock()


def _build_dir() -> str:
    """Where the libraries are built; decided once (the probe below must not race with itself when
    several libraries are built at a time)."""
    global _build_dir_cache
    with _build_dir_lock:
        if _build_dir_cache is None:
            _build_dir_cache = _choose_build_dir()
        return _build_dir_cache


def _choose_build_dir() -> str:
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


# ---- the host library (sandyrt_b200/core/*.cpp -> libsandy_core.so) ---------------------------------
CORE_DIR = os.path.join(os.path.dirname(CSRC_DIR), "core")
CORE_NAME = "libsandy_core"
CXX_FLAGS = ["-O2", "-std=c++17", "-fPIC", "-Wall", "-Wno-unused-function"]
# -Bsymbolic: the library binds its own template instantiations (std::regex and the like) instead of
# same-named ones another library of the process may export (torch does, built against another ABI).
LINK_FLAGS = ["-Wl,-Bsymbolic"]


def _core_sources() -> List[str]:
    return sorted(f for f in os.listdir(CORE_DIR) if f.endswith(".cpp"))


def _core_hash() -> str:
    h = hashlib.sha256()
    names = sorted(f for f in os.listdir(CORE_DIR) if f.endswith((".cpp", ".h"))) 
    for fname in names:
        with open(os.path.join(CORE_DIR, fname), "rb") as f:
            h.update(fname.encode())
            h.update(f.read())
    with open(os.path.join(CSRC_DIR, "sandy_kernels.h"), "rb") as f:
        h.update(f.read())
    h.update(" ".join(CXX_FLAGS + LINK_FLAGS).encode())
    return h.hexdigest()


def core_library_path() -> str:
    return os.path.join(_build_dir(), CORE_NAME + ".so")


def core_is_current() -> bool:
    so = core_library_path()
    stamp = so + ".stamp"
    if not (os.path.isfile(so) and os.path.isfile(stamp)):
        return False
    with open(stamp) as f:
        return f.read().strip() == _core_hash()


def compile_core(verbose: bool = True) -> str:
    """Build the host library: every core/*.cpp with the C++ compiler (in parallel), linked against
    the CUDA runtime.  No device code is in it; the kernels stay in their own libraries."""
    nvcc = _find_nvcc()
    cuda_home = os.path.dirname(os.path.dirname(os.path.realpath(nvcc)))
    # the system's compiler first: it links the C++ runtime the rest of the process uses ($CXX may name a
    # toolchain with a runtime of its own, linked statically)
    cxx = os.environ.get("SANDYRT_CXX") or shutil.which("g++") or shutil.which("c++") or os.environ.get("CXX")
    if not cxx:
        raise KernelBuildError("no C++ compiler found (looked at $SANDYRT_CXX, g++, c++, $CXX); the host library cannot be built")
    so = core_library_path()
    objdir = os.path.join(_build_dir(), f"core_obj_{os.getpid()}")
    os.makedirs(objdir, exist_ok=True)
    t0 = time.time()
    if verbose:
        print(f"[sandyrt_b200] compiling the host library ({len(_core_sources())} files) ...", file=sys.stderr, flush=True)
    errors: List[str] = []
    objects: List[str] = []

    def work(src):
        obj = os.path.join(objdir, src[:-4] + ".o")
        objects.append(obj)
        cmd = [cxx] + CXX_FLAGS + ["-I", os.path.join(cuda_home, "include"), "-c", os.path.join(CORE_DIR, src), "-o", obj]
        res = subprocess.run(cmd, stdout=subprocess.PIPE, stderr=subprocess.STDOUT, cwd=CORE_DIR)
        if res.returncode != 0:
            errors.append(f"{src}:\n" + res.stdout.decode("utf-8", "replace"))

    threads = [threading.Thread(target=work, args=(s,)) for s in _core_sources()]
    for t in threads:
        t.start()
    while any(t.is_alive() for t in threads):
        for t in threads:
            t.join(timeout=5.0 / max(1, len(threads)))
        if verbose and time.time() - t0 > 5 and int(time.time() - t0) % 5 == 0:
            print(f"[sandyrt_b200]   still compiling the host library ({time.time() - t0:.0f} s)", file=sys.stderr, flush=True)
            time.sleep(1.0)
    try:
        if errors:
            raise KernelBuildError("the host library failed to compile:\n" + "\n".join(errors))
        tmp = f"{so}.{os.getpid()}.tmp"
        libdir = os.path.join(cuda_home, "lib64")
        cmd = [cxx, "-shared"] + LINK_FLAGS + ["-o", tmp] + sorted(objects) + ["-L", libdir, "-lcudart_static", "-lrt", "-lpthread", "-ldl"]
        res = subprocess.run(cmd, stdout=subprocess.PIPE, stderr=subprocess.STDOUT)
        if res.returncode != 0:
            raise KernelBuildError("the host library failed to link:\n" + res.stdout.decode("utf-8", "replace"))
        os.replace(tmp, so)
        with open(so + ".stamp", "w") as f:
            f.write(_core_hash())
    finally:
        shutil.rmtree(objdir, ignore_errors=True)
    if verbose:
        print(f"[sandyrt_b200] built {CORE_NAME}.so in {time.time() - t0:.1f} s", file=sys.stderr, flush=True)
    return so


_core: Optional[ctypes.CDLL] = None


def load_core() -> ctypes.CDLL:
    """The loaded host library, building it first if it is missing or stale."""
    global _core
    with _lock:
        if _core is not None:
            return _core
        if not core_is_current():
            compile_core()
        try:
            _core = ctypes.CDLL(core_library_path())
        except OSError as e:
            raise KernelBuildError(f"cannot load {core_library_path()}: {e}") from e
        return _core


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
    out = [library_path(n) for n in names]
    if not core_is_current():
        compile_core(verbose)
    out.append(core_library_path())
    return out
