"""Compiles the engine's CUDA sources for sm_100a and loads them.

Every ``.cu`` file becomes a shared library of its own (``_build/<name>.<hash>.so`` beside the
sources), compiled on first use with ``nvcc`` and cached by a hash of the source, the shared
header and the flags.  The entry points are plain C symbols called through ``ctypes``; there is no
fallback: if a library cannot be built or loaded the caller gets :class:`KernelBuildError`.

While a compile runs, a line is printed to stderr every few seconds so that a first call on a
fresh checkout does not look hung.
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
from typing import Dict, Iterable, List, Optional

HERE = os.path.dirname(os.path.abspath(__file__))
ARCH_FLAGS = ["-gencode", "arch=compute_100a,code=sm_100a"]
BASE_FLAGS = ["-O3", "-std=c++17", "-lineinfo", "--shared", "-Xcompiler", "-fPIC,-fvisibility=hidden",
              "--expt-relaxed-constexpr"]
SHARED_HEADERS = ["common.cuh"]

# every library of the engine; build_all() compiles them all
SOURCES = ["elementwise", "rope_kv", "attention_generic", "gemm_simt", "sampling", "gemm_skinny", "attention_mma", "prefetch", "gemm_tcgen05",
           "attention_tc", "gemm_stream"]
# libraries only the bfloat16 serving path uses
BF16_SOURCES: List[str] = ["gemm_skinny", "attention_mma", "prefetch", "gemm_tcgen05", "attention_tc", "gemm_stream"]
# extra link flags per source
EXTRA_FLAGS: Dict[str, List[str]] = {}
# extra compiler flags for every source, from the environment (e.g. "-DIIAN_SOMETHING=1" to build a variant of a
# kernel for a measurement); they are part of the cache key, so variants live side by side
ENV_FLAGS: List[str] = os.environ.get("IIAN_NVCC_FLAGS", "").split()


class KernelBuildError(RuntimeError):
    pass


_lock = threading.Lock()
_dir_lock = threading.Lock()
_loaded: Dict[str, ctypes.CDLL] = {}


def _nvcc() -> str:
    for cand in (os.environ.get("NVCC"), shutil.which("nvcc"), "/usr/local/cuda/bin/nvcc"):
        if cand and os.path.isfile(cand):
            return cand
    raise KernelBuildError("nvcc not found (set NVCC or put it on PATH); the engine has no path without its CUDA kernels")


_build_dir: Optional[str] = None


def build_dir() -> str:
    """``_build`` beside the sources; a per-user temporary folder if the tree is read-only."""
    global _build_dir
    if _build_dir is None:
        with _dir_lock:
            if _build_dir is None:
                _build_dir = _pick_build_dir()
    return _build_dir


def _pick_build_dir() -> str:
    d = os.environ.get("IIAN_B200_BUILD_DIR") or os.path.join(HERE, "_build")
    try:
        os.makedirs(d, exist_ok=True)
        probe = os.path.join(d, f".w{os.getpid()}")
        with open(probe, "w"):
            pass
        os.remove(probe)
        return d
    except OSError:
        d = os.path.join(tempfile.gettempdir(), f"iian_b200_build_{os.getuid()}")
        os.makedirs(d, exist_ok=True)
        return d


def _source_hash(name: str) -> str:
    h = hashlib.sha256()
    for fn in [f"{name}.cu"] + SHARED_HEADERS:
        p = os.path.join(HERE, fn)
        if os.path.isfile(p):
            with open(p, "rb") as f:
                h.update(f.read())
    extra = os.path.join(HERE, f"{name}.cuh")
    if os.path.isfile(extra):
        with open(extra, "rb") as f:
            h.update(f.read())
    h.update(" ".join(ARCH_FLAGS + BASE_FLAGS + EXTRA_FLAGS.get(name, []) + ENV_FLAGS).encode())
    return h.hexdigest()[:16]


def library_path(name: str) -> str:
    return os.path.join(build_dir(), f"{name}.{_source_hash(name)}.so")


def _compile(name: str, verbose: bool = True) -> str:
    src = os.path.join(HERE, f"{name}.cu")
    if not os.path.isfile(src):
        raise KernelBuildError(f"no such kernel source: {src}")
    out = library_path(name)
    if os.path.isfile(out):
        return out
    tmp = f"{out}.{os.getpid()}.{threading.get_ident()}.tmp"
    cmd = [_nvcc()] + ARCH_FLAGS + BASE_FLAGS + EXTRA_FLAGS.get(name, []) + ENV_FLAGS + ["-I", HERE, "-o", tmp, src]
    t0 = time.time()
    if verbose:
        print(f"[iian_b200] compiling {name}.cu for sm_100a ...", file=sys.stderr, flush=True)
    proc = subprocess.Popen(cmd, stdout=subprocess.PIPE, stderr=subprocess.STDOUT, text=True)
    done = threading.Event()

    def ticker():
        while not done.wait(5.0):
            if verbose:
                print(f"[iian_b200] still compiling {name}.cu ({time.time() - t0:.0f} s)", file=sys.stderr, flush=True)

    th = threading.Thread(target=ticker, daemon=True)
    th.start()
    try:
        log, _ = proc.communicate()
    finally:
        done.set()
    if proc.returncode != 0:
        if os.path.exists(tmp):
            os.remove(tmp)
        raise KernelBuildError(f"nvcc failed for {name}.cu (exit {proc.returncode}):\n{' '.join(cmd)}\n{log}")
    os.replace(tmp, out)
    # drop stale builds of the same source (variants built with extra flags are kept beside the default)
    prefix = f"{name}."
    for fn in ([] if ENV_FLAGS else os.listdir(os.path.dirname(out))):
        if fn.startswith(prefix) and fn.endswith(".so") and os.path.join(os.path.dirname(out), fn) != out:
            try:
                os.remove(os.path.join(os.path.dirname(out), fn))
            except OSError:
                pass
    if verbose:
        print(f"[iian_b200] built {os.path.basename(out)} in {time.time() - t0:.1f} s", file=sys.stderr, flush=True)
    return out


# ---- the host runtime (block pool, cache manager, scheduler, step packing): plain C++17, no CUDA --------
HOST_NAME = "host"
HOST_DIR = os.path.join(HERE, "host")
INCLUDE_DIR = os.path.join(os.path.dirname(os.path.dirname(HERE)), "include")
HOST_FLAGS = ["-O2", "-std=c++17", "-shared", "-fPIC", "-Wall"]


def _host_sources() -> List[str]:
    return sorted(os.path.join(HOST_DIR, f) for f in os.listdir(HOST_DIR) if f.endswith(".cc"))


def _host_hash() -> str:
    h = hashlib.sha256()
    headers = sorted(os.path.join(INCLUDE_DIR, "iian_b200", f) for f in os.listdir(os.path.join(INCLUDE_DIR, "iian_b200")))
    for p in _host_sources() + headers:
        with open(p, "rb") as f:
            h.update(f.read())
    h.update(" ".join(HOST_FLAGS).encode())
    return h.hexdigest()[:16]


def _cxx() -> str:
    for cand in (os.environ.get("CXX"), shutil.which("g++"), shutil.which("c++"), shutil.which("clang++")):
        if cand and os.path.isfile(cand):
            return cand
    raise KernelBuildError("no C++ compiler found (set CXX or put g++ on PATH); the host runtime is native code")


def _compile_host(verbose: bool = True) -> str:
    out = os.path.join(build_dir(), f"{HOST_NAME}.{_host_hash()}.so")
    if os.path.isfile(out):
        return out
    tmp = f"{out}.{os.getpid()}.{threading.get_ident()}.tmp"
    cmd = [_cxx()] + HOST_FLAGS + ["-I", INCLUDE_DIR, "-o", tmp] + _host_sources()
    t0 = time.time()
    if verbose:
        print("[iian_b200] compiling the host runtime ...", file=sys.stderr, flush=True)
    proc = subprocess.run(cmd, stdout=subprocess.PIPE, stderr=subprocess.STDOUT, text=True)
    if proc.returncode != 0:
        if os.path.exists(tmp):
            os.remove(tmp)
        raise KernelBuildError(f"compiling the host runtime failed (exit {proc.returncode}):\n{' '.join(cmd)}\n{proc.stdout}")
    os.replace(tmp, out)
    for fn in os.listdir(os.path.dirname(out)):
        if fn.startswith(f"{HOST_NAME}.") and fn.endswith(".so") and os.path.join(os.path.dirname(out), fn) != out:
            try:
                os.remove(os.path.join(os.path.dirname(out), fn))
            except OSError:
                pass
    if verbose:
        print(f"[iian_b200] built {os.path.basename(out)} in {time.time() - t0:.1f} s", file=sys.stderr, flush=True)
    return out


# ---- the native step function and engine loop: C++17 host code that calls CUDA's runtime and cuBLAS and opens the
# kernel libraries above with dlopen; it carries a copy of the host runtime's sources (it packs decode steps itself) ----
ENGINE_NAME = "engine"
ENGINE_DIR = os.path.join(HERE, "engine")
ENGINE_FLAGS = ["-shared", "-std=c++17", "-O2", "-Xcompiler", "-fPIC", "-Wno-deprecated-gpu-targets"]
ENGINE_LIBS = ["-lcublas", "-ldl"]


def _engine_sources() -> List[str]:
    return sorted(os.path.join(ENGINE_DIR, f) for f in os.listdir(ENGINE_DIR) if f.endswith(".cc")) + _host_sources()


def _engine_hash() -> str:
    h = hashlib.sha256()
    headers = sorted(os.path.join(INCLUDE_DIR, "iian_b200", f) for f in os.listdir(os.path.join(INCLUDE_DIR, "iian_b200")))
    for p in _engine_sources() + headers:
        with open(p, "rb") as f:
            h.update(f.read())
    h.update(" ".join(ENGINE_FLAGS + ENGINE_LIBS).encode())
    return h.hexdigest()[:16]


def _compile_engine(verbose: bool = True) -> str:
    out = os.path.join(build_dir(), f"{ENGINE_NAME}.{_engine_hash()}.so")
    if os.path.isfile(out):
        return out
    tmp = f"{out}.{os.getpid()}.{threading.get_ident()}.tmp"
    cmd = [_nvcc()] + ENGINE_FLAGS + ["-I", INCLUDE_DIR, "-o", tmp] + _engine_sources() + ENGINE_LIBS
    t0 = time.time()
    if verbose:
        print("[iian_b200] compiling the native engine ...", file=sys.stderr, flush=True)
    proc = subprocess.run(cmd, stdout=subprocess.PIPE, stderr=subprocess.STDOUT, text=True)
    if proc.returncode != 0:
        if os.path.exists(tmp):
            os.remove(tmp)
        raise KernelBuildError(f"compiling the native engine failed (exit {proc.returncode}):\n{' '.join(cmd)}\n{proc.stdout}")
    os.replace(tmp, out)
    for fn in os.listdir(os.path.dirname(out)):
        if fn.startswith(f"{ENGINE_NAME}.") and fn.endswith(".so") and os.path.join(os.path.dirname(out), fn) != out:
            try:
                os.remove(os.path.join(os.path.dirname(out), fn))
            except OSError:
                pass
    if verbose:
        print(f"[iian_b200] built {os.path.basename(out)} in {time.time() - t0:.1f} s", file=sys.stderr, flush=True)
    return out


def load_engine() -> ctypes.CDLL:
    """The native step function and engine loop, compiled first if needed (needs nvcc for its CUDA headers and libraries)."""
    with _lock:
        lib = _loaded.get(ENGINE_NAME)
        if lib is None:
            path = _compile_engine()
            try:
                lib = ctypes.CDLL(path)
            except OSError as e:
                raise KernelBuildError(f"cannot load {path}: {e}") from None
            _loaded[ENGINE_NAME] = lib
        return lib


def load_host() -> ctypes.CDLL:
    """The host runtime library, compiled first if needed (needs a C++ compiler, no GPU and no nvcc)."""
    with _lock:
        lib = _loaded.get(HOST_NAME)
        if lib is None:
            path = _compile_host()
            try:
                lib = ctypes.CDLL(path)
            except OSError as e:
                raise KernelBuildError(f"cannot load {path}: {e}") from None
            _loaded[HOST_NAME] = lib
        return lib


def build(names: Optional[Iterable[str]] = None, verbose: bool = True) -> List[str]:
    """Compile the named libraries (all by default), in parallel.  Needs no GPU."""
    everything = names is None
    names = list(names) if names is not None else list(SOURCES)
    with ThreadPoolExecutor(max_workers=min(8, max(1, len(names)))) as pool:
        built = list(pool.map(lambda n: _compile(n, verbose), names))
    if everything:
        built.append(_compile_host(verbose))
        built.append(_compile_engine(verbose))
    return built


def load(name: str) -> ctypes.CDLL:
    """The loaded library ``name``, compiling it first if needed."""
    with _lock:
        lib = _loaded.get(name)
        if lib is not None:
            return lib
        path = _compile(name)
        try:
            lib = ctypes.CDLL(path)
        except OSError as e:
            raise KernelBuildError(f"cannot load {path}: {e}") from None
        _loaded[name] = lib
        return lib


def preload(names: Iterable[str]) -> None:
    """Compile several libraries at once (parallel), then load them."""
    names = [n for n in names if n not in _loaded]
    if not names:
        return
    build(names)
    for n in names:
        load(n)
