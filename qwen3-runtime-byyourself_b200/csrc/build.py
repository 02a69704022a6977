"""Compiles the CUDA sources of this folder for sm_100a and loads them with ctypes.

Each `.cu` file becomes one shared library, compiled the first time one of its entry
points is needed: a model only pays for the kernels it uses (an attention kernel is
compiled for the model's own head size through `-D` definitions).  The library's name
carries a hash of the source, the files it includes, the definitions and the flags, so a
stale build is never loaded.  Libraries are kept under `csrc/_build/` inside the
package when that folder can be written, else under a per-user temporary folder; no
home directory is needed.  There is no fallback: without nvcc, or when the compile
fails, the caller gets a `KernelBuildError`.
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
from typing import Dict, Iterable, Optional, Tuple

HERE = os.path.dirname(os.path.abspath(__file__))
ARCH_FLAGS = ["-gencode", "arch=compute_100a,code=sm_100a"]
BASE_FLAGS = ["-O3", "-std=c++17", "-lineinfo", "--shared", "-Xcompiler", "-fPIC", "-Xcompiler", "-fvisibility=hidden",
              "--expt-relaxed-constexpr"]

def _page_define() -> str:
    """The cache's page size, handed to every kernel source: one constant, in cache/book.py."""
    from ..cache.book import PAGE_TOKENS
    return f"Q3_PAGE_TOKENS={PAGE_TOKENS}"


_loaded: Dict[Tuple[str, Tuple[str, ...]], ctypes.CDLL] = {}
_lock = threading.Lock()


class KernelBuildError(RuntimeError):
    """The CUDA extension could not be built or loaded."""


def find_nvcc() -> str:
    for candidate in (os.environ.get("NVCC"),
                      os.path.join(os.environ.get("CUDA_HOME", ""), "bin", "nvcc") if os.environ.get("CUDA_HOME") else None,
                      shutil.which("nvcc"), "/usr/local/cuda/bin/nvcc"):
        if candidate and os.path.isfile(candidate) and os.access(candidate, os.X_OK):
            return candidate
    raise KernelBuildError("nvcc not found (looked at $NVCC, $CUDA_HOME/bin, PATH, /usr/local/cuda/bin); "
                           "the kernels of this library have to be compiled for sm_100a")


def build_dir() -> str:
    override = os.environ.get("QWEN3_B200_BUILD_DIR")
    candidates = [override] if override else []
    candidates.append(os.path.join(HERE, "_build"))
    candidates.append(os.path.join(tempfile.gettempdir(), f"qwen3_b200_build_{os.getuid()}"))
    for path in candidates:
        try:
            os.makedirs(path, exist_ok=True)
            probe = os.path.join(path, f".probe_{os.getpid()}")
            with open(probe, "w"):
                pass
            os.remove(probe)
            return path
        except OSError:
            continue
    raise KernelBuildError(f"no writable build folder among {candidates}")


def _sources_of(source: str):
    """`source` and every file of this folder that it includes, directly or not."""
    seen, todo = [], [source]
    while todo:
        name = todo.pop()
        path = os.path.join(HERE, name)
        if name in seen or not os.path.isfile(path):
            continue
        seen.append(name)
        with open(path, "r", encoding="utf-8") as f:
            for line in f:
                line = line.strip()
                if line.startswith("#include \""):
                    todo.append(line.split("\"")[1])
    return sorted(seen)


def _digest(source: str, defines: Tuple[str, ...], extra: Tuple[str, ...]) -> str:
    h = hashlib.sha256()
    for name in _sources_of(source):
        with open(os.path.join(HERE, name), "rb") as f:
            h.update(f.read())
    h.update(repr((defines, extra, ARCH_FLAGS, BASE_FLAGS, _page_define())).encode())
    return h.hexdigest()[:12]


def library_path(source: str, defines: Iterable[str] = (), extra_flags: Iterable[str] = ()) -> str:
    defines, extra = tuple(defines), tuple(extra_flags)
    stem = os.path.splitext(os.path.basename(source))[0]
    return os.path.join(build_dir(), f"libq3_{stem}_{_digest(source, defines, extra)}.so")


def compile_library(source: str, defines: Iterable[str] = (), extra_flags: Iterable[str] = (),
                    verbose: bool = True) -> str:
    """Compile `source` (a file name inside this folder) if its library is not there yet; return the path."""
    defines, extra = tuple(defines), tuple(extra_flags)
    out = library_path(source, defines, extra)
    if os.path.isfile(out):
        return out
    nvcc = find_nvcc()
    tmp = f"{out}.{os.getpid()}.tmp"
    cmd = [nvcc, *ARCH_FLAGS, *BASE_FLAGS, *extra, f"-D{_page_define()}", *[f"-D{d}" for d in defines], "-I", HERE,
           "-o", tmp, os.path.join(HERE, source)]
    label = source + (" [" + " ".join(defines) + "]" if defines else "")
    if verbose:
        print(f"[qwen3_b200] compiling {label} for sm_100a ...", file=sys.stderr, flush=True)
    start = time.time()
    proc = subprocess.Popen(cmd, stdout=subprocess.PIPE, stderr=subprocess.STDOUT, text=True)
    done = threading.Event()

    def heartbeat():
        while not done.wait(10.0):
            if verbose:
                print(f"[qwen3_b200]   still compiling {label} ({time.time() - start:.0f} s)", file=sys.stderr, flush=True)

    beat = threading.Thread(target=heartbeat, daemon=True)
    beat.start()
    try:
        log, _ = proc.communicate()
    finally:
        done.set()
    if proc.returncode != 0:
        if os.path.exists(tmp):
            os.remove(tmp)
        raise KernelBuildError(f"nvcc failed on {label}:\n{' '.join(cmd)}\n{log}")
    os.replace(tmp, out)  # atomic: concurrent processes may build the same file
    if verbose:
        print(f"[qwen3_b200]   built {os.path.basename(out)} in {time.time() - start:.1f} s", file=sys.stderr, flush=True)
    return out


def load_library(source: str, defines: Iterable[str] = (), extra_flags: Iterable[str] = ()) -> ctypes.CDLL:
    key = (source, tuple(defines) + ("|",) + tuple(extra_flags))
    with _lock:
        lib = _loaded.get(key)
        if lib is None:
            path = compile_library(source, defines, extra_flags)
            try:
                lib = ctypes.CDLL(path)
            except OSError as e:
                raise KernelBuildError(f"cannot load {path}: {e}") from None
            _loaded[key] = lib
        return lib


def loaded_libraries():
    return [lib._name for lib in _loaded.values()]
