"""Compiles the CUDA sources under `csrc/` for sm_100a and loads them through their C ABI.

Every `csrc/<module>.cu` becomes one shared library `csrc/_build/<module>_<hash>.so`,
built with `nvcc -gencode arch=compute_100a,code=sm_100a`.  The hash covers the source,
the shared headers and the flags, so a library built from the same sources is found again
(also on another machine that received the tree) and a changed source is rebuilt.  A model
asks for the modules its parts need (`ensure_built([...])`), so the first call of a
program compiles what this model needs, in parallel, and prints a line now and then while
it waits.  The libraries export plain `extern "C"` functions taking device pointers,
sizes and a stream, and are bound with `ctypes`; there is no CPU fallback: a missing
compiler or a failed build raises `KernelBuildError`.

If the package folder is not writable the build goes to a per-user folder under the
system's temporary directory.

The reference compiles its `.cu` files with `nvcc -c -O3 -std=c++17 -arch=sm_86` from
build.zig:74-103 and binds them as `extern "C"` symbols from Zig
(src/backend/cuda/**/*.zig); this is the same shape for sm_100a.
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
from typing import Dict, Iterable, List

CSRC_DIR = os.path.normpath(os.path.join(os.path.dirname(os.path.abspath(__file__)), "..", "csrc"))
ARCH_FLAGS = ["-gencode", "arch=compute_100a,code=sm_100a"]
NVCC_FLAGS = ["-O3", "-std=c++17", "-lineinfo", "--shared", "-Xcompiler", "-fPIC",
              "--expt-relaxed-constexpr", "-Xcompiler", "-fvisibility=hidden"]

# Every module, with the extra link flags it needs.
MODULES: Dict[str, List[str]] = {
    "elementwise": [],
    "attn_prep": [],
    "gemm_simt": [],
    "gemv": [],
    "gemm_tc": [],
    "gemm_skinny": [],
    "gemm_rows8": [],
    "attention": [],
    "attention_decode": [],
    "attention_tc": [],
    "sampling": [],
    "runtime": [],      # host code only: cache manager, scheduler, step arrays
}


class KernelBuildError(RuntimeError):
    pass


_lock = threading.Lock()
_loaded: Dict[str, ctypes.CDLL] = {}


def register_module(name: str, link_flags: Iterable[str] = ()) -> None:
    """Add a `csrc/<name>.cu` module to the build list."""
    MODULES.setdefault(name, list(link_flags))


def _log(msg: str) -> None:
    print(f"[llmgen_b200] {msg}", file=sys.stderr, flush=True)


def find_nvcc() -> str:
    for cand in (os.environ.get("LLMGEN_NVCC"), shutil.which("nvcc"), "/usr/local/cuda/bin/nvcc"):
        if cand and os.path.isfile(cand) and os.access(cand, os.X_OK):
            return cand
    raise KernelBuildError("nvcc not found (looked at $LLMGEN_NVCC, PATH and /usr/local/cuda/bin): "
                           "the CUDA kernels cannot be built and there is no fallback")


def _headers() -> List[str]:
    return sorted(os.path.join(CSRC_DIR, f) for f in os.listdir(CSRC_DIR) if f.endswith((".cuh", ".h")))


def _source_hash(module: str) -> str:
    h = hashlib.sha256()
    for path in [os.path.join(CSRC_DIR, module + ".cu")] + _headers():
        with open(path, "rb") as f:
            h.update(os.path.basename(path).encode())
            h.update(f.read())
    h.update(" ".join(ARCH_FLAGS + NVCC_FLAGS + MODULES.get(module, [])).encode())
    return h.hexdigest()[:16]


def _build_dirs() -> List[str]:
    dirs = []
    env = os.environ.get("LLMGEN_BUILD_DIR")
    if env:
        dirs.append(env)
    dirs.append(os.path.join(CSRC_DIR, "_build"))
    uid = os.getuid() if hasattr(os, "getuid") else 0
    dirs.append(os.path.join(tempfile.gettempdir(), f"llmgen_b200_build_{uid}"))
    return dirs


_build_dir_cache: List[str] = []


def _writable_build_dir() -> str:
    if _build_dir_cache:
        return _build_dir_cache[0]
    for d in _build_dirs():
        try:
            os.makedirs(d, exist_ok=True)
            probe = os.path.join(d, f".probe_{os.getpid()}_{threading.get_ident()}")
            with open(probe, "w") as f:
                f.write("x")
            os.remove(probe)
            _build_dir_cache.append(d)
            return d
        except OSError:
            continue
    raise KernelBuildError("no writable folder for the kernel build (tried: " + ", ".join(_build_dirs()) + ")")


def library_path(module: str, must_exist: bool = True) -> str | None:
    name = f"{module}_{_source_hash(module)}.so"
    for d in _build_dirs():
        p = os.path.join(d, name)
        if os.path.isfile(p):
            return p
    return None if must_exist else os.path.join(_writable_build_dir(), name)


def _compile(module: str, verbose_ptxas: bool = False) -> str:
    src = os.path.join(CSRC_DIR, module + ".cu")
    if not os.path.isfile(src):
        raise KernelBuildError(f"no such kernel module: {src}")
    out = library_path(module, must_exist=False)
    tmp_out = f"{out}.{os.getpid()}.tmp"
    cmd = [find_nvcc()] + ARCH_FLAGS + NVCC_FLAGS + ["-I", CSRC_DIR, "-o", tmp_out, src] + MODULES.get(module, [])
    if verbose_ptxas:
        cmd += ["-Xptxas", "-v"]
    env = dict(os.environ)
    env.setdefault("TMPDIR", tempfile.gettempdir())
    proc = subprocess.run(cmd, stdout=subprocess.PIPE, stderr=subprocess.STDOUT, text=True, env=env)
    if proc.returncode != 0:
        try:
            os.remove(tmp_out)
        except OSError:
            pass
        raise KernelBuildError(f"nvcc failed for {module}.cu:\n{' '.join(cmd)}\n{proc.stdout}")
    os.replace(tmp_out, out)
    _prune_stale(module, out)
    if verbose_ptxas:
        _log(proc.stdout)
    return out


def _prune_stale(module: str, keep: str) -> None:
    """Remove libraries of `module` built from older sources (same folder, other hash)."""
    folder = os.path.dirname(keep)
    prefix = module + "_"
    for name in os.listdir(folder):
        stem = name[len(prefix):-3] if name.startswith(prefix) and name.endswith(".so") else ""
        if len(stem) == 16 and all(c in "0123456789abcdef" for c in stem) and os.path.join(folder, name) != keep:
            try:
                os.remove(os.path.join(folder, name))
            except OSError:
                pass


def ensure_built(modules: Iterable[str], verbose_ptxas: bool = False) -> Dict[str, str]:
    """Build what is missing of `modules` (in parallel) and return their library paths."""
    modules = list(dict.fromkeys(modules))
    paths: Dict[str, str] = {}
    todo = []
    for m in modules:
        if m not in MODULES:
            raise KernelBuildError(f"unknown kernel module {m!r}; known: {', '.join(sorted(MODULES))}")
        p = None if verbose_ptxas else library_path(m)
        if p:
            paths[m] = p
        else:
            todo.append(m)
    if not todo:
        return paths
    with _lock:
        todo = [m for m in todo if verbose_ptxas or not library_path(m)]
        if todo:
            _writable_build_dir()
            _log(f"compiling {len(todo)} CUDA module(s) for sm_100a: {', '.join(todo)}")
            t0 = time.time()
            workers = max(1, min(len(todo), os.cpu_count() or 1))
            with ThreadPoolExecutor(max_workers=workers) as pool:
                futures = {m: pool.submit(_compile, m, verbose_ptxas) for m in todo}
                pending = set(todo)
                last = time.time()
                while pending:
                    for m in list(pending):
                        if futures[m].done():
                            pending.discard(m)
                            futures[m].result()
                            _log(f"  built {m} ({time.time() - t0:.0f} s)")
                    if pending:
                        time.sleep(0.2)
                        if time.time() - last > 10:
                            last = time.time()
                            _log(f"  still compiling: {', '.join(sorted(pending))} ({time.time() - t0:.0f} s)")
    for m in modules:
        paths[m] = library_path(m)
    return paths


def load(module: str) -> ctypes.CDLL:
    """The loaded library of one module (built first if needed)."""
    lib = _loaded.get(module)
    if lib is None:
        path = ensure_built([module])[module]
        lib = ctypes.CDLL(path)
        lib.llmk_last_error.restype = ctypes.c_char_p
        _loaded[module] = lib
    return lib


def build_all(verbose_ptxas: bool = False) -> Dict[str, str]:
    return ensure_built(sorted(MODULES), verbose_ptxas=verbose_ptxas)
