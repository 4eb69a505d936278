"""Builds and loads the two native libraries of the package.

* ``libyalis_host``: the page allocator of the cache manager and the launch model of the prompt-attention
  kernel (C++, no CUDA); it
  is what the CPU-only tests use.
* ``libyalis_cuda``: every GPU kernel (CUDA C++ for sm_100a only).

Both are plain shared objects with ``extern "C"`` entry points, loaded through
``ctypes``; tensors cross the boundary as raw device pointers.  Nothing is
compiled at install time: the first call that needs a library compiles the
sources that lie beside this file (``csrc/``) with ``g++`` / ``nvcc``, one
process per translation unit, and prints a progress line for each.  Objects are
keyed by a hash of their source, the shared headers and the flags, so a second
call is a no-op.  The build folder is ``yalis_b200/_build`` when that is
writable, else a per-user folder under the system's temporary directory.

There is no fallback: if the CUDA library cannot be built or loaded the caller
gets a ``NativeBuildError`` naming the command that failed.
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

_PKG_DIR = os.path.dirname(os.path.abspath(__file__))
_CSRC = os.path.join(_PKG_DIR, "csrc")

CUDA_ARCH_FLAGS = ["-gencode", "arch=compute_100a,code=sm_100a"]
# --use_fast_math is never given: sin, cos, exp and division stay accurate.
NVCC_FLAGS = ["-O3", "-std=c++17", "-lineinfo",
              "-Xcompiler", "-fPIC", "-Xcompiler", "-fvisibility=hidden",
              "--expt-relaxed-constexpr"]
GXX_FLAGS = ["-O2", "-std=c++17", "-fPIC", "-Wall"]

HOST_SOURCES = ["host/page_allocator.cpp", "host/attention_policy.cpp"]


class NativeBuildError(RuntimeError):
    pass


_lock = threading.Lock()
_loaded = {}


def _log(msg: str) -> None:
    print(f"[yalis_b200] {msg}", file=sys.stderr, flush=True)


def cuda_sources() -> List[str]:
    return sorted(f for f in os.listdir(_CSRC) if f.endswith(".cu"))


def _headers() -> List[str]:
    out = []
    for root, _, files in os.walk(_CSRC):
        for f in files:
            if f.endswith((".cuh", ".h", ".hpp")):
                out.append(os.path.join(root, f))
    return sorted(out)


def build_dir() -> str:
    """In-tree when writable, else a per-user temporary folder."""
    override = os.environ.get("YALIS_B200_BUILD_DIR")
    candidates = [override] if override else []
    candidates.append(os.path.join(_PKG_DIR, "_build"))
    candidates.append(os.path.join(tempfile.gettempdir(), f"yalis_b200_build_{os.getuid()}"))
    for d in candidates:
        try:
            os.makedirs(d, exist_ok=True)
            probe = os.path.join(d, f".w{os.getpid()}")
            with open(probe, "w"):
                pass
            os.remove(probe)
            return d
        except OSError:
            continue
    raise NativeBuildError("no writable build folder among: " + ", ".join(candidates))


def _digest(paths: List[str], flags: List[str]) -> str:
    h = hashlib.sha256()
    for p in paths:
        with open(p, "rb") as f:
            h.update(f.read())
        h.update(b"\0")
    h.update(" ".join(flags).encode())
    return h.hexdigest()[:20]


def _find(tool: str, env: str, extra: Optional[str] = None) -> str:
    path = os.environ.get(env) or shutil.which(tool)
    if path is None and extra and os.path.exists(extra):
        path = extra
    if path is None:
        raise NativeBuildError(f"`{tool}` not found (set {env}); the native library cannot be built")
    return path


def _run(cmd: List[str], what: str) -> None:
    env = dict(os.environ)
    env.setdefault("HOME", tempfile.gettempdir())
    proc = subprocess.run(cmd, stdout=subprocess.PIPE, stderr=subprocess.STDOUT, text=True, env=env)
    if proc.returncode != 0:
        raise NativeBuildError(f"{what} failed ({proc.returncode}):\n  {' '.join(cmd)}\n{proc.stdout}")
    if proc.stdout.strip() and os.environ.get("YALIS_B200_BUILD_VERBOSE"):
        _log(proc.stdout.strip())


def _compile_all(compiler: List[str], sources: List[str], flags: List[str], out_dir: str,
                 tag: str) -> List[str]:
    """Compile each source to an object named by its content hash; returns the objects."""
    headers = _headers()
    jobs = []
    objects = []
    for src in sources:
        path = os.path.join(_CSRC, src)
        # the include path differs between checkouts of the same sources: keep it out of the key
        key = _digest([path] + headers, [os.path.basename(compiler[0])] + [f for f in flags if f != _CSRC])
        obj = os.path.join(out_dir, f"{tag}_{os.path.basename(src)}.{key}.o")
        objects.append(obj)
        if not os.path.exists(obj):
            jobs.append((src, path, obj))
    if not jobs:
        return objects
    done = [0]
    t0 = time.time()

    def one(job):
        src, path, obj = job
        tmp = f"{obj}.{os.getpid()}.tmp"
        _run(compiler + flags + ["-c", path, "-o", tmp], f"compiling {src}")
        os.replace(tmp, obj)
        done[0] += 1
        _log(f"compiled {src} ({done[0]}/{len(jobs)}, {time.time() - t0:.0f}s)")

    _log(f"compiling {len(jobs)} {tag} source file(s) for first use ...")
    workers = max(1, min(len(jobs), (os.cpu_count() or 2)))
    with ThreadPoolExecutor(workers) as pool:
        for f in [pool.submit(one, j) for j in jobs]:
            f.result()
    return objects


def _link(linker: List[str], objects: List[str], out: str) -> None:
    tmp = f"{out}.{os.getpid()}.tmp"
    _run(linker + objects + ["-o", tmp], f"linking {os.path.basename(out)}")
    os.replace(tmp, out)


def _sweep(out_dir: str, prefix: str, lib_prefix: str, keep: List[str]) -> None:
    """Remove objects and libraries of older source versions (best effort)."""
    keep_names = {os.path.basename(k) for k in keep}
    try:
        for name in os.listdir(out_dir):
            stale_obj = name.startswith(prefix + "_") and name.endswith(".o")
            stale_lib = name.startswith(lib_prefix + ".") and name.endswith(".so")
            if (stale_obj or stale_lib) and name not in keep_names:
                os.remove(os.path.join(out_dir, name))
    except OSError:
        pass


def _build(kind: str) -> str:
    out_dir = build_dir()
    if kind == "host":
        cxx = _find("g++", "CXX")
        objs = _compile_all([cxx], HOST_SOURCES, GXX_FLAGS, out_dir, "host")
        key = hashlib.sha256(" ".join(objs).encode()).hexdigest()[:16]
        lib = os.path.join(out_dir, f"libyalis_host.{key}.so")
        if not os.path.exists(lib):
            _link([cxx, "-shared"], objs, lib)
            _sweep(out_dir, "host", "libyalis_host", objs + [lib])
        return lib
    nvcc = _find("nvcc", "NVCC", "/usr/local/cuda/bin/nvcc")
    flags = CUDA_ARCH_FLAGS + NVCC_FLAGS + ["-I", _CSRC]
    objs = _compile_all([nvcc], cuda_sources(), flags, out_dir, "cuda")
    key = hashlib.sha256(" ".join(objs).encode()).hexdigest()[:16]
    lib = os.path.join(out_dir, f"libyalis_cuda.{key}.so")
    if not os.path.exists(lib):
        _log("linking libyalis_cuda ...")
        _link([nvcc, "-shared"] + CUDA_ARCH_FLAGS, objs, lib)
        _sweep(out_dir, "cuda", "libyalis_cuda", objs + [lib])
    return lib


def build(kind: str) -> str:
    """Build (if needed) and return the path of the ``host`` or ``cuda`` library."""
    with _lock:
        return _build(kind)


def load(kind: str) -> ctypes.CDLL:
    """Build if needed, then load the ``host`` or ``cuda`` library (once per process)."""
    with _lock:
        if kind in _loaded:
            return _loaded[kind]
        path = _build(kind)
        try:
            lib = ctypes.CDLL(path)
        except OSError as e:
            raise NativeBuildError(f"cannot load {path}: {e}") from e
        _loaded[kind] = lib
        return lib


def loaded_path(kind: str) -> Optional[str]:
    lib = _loaded.get(kind)
    return getattr(lib, "_name", None) if lib is not None else None
