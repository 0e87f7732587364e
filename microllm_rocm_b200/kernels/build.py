"""Compile the CUDA sources under `csrc/` for sm_100a and load them with ctypes.

Every `.cu` file becomes one shared object, named after the source, its compile-time
definitions and a hash of everything that went into it, so a changed source or flag can
never pick up a stale binary.  Objects are built into `csrc/_build/` inside the package
(or a per-user temporary folder when the tree is read-only) the first time they are asked
for, one `nvcc` process per object, several at once; while that runs a line goes to
stderr every few seconds.  Nothing here needs torch headers, a GPU, a home directory or
the network.

The reference reaches its kernels through a C ABI loaded with ctypes as well
(python/microllm/_capi.py:32-48 finds the library, :109-114 turns a status into an error).
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
from typing import Dict, Iterable, Optional, Tuple

CSRC = os.path.normpath(os.path.join(os.path.dirname(os.path.abspath(__file__)), "..", "csrc"))
ARCH_FLAGS = ["-gencode", "arch=compute_100a,code=sm_100a"]
BASE_FLAGS = ["-O3", "-std=c++17", "-lineinfo", "--shared", "-Xcompiler", "-fPIC",
              "-Xcompiler", "-fvisibility=hidden", "--expt-relaxed-constexpr"]


class KernelBuildError(RuntimeError):
    pass


class KernelError(RuntimeError):
    """A launcher refused its arguments or CUDA reported an error."""


def _nvcc() -> str:
    for cand in (os.environ.get("MLB_NVCC"), shutil.which("nvcc"), "/usr/local/cuda/bin/nvcc"):
        if cand and os.path.exists(cand):
            return cand
    raise KernelBuildError("nvcc not found: the CUDA kernels cannot be built (set MLB_NVCC)")


_build_dir_cache: Optional[str] = None
_build_dir_lock = threading.Lock()


def _build_dir() -> str:
    global _build_dir_cache
    with _build_dir_lock:
        if _build_dir_cache is None:
            _build_dir_cache = _find_build_dir()
        return _build_dir_cache


def _find_build_dir() -> str:
    override = os.environ.get("MLB_BUILD_DIR")
    candidates = [override] if override else []
    candidates.append(os.path.join(CSRC, "_build"))
    candidates.append(os.path.join(tempfile.gettempdir(), f"microllm_b200_build_{os.getuid()}"))
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
    raise KernelBuildError("no writable folder for compiled kernels (tried " + ", ".join(map(str, candidates)) + ")")


def _source_hash(source: str, defines: Dict[str, object], extra_flags: Iterable[str]) -> str:
    h = hashlib.sha256()
    for name in sorted(os.listdir(CSRC)):
        if name.endswith((".cuh", ".h")) or name == source:
            with open(os.path.join(CSRC, name), "rb") as f:
                h.update(name.encode())
                h.update(f.read())
    h.update(repr(sorted(defines.items())).encode())
    h.update(repr(list(ARCH_FLAGS) + list(BASE_FLAGS) + list(extra_flags)).encode())
    return h.hexdigest()[:12]


def object_path(source: str, defines: Optional[Dict[str, object]] = None, extra_flags: Iterable[str] = ()) -> str:
    defines = defines or {}
    tag = "".join(f"-{k.lower()}{v}" for k, v in sorted(defines.items()))
    stem = os.path.splitext(source)[0]
    return os.path.join(_build_dir(), f"{stem}{tag}-{_source_hash(source, defines, extra_flags)}.so")


_progress_lock = threading.Lock()
_in_flight: Dict[str, float] = {}
_reporter: Optional[threading.Thread] = None


def _report_loop():
    while True:
        time.sleep(5.0)
        with _progress_lock:
            if not _in_flight:
                global _reporter
                _reporter = None
                return
            now = time.time()
            names = ", ".join(f"{os.path.basename(k)} ({now - t:.0f}s)" for k, t in _in_flight.items())
        print(f"[microllm_b200] compiling CUDA kernels for sm_100a: {names}", file=sys.stderr, flush=True)


def compile_object(source: str, defines: Optional[Dict[str, object]] = None, extra_flags: Iterable[str] = (),
                   verbose: bool = False) -> str:
    """Build (if needed) and return the path of the shared object for `source`."""
    defines = defines or {}
    out = object_path(source, defines, extra_flags)
    if os.path.exists(out):
        return out
    src = os.path.join(CSRC, source)
    if not os.path.exists(src):
        raise KernelBuildError(f"kernel source {src} does not exist")
    tmp = f"{out}.{os.getpid()}.{threading.get_ident()}.tmp"
    cmd = [_nvcc(), *ARCH_FLAGS, *BASE_FLAGS, *extra_flags, *[f"-D{k}={v}" for k, v in sorted(defines.items())],
           "-I", CSRC, "-o", tmp, src]
    if verbose:
        cmd.insert(1, "-Xptxas")
        cmd.insert(2, "-v")
    global _reporter
    with _progress_lock:
        _in_flight[out] = time.time()
        if _reporter is None:
            _reporter = threading.Thread(target=_report_loop, daemon=True)
            _reporter.start()
    print(f"[microllm_b200] nvcc {source} {' '.join(f'{k}={v}' for k, v in sorted(defines.items()))}".rstrip(),
          file=sys.stderr, flush=True)
    try:
        proc = subprocess.run(cmd, capture_output=True, text=True)
    finally:
        with _progress_lock:
            _in_flight.pop(out, None)
    if proc.returncode != 0:
        if os.path.exists(tmp):
            os.remove(tmp)
        raise KernelBuildError(f"nvcc failed for {source}:\n{' '.join(cmd)}\n{proc.stdout}\n{proc.stderr}")
    if verbose:
        print(proc.stderr, file=sys.stderr)
    os.replace(tmp, out)          # atomic: another process building the same object just wins or loses
    _prune_older_builds(out)
    return out


def _prune_older_builds(current: str) -> None:
    """Objects of the same source and defines built from an earlier state of the sources (another hash) are
    of no use any more; a process that still has one loaded keeps its mapping."""
    folder, name = os.path.split(current)
    prefix = name[:name.rfind("-") + 1]                   # "<stem><defines>-"
    for other in os.listdir(folder):
        if other != name and other.startswith(prefix) and other.endswith(".so") and len(other) == len(name):
            try:
                os.remove(os.path.join(folder, other))
            except OSError:
                pass


def compile_many(items: Iterable[Tuple[str, Dict[str, object]]], jobs: int = 0) -> Dict[Tuple[str, tuple], str]:
    """Build several objects at once.  `items` are (source, defines)."""
    items = list(items)
    jobs = jobs or min(len(items), max(1, (os.cpu_count() or 2)))
    out = {}
    with ThreadPoolExecutor(max_workers=max(1, jobs)) as pool:
        futures = {(s, tuple(sorted(d.items()))): pool.submit(compile_object, s, d) for s, d in items}
        for key, fut in futures.items():
            out[key] = fut.result()
    return out


_loaded: Dict[str, ctypes.CDLL] = {}
_load_lock = threading.Lock()


def load(source: str, defines: Optional[Dict[str, object]] = None) -> ctypes.CDLL:
    """The loaded library for `source` compiled with `defines` (built at first use)."""
    path = compile_object(source, defines)
    with _load_lock:
        lib = _loaded.get(path)
        if lib is None:
            lib = ctypes.CDLL(path)
            lib.mlb_last_error.restype = ctypes.c_char_p
            _loaded[path] = lib
    return lib


class LaunchCounter:
    """How many kernels of this library were launched (one per successful launcher call)."""
    own = 0
    library = 0          # library matrix products issued on the same path


def check(lib: ctypes.CDLL, status: int) -> None:
    LaunchCounter.own += 1
    if status != 0:
        message = lib.mlb_last_error()
        raise KernelError(message.decode("utf-8", "replace") if message else f"kernel launcher returned {status}")
