"""Compile the CUDA sources under ``csrc/`` for sm_100a with nvcc and load them.

The kernels are plain ``extern "C"`` entry points in shared libraries; there is
no dependency on the torch C++ headers, so a cold build takes seconds per file.
Libraries are built in-tree (``csrc/_build``) when that folder is writable,
otherwise in ``$PAGEDSERVE_B200_BUILD_DIR`` or a per-user temporary folder.  A
library is rebuilt when the hash of its sources and flags changes.  While nvcc
runs, a progress line is printed every few seconds.
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
from typing import Dict, List, Sequence

CSRC = os.path.normpath(os.path.join(os.path.dirname(os.path.abspath(__file__)), "..", "csrc"))

NVCC_FLAGS = [
    "-gencode", "arch=compute_100a,code=sm_100a",
    "-lineinfo", "-O3", "-std=c++17",
    "-Xcompiler", "-fPIC",
    "--expt-relaxed-constexpr",
]

# library name -> sources (relative to csrc/)
LIBRARIES: Dict[str, List[str]] = {
    "core": ["embed_norm.cu", "gemm_simt.cu", "attention_simt.cu", "sampling.cu", "host_io.cu", "step_state.cu", "step_build.cu"],
    "bf16": ["gemm_skinny.cu", "attention_decode.cu", "attention_prefill.cu"],
    "tc": ["gemm_tc.cu", "gemm_rows_tc.cu", "attention_prefill_tc.cu"],
}

_loaded: Dict[str, ctypes.CDLL] = {}
_lock = threading.Lock()


class BuildError(RuntimeError):
    pass


def register_library(name: str, sources: Sequence[str]) -> None:
    LIBRARIES[name] = list(sources)


def _nvcc() -> str:
    for candidate in (os.environ.get("PAGEDSERVE_B200_NVCC"), shutil.which("nvcc"), "/usr/local/cuda/bin/nvcc"):
        if candidate and os.path.isfile(candidate):
            return candidate
    raise BuildError("nvcc not found: the CUDA kernels of pagedserve_b200 cannot be compiled")


def _writable(path: str) -> bool:
    try:
        os.makedirs(path, exist_ok=True)
        probe = os.path.join(path, f".probe_{os.getpid()}")
        with open(probe, "w"):
            pass
        os.remove(probe)
        return True
    except OSError:
        return False


def build_dir() -> str:
    override = os.environ.get("PAGEDSERVE_B200_BUILD_DIR")
    if override:
        os.makedirs(override, exist_ok=True)
        return override
    in_tree = os.path.join(CSRC, "_build")
    if _writable(in_tree):
        return in_tree
    fallback = os.path.join(tempfile.gettempdir(), f"pagedserve_b200_build_{os.getuid()}")
    os.makedirs(fallback, exist_ok=True)
    return fallback


def _digest(sources: Sequence[str]) -> str:
    h = hashlib.sha256()
    h.update(" ".join(NVCC_FLAGS).encode())
    names = list(sources) + sorted(f for f in os.listdir(CSRC) if f.endswith((".cuh", ".h")))
    for name in names:
        h.update(name.encode())
        with open(os.path.join(CSRC, name), "rb") as handle:
            h.update(handle.read())
    return h.hexdigest()[:16]


def _say(message: str) -> None:
    print(f"[pagedserve_b200] {message}", file=sys.stderr, flush=True)


def _compile(name: str, sources: Sequence[str], out_dir: str, target: str, verbose_ptxas: bool) -> None:
    nvcc = _nvcc()
    started = time.time()
    _say(f"compiling library '{name}' ({len(sources)} CUDA files) for sm_100a ...")
    procs = []
    objects = []
    for source in sources:
        obj = os.path.join(out_dir, f"{name}_{os.path.splitext(source)[0]}.{os.getpid()}.o")
        objects.append(obj)
        cmd = [nvcc, *NVCC_FLAGS, "-I", CSRC, "-c", os.path.join(CSRC, source), "-o", obj]
        if verbose_ptxas:
            cmd[1:1] = ["-Xptxas", "-v"]
        procs.append((source, subprocess.Popen(cmd, stdout=subprocess.PIPE, stderr=subprocess.STDOUT, text=True)))
    pending = list(procs)
    last = time.time()
    while pending:
        pending = [(s, p) for s, p in pending if p.poll() is None]
        if pending and time.time() - last > 5.0:
            _say(f"  still compiling {', '.join(s for s, _ in pending)} ({time.time() - started:.0f} s)")
            last = time.time()
        time.sleep(0.1)
    failed = []
    for source, proc in procs:
        output = proc.stdout.read()
        if proc.returncode != 0:
            failed.append(f"--- {source} ---\n{output}")
        elif verbose_ptxas and output:
            _say(output)
    if failed:
        for obj in objects:
            if os.path.exists(obj):
                os.remove(obj)
        raise BuildError("nvcc failed:\n" + "\n".join(failed))
    tmp_target = f"{target}.{os.getpid()}.tmp"
    link = [nvcc, "-shared", "-o", tmp_target, *objects, "-lcudart"]
    result = subprocess.run(link, stdout=subprocess.PIPE, stderr=subprocess.STDOUT, text=True)
    for obj in objects:
        if os.path.exists(obj):
            os.remove(obj)
    if result.returncode != 0:
        raise BuildError("link failed:\n" + result.stdout)
    os.replace(tmp_target, target)
    _say(f"library '{name}' built in {time.time() - started:.1f} s -> {target}")


def library_path(name: str) -> str:
    return os.path.join(build_dir(), f"libps_{name}_{_digest(LIBRARIES[name])}.so")


def build(name: str, verbose_ptxas: bool = False) -> str:
    """Make sure library ``name`` is compiled; return the path of the .so."""
    if name not in LIBRARIES:
        raise BuildError(f"unknown kernel library {name!r}")
    target = library_path(name)
    if os.path.isfile(target) and not verbose_ptxas:
        return target
    out_dir = os.path.dirname(target)
    lock_path = os.path.join(out_dir, f".lock_{name}")
    import fcntl

    with open(lock_path, "w") as lock_file:
        fcntl.flock(lock_file, fcntl.LOCK_EX)
        try:
            if not os.path.isfile(target) or verbose_ptxas:
                # drop stale builds of this library
                for entry in os.listdir(out_dir):
                    if entry.startswith(f"libps_{name}_") and entry.endswith(".so") and \
                            os.path.join(out_dir, entry) != target:
                        try:
                            os.remove(os.path.join(out_dir, entry))
                        except OSError:
                            pass
                _compile(name, LIBRARIES[name], out_dir, target, verbose_ptxas)
        finally:
            fcntl.flock(lock_file, fcntl.LOCK_UN)
    return target


def load(name: str) -> ctypes.CDLL:
    """Build if needed and dlopen library ``name``; raises if that is impossible."""
    with _lock:
        if name in _loaded:
            return _loaded[name]
        path = build(name)
        try:
            lib = ctypes.CDLL(path)
        except OSError as error:
            raise BuildError(f"cannot load {path}: {error}") from error
        _loaded[name] = lib
        return lib


def build_all(verbose_ptxas: bool = False) -> List[str]:
    return [build(name, verbose_ptxas) for name in sorted(LIBRARIES)]
