"""Compiling and loading the CUDA modules of this package.

Each ``.cu`` file here becomes one shared library for sm_100a, built with nvcc alone
(no torch headers: the launchers are plain ``extern "C"`` functions taking device
pointers and a stream, in the manner of maeddesg/ROCmForge's ``extern "C"`` HIP launchers,
hip_kernels/norm.hip:154-171, which its build.rs:42-131 compiles one file at a time).
Libraries are kept beside the sources in ``_build/`` and rebuilt when a source changes;
only the modules a model asks for are compiled, at the first call that needs them.
There is no fallback: a module that cannot be built or loaded is an error.
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
from typing import Dict, Iterable, List

HERE = os.path.dirname(os.path.abspath(__file__))

NVCC_FLAGS = ["-gencode", "arch=compute_100a,code=sm_100a", "-lineinfo", "-O3", "-std=c++17",
              "--shared", "-Xcompiler", "-fPIC"]

# module name -> sources (first is the translation unit, the rest are headers it includes)
MODULES: Dict[str, List[str]] = {
    "elementwise": ["elementwise.cu", "common.cuh"],
    "gemm_simt": ["gemm_simt.cu", "common.cuh"],
    "attention_generic": ["attention_generic.cu", "common.cuh"],
    "sampling": ["sampling.cu", "common.cuh"],
    "random_fill": ["random_fill.cu", "common.cuh"],
    "gemm_tcgen05": ["gemm_tcgen05.cu", "tcgen05_common.cuh", "common.cuh"],
    # has one CTA load a tile for its whole cluster (this GPU's memory only): a file of its own, left out of
    # multi-GPU runs; the package works without it
    "gemm_tcgen05_cluster": ["gemm_tcgen05_cluster.cu", "tcgen05_common.cuh", "common.cuh"],
    "attention_decode": ["attention_decode.cu", "common.cuh"],
    "attention_prefill": ["attention_prefill.cu", "common.cuh"],
    "attention_prefill_tc": ["attention_prefill_tc.cu", "tcgen05_common.cuh", "common.cuh"],
    "attention_decode_noalloc": ["attention_decode_noalloc.cu", "attention_decode_noalloc.h", "attention_decode.cu",
                                 "common.cuh"],
}

_loaded: Dict[str, ctypes.CDLL] = {}
_lock = threading.Lock()


class BuildError(RuntimeError):
    pass


def _say(msg: str) -> None:
    print(f"[rocmforge_b200] {msg}", file=sys.stderr, flush=True)


def build_dir() -> str:
    d = os.environ.get("ROCMFORGE_B200_BUILD_DIR") or os.path.join(HERE, "_build")
    try:
        os.makedirs(d, exist_ok=True)
        probe = os.path.join(d, f".w{os.getpid()}")
        with open(probe, "w"):
            pass
        os.remove(probe)
        return d
    except OSError:
        d = os.path.join(tempfile.gettempdir(), f"rocmforge_b200_build_{os.getuid()}")
        os.makedirs(d, exist_ok=True)
        return d


def _nvcc() -> str:
    for cand in (os.environ.get("NVCC"), shutil.which("nvcc"), "/usr/local/cuda/bin/nvcc"):
        if cand and os.path.exists(cand):
            return cand
    raise BuildError("nvcc not found: the CUDA modules of rocmforge_b200 cannot be compiled")


def _digest(name: str) -> str:
    h = hashlib.sha256()
    h.update(" ".join(NVCC_FLAGS).encode())
    for src in MODULES[name]:
        with open(os.path.join(HERE, src), "rb") as f:
            h.update(f.read())
    return h.hexdigest()


def lib_path(name: str) -> str:
    return os.path.join(build_dir(), f"librf_{name}.so")


def is_current(name: str) -> bool:
    so = lib_path(name)
    tag = so + ".sha256"
    if not (os.path.exists(so) and os.path.exists(tag)):
        return False
    with open(tag) as f:
        return f.read().strip() == _digest(name)


def _compile(name: str) -> subprocess.Popen:
    so = lib_path(name)
    tmp = so + f".tmp{os.getpid()}"
    cmd = [_nvcc(), *NVCC_FLAGS, "-I", HERE, os.path.join(HERE, MODULES[name][0]), "-o", tmp]
    extra = os.environ.get("ROCMFORGE_B200_NVCC_EXTRA")
    if extra:
        cmd[1:1] = extra.split()
    p = subprocess.Popen(cmd, stdout=subprocess.PIPE, stderr=subprocess.STDOUT, text=True)
    p._rf = (name, so, tmp, cmd)          # type: ignore[attr-defined]
    return p


def ensure_built(names: Iterable[str]) -> None:
    """Compile, in parallel, those of ``names`` whose library is missing or stale."""
    todo = [n for n in dict.fromkeys(names) if not is_current(n)]
    for n in todo:
        if n not in MODULES:
            raise BuildError(f"unknown CUDA module {n!r}")
    if not todo:
        return
    _say(f"compiling {len(todo)} CUDA module(s) for sm_100a: {', '.join(todo)}")
    procs = [_compile(n) for n in todo]
    t0 = last = time.time()
    pending = list(procs)
    while pending:
        time.sleep(0.2)
        pending = [p for p in pending if p.poll() is None]
        if pending and time.time() - last > 10:
            last = time.time()
            _say(f"  still compiling {', '.join(p._rf[0] for p in pending)} ({last - t0:.0f} s)")
    for p in procs:
        name, so, tmp, cmd = p._rf
        out = p.stdout.read() if p.stdout else ""
        if p.returncode != 0:
            raise BuildError(f"nvcc failed for module {name}:\n{' '.join(cmd)}\n{out}")
        os.replace(tmp, so)
        with open(so + ".sha256", "w") as f:
            f.write(_digest(name))
    _say(f"  done in {time.time() - t0:.0f} s")


def load(name: str) -> ctypes.CDLL:
    """The module's library, compiled first if needed."""
    with _lock:
        if name in _loaded:
            return _loaded[name]
        ensure_built([name])
        try:
            lib = ctypes.CDLL(lib_path(name))
        except OSError as e:
            raise BuildError(f"CUDA module {name} was built but cannot be loaded: {e}") from None
        if hasattr(lib, "rf_set_pdl"):
            lib.rf_set_pdl(ctypes.c_int(0 if os.environ.get("ROCMFORGE_B200_PDL", "1") == "0" else 1))
        _loaded[name] = lib
        return lib


def available(name: str) -> bool:
    """Whether the module's sources are present (an optional module may have been left out)."""
    return name in MODULES and all(os.path.exists(os.path.join(HERE, src)) for src in MODULES[name])


def build_all() -> None:
    ensure_built([n for n in MODULES if available(n)])
