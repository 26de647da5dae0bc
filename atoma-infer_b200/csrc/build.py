"""Builds the native libraries in-tree and loads them with ctypes.

Two kinds of library: the host library (cache manager and scheduler, g++) and the
kernel libraries (nvcc, ``-gencode arch=compute_100a,code=sm_100a``).  A kernel
library may be specialised by preprocessor defines (the head size of the attention
kernels); what a model needs is compiled at its first use and kept under
``_build/`` beside the sources, named by a hash of sources, defines and flags.
Nothing is written outside the package folder, so an empty HOME is fine.  While a
compiler runs, a progress line goes to stderr every few seconds.
"""
from __future__ import annotations

import ctypes
import hashlib
import os
import shutil
import subprocess
import sys
import tempfile
import time
from typing import Dict, Mapping, Optional, Sequence

CSRC = os.path.dirname(os.path.abspath(__file__))
BUILD_DIR = os.environ.get("ATOMA_INFER_BUILD_DIR") or os.path.join(CSRC, "_build")
ARCH_FLAGS = ["-gencode", "arch=compute_100a,code=sm_100a"]
NVCC_FLAGS = ["-O3", "-std=c++17", "-lineinfo", "--expt-relaxed-constexpr", "-Xcompiler", "-fPIC", "-shared"]
GXX_FLAGS = ["-O2", "-std=c++17", "-fPIC", "-shared", "-Wall"]

_loaded: Dict[str, ctypes.CDLL] = {}


class BuildError(RuntimeError):
    pass


def find_nvcc() -> str:
    for cand in (
        os.path.join(os.environ.get("CUDA_HOME", ""), "bin", "nvcc") if os.environ.get("CUDA_HOME") else None,
        shutil.which("nvcc"),
        "/usr/local/cuda/bin/nvcc",
    ):
        if cand and os.path.isfile(cand):
            return cand
    raise BuildError("nvcc was not found (looked at $CUDA_HOME/bin, PATH and /usr/local/cuda/bin)")


def _digest(paths: Sequence[str], extra: str) -> str:
    h = hashlib.sha256(extra.encode())
    for p in paths:
        h.update(os.path.relpath(p, CSRC).encode())  # the same name wherever the checkout lies
        with open(p, "rb") as f:
            h.update(f.read())
    return h.hexdigest()[:16]


def _with_includes(paths: Sequence[str]) -> Sequence[str]:
    """The sources and every file they include with quotes, transitively (for the cache key)."""
    import re

    seen, todo = [], list(paths)
    while todo:
        p = todo.pop()
        if p in seen or not os.path.isfile(p):
            continue
        seen.append(p)
        with open(p, errors="replace") as f:
            for inc in re.findall(r'^\s*#\s*include\s+"([^"]+)"', f.read(), flags=re.M):
                for base in (os.path.dirname(p), CSRC):
                    q = os.path.normpath(os.path.join(base, inc))
                    if os.path.isfile(q):
                        todo.append(q)
                        break
    return sorted(seen)


def _run(cmd: Sequence[str], what: str) -> None:
    t0 = time.time()
    proc = subprocess.Popen(cmd, stdout=subprocess.PIPE, stderr=subprocess.STDOUT, text=True)
    last = t0
    while True:
        try:
            out, _ = proc.communicate(timeout=5)
            break
        except subprocess.TimeoutExpired:
            if time.time() - last >= 5:
                print(f"[build] compiling {what} ... {time.time() - t0:.0f} s", file=sys.stderr, flush=True)
                last = time.time()
    if proc.returncode != 0:
        raise BuildError(f"building {what} failed:\n$ {' '.join(cmd)}\n{out}")


def build_library(name: str, sources: Sequence[str], *, cuda: bool, defines: Optional[Mapping[str, object]] = None,
                  extra_flags: Sequence[str] = (), verbose: bool = True) -> str:
    """Compiles ``sources`` (paths relative to csrc/) into ``_build/<name>-<hash>.so``; returns the path."""
    srcs = [os.path.join(CSRC, s) for s in sources]
    defs = [f"-D{k}={v}" for k, v in sorted((defines or {}).items())]
    flags = (NVCC_FLAGS + ARCH_FLAGS if cuda else GXX_FLAGS) + list(extra_flags) + defs
    tag = _digest(list(_with_includes(srcs)), " ".join(flags))
    os.makedirs(BUILD_DIR, exist_ok=True)
    out = os.path.join(BUILD_DIR, f"{name}-{tag}.so")
    if os.path.isfile(out):
        return out
    compiler = find_nvcc() if cuda else (shutil.which("g++") or "g++")
    fd, tmp = tempfile.mkstemp(suffix=".so", dir=BUILD_DIR)
    os.close(fd)
    if verbose:
        print(f"[build] compiling {name} ({', '.join(sources)})", file=sys.stderr, flush=True)
    try:
        _run([compiler, *flags, f"-I{CSRC}", "-o", tmp, *srcs], name)
        os.replace(tmp, out)  # atomic: a concurrent builder sees a whole file or none
    finally:
        if os.path.exists(tmp):
            os.remove(tmp)
    return out


def load_library(name: str, sources: Sequence[str], *, cuda: bool, defines: Optional[Mapping[str, object]] = None,
                 extra_flags: Sequence[str] = ()) -> ctypes.CDLL:
    key = name + repr(sorted((defines or {}).items()))
    lib = _loaded.get(key)
    if lib is None:
        path = build_library(name, sources, cuda=cuda, defines=defines, extra_flags=extra_flags)
        lib = ctypes.CDLL(path)
        lib._path = path
        _loaded[key] = lib
    return lib


HOST_SOURCES = ["host/capi.cpp", "host/cache_manager.cpp", "host/scheduler.cpp", "host/step_meta.cpp"]


def host_library() -> ctypes.CDLL:
    return load_library("host", HOST_SOURCES, cuda=False)


def all_kernel_libraries():
    """(name, sources, defines) of every kernel library, for the build check."""
    from .ops import (ATTENTION_HEAD_DIMS, ATTENTION_SOURCES, ATTENTION_TC_HEAD_DIMS, ATTENTION_TC_SOURCES, CORE_SOURCES,
                      DECODE_STACK_SOURCES, GEMM_SOURCES)

    return [("core", CORE_SOURCES, None), ("gemm_tcgen05", GEMM_SOURCES, None)] + [
        (f"attention_d{d}", ATTENTION_SOURCES, {"HEAD_DIM": d}) for d in ATTENTION_HEAD_DIMS] + [
        (f"attention_noalloc_d{d}", ["kernels/attention_noalloc.cu"], {"HEAD_DIM": d}) for d in (64, 128)] + [
        (f"attention_tc_d{d}", ATTENTION_TC_SOURCES, {"HEAD_DIM": d}) for d in ATTENTION_TC_HEAD_DIMS] + [
        (f"decode_stack_d{d}", DECODE_STACK_SOURCES, {"HEAD_DIM": d}) for d in (64, 128)]
