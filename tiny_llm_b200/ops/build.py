"""Builds the CUDA sources under csrc/ for sm_100a, one shared object per source, on first use.

A library is compiled when the first op that needs it is called, so a run compiles what its model
needs and nothing else.  Objects are kept in `csrc/_build/` (or, if the package folder cannot be
written, in a per-user folder under the system's temporary directory) under a name that carries a
hash of the source, the shared headers and the flags; a matching object is loaded as it is.
While nvcc runs, a line is printed to stderr every few seconds."""
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
from typing import Dict, Optional

CSRC = os.path.join(os.path.dirname(os.path.dirname(os.path.abspath(__file__))), "csrc")
ARCH_FLAGS = ["-gencode", "arch=compute_100a,code=sm_100a"]
BASE_FLAGS = ["-O3", "-std=c++17", "-lineinfo", "-shared", "-Xcompiler", "-fPIC", "--expt-relaxed-constexpr"]
HEADERS = ["common.cuh"]
EXTRA_HEADERS = {"sampling": ["sampling_noalloc.h"], "attention_mma": ["attention_tiles.cuh"],
                 "linear_tc": ["tc_common.cuh"],
                 "attention_tc": ["tc_common.cuh"]}   # per-source headers that enter the hash

_loaded: Dict[str, ctypes.CDLL] = {}
_lock = threading.Lock()


class BuildError(RuntimeError):
    pass


def nvcc_path() -> str:
    for cand in (os.environ.get("TLLM_NVCC"), shutil.which("nvcc"), "/usr/local/cuda/bin/nvcc"):
        if cand and os.path.isfile(cand):
            return cand
    raise BuildError("nvcc was not found (looked at $TLLM_NVCC, PATH and /usr/local/cuda/bin); "
                     "the engine has no path without its CUDA kernels")


def build_dir() -> str:
    d = os.environ.get("TLLM_BUILD_DIR") or os.path.join(CSRC, "_build")
    try:
        os.makedirs(d, exist_ok=True)
        probe = os.path.join(d, f".w{os.getpid()}")
        with open(probe, "w"):
            pass
        os.remove(probe)
        return d
    except OSError:
        d = os.path.join(tempfile.gettempdir(), f"tiny_llm_b200_build_{os.getuid()}")
        os.makedirs(d, exist_ok=True)
        return d


def _extra_flags(source: str):
    """Flags from the environment (builds for measurements): TLLM_TRACE=1 adds the timeline notes to every
    source; TLLM_NVCC_FLAGS_<SOURCE> gives one source further flags (for instance
    TLLM_NVCC_FLAGS_ATTENTION_TC=-DTLLM_ATT_TIMING=1 for attention_tc.cu)."""
    flags = ["-DTLLM_TRACE=1"] if os.environ.get("TLLM_TRACE") == "1" else []
    return flags + os.environ.get("TLLM_NVCC_FLAGS_" + source[:-3].upper(), "").split()


def _hash(source: str, extra_headers, flags) -> str:
    h = hashlib.sha256()
    for f in [source] + list(HEADERS) + list(EXTRA_HEADERS.get(source[:-3], [])) + list(extra_headers):
        with open(os.path.join(CSRC, f), "rb") as fh:
            h.update(f.encode() + b"\0" + fh.read())
    h.update(" ".join(ARCH_FLAGS + BASE_FLAGS + list(flags) + _extra_flags(source)).encode())
    return h.hexdigest()[:16]


def _tag(flags) -> str:
    """A readable suffix from -DNAME=VALUE flags: attention_mma with -DTLLM_HEAD_DIM=64 -> _head_dim64."""
    out = ""
    for f in flags:
        if f.startswith("-DTLLM_") and "=" in f:
            k, v = f[len("-DTLLM_"):].split("=", 1)
            out += f"_{k.lower()}{v}"
    return out


def object_path(name: str, extra_headers=(), flags=()) -> str:
    return os.path.join(build_dir(), f"{name}{_tag(flags)}-{_hash(name + '.cu', extra_headers, flags)}.so")


def compile_library(name: str, extra_headers=(), flags=(), verbose: bool = True) -> str:
    """Compiles csrc/<name>.cu if no current object exists; returns the object's path."""
    out = object_path(name, extra_headers, flags)
    if os.path.isfile(out):
        return out
    tmp = f"{out}.{os.getpid()}.tmp"
    cmd = [nvcc_path()] + ARCH_FLAGS + BASE_FLAGS + list(flags) + _extra_flags(name + ".cu") + ["-I", CSRC, "-o", tmp,
                                                                                       os.path.join(CSRC, name + ".cu")]
    if verbose:
        print(f"[tiny_llm_b200] compiling {name}.cu{' ' + ' '.join(flags) if flags else ''} for sm_100a ...",
              file=sys.stderr, flush=True)
    t0 = time.time()
    proc = subprocess.Popen(cmd, stdout=subprocess.PIPE, stderr=subprocess.STDOUT, text=True)
    last = t0
    while True:
        try:
            output, _ = proc.communicate(timeout=5)
            break
        except subprocess.TimeoutExpired:
            if verbose and time.time() - last >= 10:
                last = time.time()
                print(f"[tiny_llm_b200] still compiling {name}.cu ({int(last - t0)} s)", file=sys.stderr, flush=True)
    if proc.returncode != 0:
        if os.path.exists(tmp):
            os.remove(tmp)
        raise BuildError(f"nvcc failed on {name}.cu:\n{output}")
    os.replace(tmp, out)
    if verbose:
        print(f"[tiny_llm_b200] compiled {name}.cu in {time.time() - t0:.1f} s", file=sys.stderr, flush=True)
    return out


def load_library(name: str, extra_headers=(), flags=()) -> ctypes.CDLL:
    key = name + _tag(flags)
    with _lock:
        lib = _loaded.get(key)
        if lib is None:
            lib = ctypes.CDLL(compile_library(name, extra_headers, flags))
            lib.tllm_last_error.restype = ctypes.c_char_p
            lib.tllm_set_pdl(1 if _pdl_default() else 0)
            _loaded[key] = lib
        return lib


def _pdl_default() -> bool:
    from .. import ops
    return ops._pdl and os.environ.get("TLLM_PDL", "1") != "0"


def loaded_libraries():
    return {k: v._name for k, v in _loaded.items()}
