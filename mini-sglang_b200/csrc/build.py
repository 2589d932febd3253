"""Compile the engine's CUDA sources for sm_100a with nvcc, at first use, and load them.

Each kernel library is one shared object with plain C entry points, loaded with ctypes.  A
library is built at most once per (sources, flags) and kept under `csrc/_build/` next to the
sources (or under a per-user folder in the system's temporary directory when the checkout is
read-only); the file name carries a hash of sources and flags, so an edited source builds a
new file.  Nothing falls back to another implementation: a missing compiler or a failed
build raises KernelBuildError.
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
from typing import Dict, List, Optional, Sequence

HERE = os.path.dirname(os.path.abspath(__file__))
ARCH_FLAGS = ["-gencode", "arch=compute_100a,code=sm_100a"]
BASE_FLAGS = ["-O3", "-std=c++17", "-lineinfo", "-shared", "-Xcompiler", "-fPIC", "-Xcompiler", "-fvisibility=hidden"]

_loaded: Dict[str, ctypes.CDLL] = {}
_lock = threading.Lock()


class KernelBuildError(RuntimeError):
    pass


def _nvcc() -> str:
    for cand in (os.environ.get("MSGL_NVCC"), shutil.which("nvcc"), "/usr/local/cuda/bin/nvcc"):
        if cand and os.path.isfile(cand) and os.access(cand, os.X_OK):
            return cand
    raise KernelBuildError("nvcc not found (looked at $MSGL_NVCC, PATH and /usr/local/cuda/bin): the engine's "
                           "kernels are compiled from source and there is no other implementation to fall back to")


def build_dir() -> str:
    """Where built libraries live: beside the sources if that is writable, else a per-user temp folder."""
    override = os.environ.get("MSGL_BUILD_DIR")
    cands = [override] if override else []
    cands.append(os.path.join(HERE, "_build"))
    cands.append(os.path.join(tempfile.gettempdir(), f"msgl_b200_build_{os.getuid()}"))
    for d in cands:
        try:
            os.makedirs(d, exist_ok=True)
            probe = os.path.join(d, f".w{os.getpid()}")
            with open(probe, "w"):
                pass
            os.unlink(probe)
            return d
        except OSError:
            continue
    raise KernelBuildError("no writable folder for built kernels; set MSGL_BUILD_DIR")


# files a source pulls in with #include: an edit of any of them rebuilds the library
INCLUDED = {"attention.cu": ["tc_common.cuh", "attention_tc.cuh", "attention_tc2.cuh"],
            "attention_noalloc.cu": ["attention.cu", "tc_common.cuh", "attention_tc.cuh", "attention_tc2.cuh", "attention_noalloc.h"],
            "gemm_tc.cu": ["tc_common.cuh"], "decode_step.cu": []}


def _digest(sources: Sequence[str], flags: Sequence[str]) -> str:
    h = hashlib.sha256()
    deps = [d for s in sources for d in INCLUDED.get(s, [])]
    for s in list(sources) + deps + ["common.cuh"]:
        with open(os.path.join(HERE, s), "rb") as f:
            h.update(f.read())
    h.update(" ".join(flags).encode())
    return h.hexdigest()[:16]


def library_path(name: str, sources: Sequence[str], defines: Optional[Dict[str, object]] = None) -> str:
    flags = [f"-D{k}={v}" for k, v in sorted((defines or {}).items())]
    return os.path.join(build_dir(), f"libmsgl_{name}_{_digest(sources, flags)}.so")


def compile_library(name: str, sources: Sequence[str], defines: Optional[Dict[str, object]] = None,
                    verbose: bool = True) -> str:
    """Build (if not built yet) and return the path of the shared object."""
    out = library_path(name, sources, defines)
    if os.path.isfile(out):
        return out
    flags = [f"-D{k}={v}" for k, v in sorted((defines or {}).items())]
    tmp = f"{out}.{os.getpid()}.tmp"
    cmd = [_nvcc()] + ARCH_FLAGS + BASE_FLAGS + flags + \
          ["-I", HERE, "-o", tmp] + [os.path.join(HERE, s) for s in sources]
    if verbose:
        print(f"[mini_sglang_b200] compiling {name} for sm_100a ...", file=sys.stderr, flush=True)
    t0 = time.time()
    proc = subprocess.Popen(cmd, stdout=subprocess.PIPE, stderr=subprocess.STDOUT, text=True)
    # a line now and then while the compiler runs
    done = threading.Event()

    def _tick():
        while not done.wait(10.0):
            if verbose:
                print(f"[mini_sglang_b200] still compiling {name} ({time.time() - t0:.0f} s)", file=sys.stderr, flush=True)

    th = threading.Thread(target=_tick, daemon=True)
    th.start()
    log, _ = proc.communicate()
    done.set()
    if proc.returncode != 0:
        if os.path.exists(tmp):
            os.unlink(tmp)
        raise KernelBuildError(f"nvcc failed for {name} ({' '.join(cmd)}):\n{log}")
    os.replace(tmp, out)   # atomic: concurrent builders produce the same file
    if verbose:
        print(f"[mini_sglang_b200] built {os.path.basename(out)} in {time.time() - t0:.1f} s", file=sys.stderr, flush=True)
    return out


def load_library(name: str, sources: Sequence[str], defines: Optional[Dict[str, object]] = None) -> ctypes.CDLL:
    key = library_path(name, sources, defines)
    with _lock:
        lib = _loaded.get(key)
        if lib is None:
            path = compile_library(name, sources, defines)
            try:
                lib = ctypes.CDLL(path)
            except OSError as e:
                raise KernelBuildError(f"cannot load {path}: {e}") from e
            _loaded[key] = lib
        return lib


# the libraries of the engine -----------------------------------------------------------

COMMON_SOURCES = ["elementwise.cu", "sampling.cu", "gemm_small_m.cu", "gemm_tc.cu"]
ATTENTION_SOURCES = ["attention.cu"]
MMA_HEAD_DIMS = tuple(range(16, 257, 16))   # head sizes the tensor-core attention kernel is built for


def common_library() -> ctypes.CDLL:
    defines = {}
    for knob in ("MSGL_GS_WARPS", "MSGL_GS_PF", "MSGL_PDL_MODE", "MSGL_PDL_SMALL", "MSGL_GT2_STAGES"):      # tuning knobs of the GEMM kernels
        if os.environ.get(knob):
            defines[knob] = int(os.environ[knob])
    return load_library("common", COMMON_SOURCES, defines or None)


def attention_library(head_dim: int) -> ctypes.CDLL:
    """Attention kernels with the tensor-core variant instantiated for `head_dim` when it is one
    of MMA_HEAD_DIMS; other head sizes get the library of head size 128, whose float32-arithmetic
    kernel takes any head size up to 512."""
    hd = head_dim if head_dim in MMA_HEAD_DIMS else 128
    defines = {"MSGL_HEAD_DIM": hd}
    for knob in ("MSGL_DEC_WARPS", "MSGL_DEC_STAGES", "MSGL_DEC_PFK", "MSGL_DEC_PFV", "MSGL_DEC_LAZY", "MSGL_TC_PROFILE", "MSGL_PDL_MODE", "MSGL_PDL_SMALL"):          # tuning knobs / phase timers
        if os.environ.get(knob):
            defines[knob] = int(os.environ[knob])
    return load_library(f"attention_d{hd}", ATTENTION_SOURCES, defines)


def attention_noalloc_library(head_dim: int) -> ctypes.CDLL:
    """The library of csrc/attention_noalloc.h (decode attention with built-in scratch memory)."""
    hd = head_dim if head_dim in MMA_HEAD_DIMS else 128
    return load_library(f"attention_noalloc_d{hd}", ["attention_noalloc.cu"], {"MSGL_HEAD_DIM": hd})


def decode_step_library(head_dim: int) -> ctypes.CDLL:
    """The whole-step decode kernel of csrc/decode_step.cu, instantiated for `head_dim` (a multiple of 32)."""
    defines = {"MSGL_HEAD_DIM": head_dim}
    for knob in ("MSGL_DS_PROFILE", "MSGL_DS_PF", "MSGL_DS_X_CA"):          # phase timers / ring depth
        if os.environ.get(knob):
            defines[knob] = int(os.environ[knob])
    return load_library(f"decode_step_d{head_dim}", ["decode_step.cu"], defines)


def build_all(head_dims: Sequence[int] = (16, 32, 48, 64, 128)) -> List[str]:
    """Compile every library ahead of time (used by the repository's build check)."""
    paths = [compile_library("common", COMMON_SOURCES)]
    for hd in head_dims:
        paths.append(compile_library(f"attention_d{hd}", ATTENTION_SOURCES, {"MSGL_HEAD_DIM": hd}))
    paths.append(compile_library("attention_noalloc_d128", ["attention_noalloc.cu"], {"MSGL_HEAD_DIM": 128}))
    for hd in head_dims:
        if hd % 32 == 0:
            paths.append(compile_library(f"decode_step_d{hd}", ["decode_step.cu"], {"MSGL_HEAD_DIM": hd}))
    return paths
