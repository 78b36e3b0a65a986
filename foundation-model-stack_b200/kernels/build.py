"""Compiling the CUDA sources for sm_100a and loading the resulting libraries.

Each ``csrc/*.cu`` becomes a shared library of its own, compiled by ``nvcc`` directly (no torch headers:
the kernels take raw pointers and a stream) and loaded with ``ctypes``.  The attention source is
compiled once per head size a model needs.  A library is named after a hash of its source, the shared
header and the flags, so it is rebuilt exactly when one of them changes.  Libraries are kept in
``csrc/_build`` inside the package when that folder can be written, else in a per-user folder under the
system's temporary directory.  What is missing is compiled at first use; meanwhile a line is printed
every few seconds.
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
from typing import Dict, List, Optional, Tuple

CSRC = os.path.join(os.path.dirname(os.path.dirname(os.path.abspath(__file__))), "csrc")
ARCH_FLAGS = ["-gencode", "arch=compute_100a,code=sm_100a"]
BASE_FLAGS = ["-O3", "-std=c++17", "-lineinfo", "-Xcompiler", "-fPIC", "-shared"]
# FMS_B200_DEBUG_BOUNDS=1: the libraries are built with index checks (csrc/common.cuh, FMS_IN) that record the first
# index outside its array instead of making the access; ops.check_error_flag then raises with its source line.  The
# flag is part of a library's name, so checked and unchecked builds lie side by side.
DEBUG_BOUNDS = os.environ.get("FMS_B200_DEBUG_BOUNDS", "0") not in ("", "0")
if DEBUG_BOUNDS:
    BASE_FLAGS = BASE_FLAGS + ["-DFMS_DEBUG_BOUNDS"]

# library name -> (source file, extra flags)
PLAIN_LIBRARIES = {
    "elementwise": ("elementwise.cu", []),
    "gemm_f32": ("gemm_f32.cu", []),
    "gemm_bf16_skinny": ("gemm_bf16_skinny.cu", []),
    "gemm_bf16_mid": ("gemm_bf16_mid.cu", []),
    "gemm_bf16_tc": ("gemm_bf16_tc.cu", []),
    "sampling": ("sampling.cu", []),
}

_TAG = "_checked" if DEBUG_BOUNDS else ""
_loaded: Dict[str, ctypes.CDLL] = {}
_lock = threading.Lock()
_dir_lock = threading.Lock()


class KernelBuildError(RuntimeError):
    pass


def find_nvcc() -> str:
    for cand in (os.environ.get("FMS_B200_NVCC"), shutil.which("nvcc"),
                 os.path.join(os.environ.get("CUDA_HOME", "/usr/local/cuda"), "bin", "nvcc"), "/usr/local/cuda/bin/nvcc"):
        if cand and os.path.isfile(cand) and os.access(cand, os.X_OK):
            return cand
    raise KernelBuildError("nvcc was not found (looked at FMS_B200_NVCC, PATH, CUDA_HOME, /usr/local/cuda): the "
                           "CUDA kernels cannot be compiled and there is no other path")


_build_dir: Optional[str] = None


def build_dir() -> str:
    global _build_dir
    with _dir_lock:
        if _build_dir is None:
            _build_dir = _pick_build_dir()
        return _build_dir


def _pick_build_dir() -> str:
    override = os.environ.get("FMS_B200_BUILD_DIR")
    candidates = [override] if override else []
    candidates.append(os.path.join(CSRC, "_build"))
    candidates.append(os.path.join(tempfile.gettempdir(), f"fms_b200_build_{os.getuid()}"))
    for c in candidates:
        try:
            os.makedirs(c, exist_ok=True)
            probe = os.path.join(c, f".probe_{os.getpid()}")
            with open(probe, "w"):
                pass
            os.remove(probe)
            return c
        except OSError:
            continue
    raise KernelBuildError(f"no writable folder for compiled kernels among {candidates}")


def _spec(name: str) -> Tuple[str, List[str]]:
    if name in PLAIN_LIBRARIES:
        return PLAIN_LIBRARIES[name]
    if name.startswith("attention_hd"):
        hd = int(name[len("attention_hd"):])
        if hd <= 0 or hd % 16 or hd > 256:
            raise KernelBuildError(f"attention kernels exist for head sizes that are multiples of 16 up to 256, not {hd}")
        return "attention.cu", [f"-DHEAD_DIM={hd}"]
    raise KernelBuildError(f"unknown kernel library {name!r}")


def _digest(source: str, flags: List[str]) -> str:
    h = hashlib.sha256()
    for path in [os.path.join(CSRC, source)] + sorted(
            os.path.join(CSRC, f) for f in os.listdir(CSRC) if f.endswith((".cuh", ".h"))):
        with open(path, "rb") as f:
            h.update(f.read())
    h.update(" ".join(ARCH_FLAGS + BASE_FLAGS + flags).encode())
    return h.hexdigest()[:12]


def library_path(name: str) -> str:
    source, flags = _spec(name)
    return os.path.join(build_dir(), f"libfms_{name}{_TAG}_{_digest(source, flags)}.so")


def find_built(name: str) -> Optional[str]:
    """The library if it is already compiled — in the package's own folder or the per-user one."""
    source, flags = _spec(name)
    fname = f"libfms_{name}{_TAG}_{_digest(source, flags)}.so"
    for d in (os.environ.get("FMS_B200_BUILD_DIR"), os.path.join(CSRC, "_build"),
              os.path.join(tempfile.gettempdir(), f"fms_b200_build_{os.getuid()}")):
        if d and os.path.isfile(os.path.join(d, fname)):
            return os.path.join(d, fname)
    return None


def compile_library(name: str, verbose: bool = True) -> str:
    source, flags = _spec(name)
    out = library_path(name)
    tmp = out + f".tmp{os.getpid()}"
    cmd = [find_nvcc()] + ARCH_FLAGS + BASE_FLAGS + flags + ["-o", tmp, os.path.join(CSRC, source)]
    start = time.time()
    if verbose:
        print(f"[fms_b200] compiling {source} {' '.join(flags)} for sm_100a ...", file=sys.stderr, flush=True)
    proc = subprocess.Popen(cmd, stdout=subprocess.PIPE, stderr=subprocess.STDOUT, text=True)
    while True:
        try:
            output, _ = proc.communicate(timeout=10)
            break
        except subprocess.TimeoutExpired:
            if verbose:
                print(f"[fms_b200] still compiling {source} ({time.time() - start:.0f} s)", file=sys.stderr, flush=True)
    if proc.returncode != 0:
        if os.path.exists(tmp):
            os.remove(tmp)
        raise KernelBuildError(f"nvcc failed on {source}:\n{' '.join(cmd)}\n{output}")
    os.replace(tmp, out)
    for stale in os.listdir(os.path.dirname(out)):  # earlier builds of this library, from other sources or flags
        if (stale.startswith(f"libfms_{name}{_TAG}_") and stale.endswith(".so") and stale != os.path.basename(out)
                and len(stale) == len(os.path.basename(out))):
            try:
                os.remove(os.path.join(os.path.dirname(out), stale))
            except OSError:
                pass
    if verbose:
        print(f"[fms_b200] compiled {os.path.basename(out)} in {time.time() - start:.0f} s", file=sys.stderr, flush=True)
    return out


def compile_many(names: List[str], verbose: bool = True) -> None:
    """Compiles the missing ones of ``names`` side by side."""
    missing = [n for n in dict.fromkeys(names) if find_built(n) is None]
    errors: List[BaseException] = []

    def work(n):
        try:
            compile_library(n, verbose)
        except BaseException as e:  # noqa: BLE001
            errors.append(e)

    threads = [threading.Thread(target=work, args=(n,)) for n in missing]
    for t in threads:
        t.start()
    for t in threads:
        t.join()
    if errors:
        raise errors[0]


def load_library(name: str) -> ctypes.CDLL:
    """The compiled library, compiling it first if need be.  Raises if that is impossible: there is no
    other implementation to fall back to."""
    with _lock:
        lib = _loaded.get(name)
        if lib is not None:
            return lib
        path = find_built(name) or compile_library(name)
        lib = ctypes.CDLL(path, mode=ctypes.RTLD_LOCAL)
        lib.fms_last_error.restype = ctypes.c_char_p
        _loaded[name] = lib
        return lib


def loaded_libraries() -> Dict[str, ctypes.CDLL]:
    with _lock:
        return dict(_loaded)


def bounds_violations() -> List[str]:
    """In a bounds-checked build: for every loaded library that met an index outside its array since the last call,
    one line with the source line, the index and the extent of the first (reading clears it).  Synchronises."""
    out = []
    if not DEBUG_BOUNDS:
        return out
    for name, lib in loaded_libraries().items():
        word = (ctypes.c_int * 4)()
        if lib.fms_debug_bounds(word) == 0 and word[0]:
            source = _spec(name)[0]
            out.append(f"{name}: {word[0]} accesses outside their arrays were skipped; the first at a check near line "
                       f"{word[1]} of {source} or of a header it includes: index {word[2]}, extent {word[3]}")
    return out


def all_library_names(head_dims=(16, 32, 48, 64, 128, 256)) -> List[str]:
    return list(PLAIN_LIBRARIES) + [f"attention_hd{h}" for h in head_dims]
