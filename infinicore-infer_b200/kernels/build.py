"""Compiling the CUDA sources in ``csrc`` for sm_100a into shared objects, in-tree.

Each module is one shared object built with nvcc from its own sources (``host``, the rules that run on the host and
need no CUDA, with the host compiler alone); a module is built
the first time something asks for it and again when its sources or flags change (a hash of
both is kept beside the object).  Nothing here needs a GPU: nvcc cross-compiles.  There is
no fallback: if a module cannot be built or loaded the caller gets an exception.
"""
from __future__ import annotations

import ctypes
import fcntl
import hashlib
import os
import shutil
import subprocess
import sys
import tempfile
import time
from typing import Dict, List

CSRC = os.path.join(os.path.dirname(os.path.dirname(os.path.abspath(__file__))), "csrc")

# module name -> its .cu sources (all may include the headers listed in HEADERS)
MODULES: Dict[str, List[str]] = {
    "elementwise": ["elementwise.cu"],
    "attention": ["attention.cu"],
    "sampling": ["sampling.cu"],
    "linear_small": ["linear_small.cu"],
    "gemm_tcgen05": ["gemm_tcgen05.cu", "gemm_skinny.cu"],
    "attention_tcgen05": ["attention_tcgen05.cu"],
    "runner": ["runner.cu", "capi.cu", "reference_abi.cu"],
    "host": ["host.cpp"],
}
# modules without device code: built by the host compiler, loadable on a machine without CUDA
HOST_ONLY = {"host"}
HOST_FLAGS = ["-O2", "-std=c++17", "-fPIC", "-shared"]
# libraries a module links against (the others need the CUDA runtime only)
LINK: Dict[str, List[str]] = {"runner": ["-lcublas"]}
HEADERS = ["common.cuh", "attention_static_scratch.h", "runner.h", "model_api.h", "tcgen05.cuh", "tma.cuh", "host_rules.h"]

# -use_fast_math is deliberately absent: expf, division and sqrt stay accurate.
NVCC_FLAGS = [
    "-gencode", "arch=compute_100a,code=sm_100a", "-lineinfo", "-O3", "-std=c++17",
    "-Xcompiler", "-fPIC", "-shared",
]


class BuildError(RuntimeError):
    pass


def find_nvcc() -> str:
    for root in (os.environ.get("CUDA_HOME"), os.environ.get("CUDA_PATH"), "/usr/local/cuda"):
        if root and os.path.isfile(os.path.join(root, "bin", "nvcc")):
            return os.path.join(root, "bin", "nvcc")
    found = shutil.which("nvcc")
    if found:
        return found
    raise BuildError("nvcc not found (looked in $CUDA_HOME, $CUDA_PATH, /usr/local/cuda and $PATH); "
                     "the engine has no CPU or library fallback")


def find_host_compiler() -> str:
    for name in (os.environ.get("CXX"), "g++", "c++", "clang++"):
        found = shutil.which(name) if name else None
        if found:
            return found
    raise BuildError("no C++ compiler found ($CXX, g++, c++, clang++) for the host-side rules")


def build_dir() -> str:
    """``csrc/_build`` when the tree is writable, else a per-user folder under the temp dir."""
    d = os.path.join(CSRC, "_build")
    try:
        os.makedirs(d, exist_ok=True)
        probe = os.path.join(d, f".w{os.getpid()}")
        with open(probe, "w"):
            pass
        os.remove(probe)
        return d
    except OSError:
        d = os.path.join(tempfile.gettempdir(), f"infinicore_infer_b200_build_{os.getuid()}")
        os.makedirs(d, exist_ok=True)
        return d


def _digest(module: str) -> str:
    h = hashlib.sha256()
    h.update(" ".join((HOST_FLAGS if module in HOST_ONLY else NVCC_FLAGS) + LINK.get(module, [])).encode())
    for name in MODULES[module] + HEADERS:
        with open(os.path.join(CSRC, name), "rb") as f:
            h.update(name.encode())
            h.update(f.read())
    return h.hexdigest()


def library_path(module: str) -> str:
    return os.path.join(build_dir(), f"libjk_{module}.so")


def is_current(module: str) -> bool:
    so = library_path(module)
    stamp = so + ".sha256"
    if not (os.path.isfile(so) and os.path.isfile(stamp)):
        return False
    with open(stamp) as f:
        return f.read().strip() == _digest(module)


def build(module: str, verbose: bool = True) -> str:
    """Build one module if it is missing or stale; return the path of its shared object."""
    if module not in MODULES:
        raise BuildError(f"no kernel module named {module}")
    so = library_path(module)
    if is_current(module):
        return so
    lock_path = so + ".lock"
    with open(lock_path, "w") as lock:
        fcntl.flock(lock, fcntl.LOCK_EX)
        try:
            if is_current(module):        # another process built it while we waited
                return so
            tmp = f"{so}.tmp{os.getpid()}"
            if module in HOST_ONLY:
                cmd = [find_host_compiler()] + HOST_FLAGS
            else:
                cmd = [find_nvcc()] + NVCC_FLAGS
            cmd = cmd + ["-I", CSRC, "-o", tmp] + [os.path.join(CSRC, s) for s in MODULES[module]] + LINK.get(module, [])
            if verbose:
                print(f"[infinicore_infer_b200] compiling module '{module}' " + ("for the host" if module in HOST_ONLY else "for sm_100a") + " ...",
                      file=sys.stderr, flush=True)
            t0 = time.time()
            proc = subprocess.Popen(cmd, stdout=subprocess.PIPE, stderr=subprocess.STDOUT, text=True)
            while True:
                try:
                    out, _ = proc.communicate(timeout=10)
                    break
                except subprocess.TimeoutExpired:
                    if verbose:
                        print(f"[infinicore_infer_b200]   ... still compiling '{module}' "
                              f"({time.time() - t0:.0f} s)", file=sys.stderr, flush=True)
            if proc.returncode != 0:
                if os.path.exists(tmp):
                    os.remove(tmp)
                raise BuildError(f"the compiler failed for module {module}:\n{' '.join(cmd)}\n{out}")
            os.replace(tmp, so)
            with open(so + ".sha256", "w") as f:
                f.write(_digest(module))
            if verbose:
                print(f"[infinicore_infer_b200]   built {os.path.basename(so)} in {time.time() - t0:.1f} s",
                      file=sys.stderr, flush=True)
        finally:
            fcntl.flock(lock, fcntl.LOCK_UN)
    return so


def build_all(verbose: bool = True) -> List[str]:
    return [build(m, verbose) for m in MODULES]


_loaded: Dict[str, ctypes.CDLL] = {}


def load(module: str) -> ctypes.CDLL:
    """Build if needed, then load; raises if either fails."""
    lib = _loaded.get(module)
    if lib is None:
        path = build(module)
        try:
            lib = ctypes.CDLL(path)
        except OSError as e:
            raise BuildError(f"cannot load {path}: {e}") from None
        _loaded[module] = lib
    return lib
