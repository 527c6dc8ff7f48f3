"""Compiles the CUDA sources of this folder for sm_100a with nvcc and loads them with ctypes.

Each module is one shared library made of a few `.cu` files, built on first use and kept in
`_build/` next to the sources, keyed by a hash of the sources and flags, so a built library
travels with the tree and a changed source is rebuilt.  If the tree is read-only the library
goes to a per-user folder under the system's temporary directory instead.  There is no other
implementation to fall back to: when nvcc is missing or a compile fails this raises, and every
op of the library fails with it.
"""
from __future__ import annotations

import ctypes
import hashlib
import shlex
import os
import shutil
import subprocess
import sys
import tempfile
import threading
import time
from concurrent.futures import ThreadPoolExecutor
from typing import Dict, List

HERE = os.path.dirname(os.path.abspath(__file__))

ARCH_FLAGS = ["-gencode", "arch=compute_100a,code=sm_100a"]
NVCC_FLAGS = ["-O3", "-std=c++17", "-lineinfo", "-Xcompiler", "-fPIC", "-Xcompiler", "-fvisibility=hidden",
              "--expt-relaxed-constexpr"]
# extra compiler flags for experiments (-D...); they are part of the library's hash
NVCC_FLAGS += shlex.split(os.environ.get("X0NE_NVCC_FLAGS", ""))

# module name -> sources.  `core` is all a 32-bit run needs; `fast` holds the bfloat16 kernels.
MODULES: Dict[str, List[str]] = {
    "core": ["elementwise.cu", "attention_generic.cu", "gemm_f32.cu", "sampling.cu", "step_plan.cu"],
    "fast": ["attention_bf16.cu", "gemm_bf16.cu", "fast_common.cu"],
    "noalloc": ["attention_decode_noalloc.cu"],
    "tc": ["gemm_tcgen05.cu", "gemm_skinny_tcgen05.cu", "attention_tcgen05.cu", "fast_common.cu"],
}
HEADERS = ["common.cuh"]
# files a module's sources include besides the headers (they change its hash too)
INCLUDED = {"noalloc": ["attention_bf16.cu", "fast_common.cu", "x0ne_noalloc.h"], "tc": ["tcgen05.cuh"]}

_loaded: Dict[str, ctypes.CDLL] = {}
_lock = threading.Lock()


class BuildError(RuntimeError):
    pass


def _say(msg: str) -> None:
    print(f"[x0ne-b200] {msg}", file=sys.stderr, flush=True)


def find_nvcc() -> str:
    for cand in (os.environ.get("NVCC"), os.path.join(os.environ.get("CUDA_HOME", "/usr/local/cuda"), "bin", "nvcc"),
                 shutil.which("nvcc")):
        if cand and os.path.isfile(cand) and os.access(cand, os.X_OK):
            return cand
    raise BuildError("nvcc was not found (set NVCC or CUDA_HOME); this library has no path without its CUDA kernels")


def _module_hash(name: str) -> str:
    h = hashlib.sha256()
    h.update(" ".join(ARCH_FLAGS + NVCC_FLAGS).encode())
    for f in HEADERS + MODULES[name] + INCLUDED.get(name, []):
        with open(os.path.join(HERE, f), "rb") as fh:
            h.update(f.encode())
            h.update(fh.read())
    return h.hexdigest()[:16]


def _build_dir() -> str:
    d = os.path.join(HERE, "_build")
    try:
        os.makedirs(d, exist_ok=True)
        probe = os.path.join(d, f".w{os.getpid()}")
        with open(probe, "w"):
            pass
        os.remove(probe)
        return d
    except OSError:
        d = os.path.join(tempfile.gettempdir(), f"x0ne_b200_build_{os.getuid()}")
        os.makedirs(d, exist_ok=True)
        return d


def library_path(name: str) -> str:
    return os.path.join(_build_dir(), f"libx0ne_{name}-{_module_hash(name)}.so")


def build(name: str, verbose: bool = True) -> str:
    """Builds module `name` if its library is not there yet; returns the library's path."""
    out = library_path(name)
    if os.path.isfile(out):
        return out
    nvcc = find_nvcc()
    bdir = os.path.dirname(out)
    tag = os.path.basename(out)[:-3]
    sources = MODULES[name]
    if verbose:
        _say(f"compiling module '{name}' for sm_100a ({len(sources)} files) ...")
    t0 = time.time()

    def compile_one(src: str) -> str:
        obj = os.path.join(bdir, f"{tag}-{os.path.splitext(src)[0]}.{os.getpid()}.o")
        cmd = [nvcc] + ARCH_FLAGS + NVCC_FLAGS + ["-I", HERE, "-c", os.path.join(HERE, src), "-o", obj]
        r = subprocess.run(cmd, capture_output=True, text=True)
        if r.returncode != 0:
            raise BuildError(f"nvcc failed on {src}:\n{r.stdout}\n{r.stderr}")
        if verbose:
            _say(f"  {src} done ({time.time() - t0:.0f} s)")
        return obj

    with ThreadPoolExecutor(max_workers=min(8, len(sources))) as pool:
        objs = list(pool.map(compile_one, sources))
    tmp = out + f".{os.getpid()}.tmp"
    # The CUDA runtime is linked as a shared library so that the process has ONE runtime: the one
    # torch has already loaded under the same soname (the rpath serves a process without torch).
    cuda_lib = os.path.join(os.path.dirname(os.path.dirname(nvcc)), "lib64")
    cmd = [nvcc] + ARCH_FLAGS + ["-shared", "--cudart", "shared", "-Xlinker", f"-rpath={cuda_lib}", "-o", tmp] + objs
    r = subprocess.run(cmd, capture_output=True, text=True)
    for o in objs:
        try:
            os.remove(o)
        except OSError:
            pass
    if r.returncode != 0:
        raise BuildError(f"link of module '{name}' failed:\n{r.stdout}\n{r.stderr}")
    os.replace(tmp, out)
    # libraries of older versions of this module's sources are of no use any more (X0NE_KEEP_BUILDS=1
    # keeps them: several sets of experiment flags built side by side)
    prefix = f"libx0ne_{name}-"
    for f in ([] if os.environ.get("X0NE_KEEP_BUILDS") == "1" else os.listdir(bdir)):
        if f.startswith(prefix) and f.endswith(".so") and os.path.join(bdir, f) != out:
            try:
                os.remove(os.path.join(bdir, f))
            except OSError:
                pass
    if verbose:
        _say(f"module '{name}' built in {time.time() - t0:.0f} s -> {out}")
    return out


def load(name: str) -> ctypes.CDLL:
    """The loaded library of module `name`, building it first if needed."""
    with _lock:
        lib = _loaded.get(name)
        if lib is None:
            lib = ctypes.CDLL(build(name))
            _loaded[name] = lib
        return lib


def build_all(verbose: bool = True) -> List[str]:
    return [build(name, verbose) for name in MODULES]
