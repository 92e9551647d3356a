"""Builds the CUDA kernels of `csrc/` into one shared library, in-tree, with nvcc.

The library is compiled for sm_100a only and loaded with ctypes; there is no
other implementation behind it.  It is rebuilt when the sources' hash changes.
Compilation happens at the first use (a few files, compiled in parallel) and
prints a line per file to stderr meanwhile.
"""

from __future__ import annotations

import hashlib
import os
import shutil
import subprocess
import sys
import tempfile
import time
from concurrent.futures import ThreadPoolExecutor

CSRC = os.path.join(os.path.dirname(os.path.dirname(os.path.abspath(__file__))), "csrc")
NVCC_FLAGS = ["-gencode", "arch=compute_100a,code=sm_100a", "-O3", "-lineinfo", "-std=c++17",
              "-Xcompiler", "-fPIC", "-Xcompiler", "-fvisibility=hidden"]
LIB_NAME = "libsomi_b200_kernels.so"


class BuildError(RuntimeError):
    pass


def _nvcc() -> str:
    for cand in (os.environ.get("NVCC"), shutil.which("nvcc"), "/usr/local/cuda/bin/nvcc"):
        if cand and os.path.isfile(cand):
            return cand
    raise BuildError("nvcc was not found (set NVCC or put it on PATH); the CUDA kernels of "
                     "this engine cannot be built and there is no other implementation")


def sources() -> list[str]:
    return sorted(os.path.join(CSRC, f) for f in os.listdir(CSRC) if f.endswith(".cu"))


def _digest() -> str:
    h = hashlib.sha256(" ".join(NVCC_FLAGS).encode())
    for f in sorted(os.listdir(CSRC)):
        if f.endswith((".cu", ".cuh", ".h")):
            h.update(f.encode())
            with open(os.path.join(CSRC, f), "rb") as fh:
                h.update(fh.read())
    return h.hexdigest()


def _build_dir() -> str:
    d = os.path.join(CSRC, "_build")
    try:
        os.makedirs(d, exist_ok=True)
        probe = os.path.join(d, f".w{os.getpid()}")
        with open(probe, "w"):
            pass
        os.remove(probe)
        return d
    except OSError:
        d = os.path.join(tempfile.gettempdir(), f"somi_b200_build_{os.getuid()}")
        os.makedirs(d, exist_ok=True)
        return d


def _say(msg: str) -> None:
    print(f"[somi_inference_b200] {msg}", file=sys.stderr, flush=True)


def build(force: bool = False, verbose: bool = True) -> str:
    """Compile if needed; return the path of the shared library."""
    bdir = _build_dir()
    lib = os.path.join(bdir, LIB_NAME)
    stamp = os.path.join(bdir, "stamp.txt")
    digest = _digest()
    if not force and os.path.isfile(lib) and os.path.isfile(stamp):
        with open(stamp) as f:
            if f.read().strip() == digest:
                return lib
    nvcc = _nvcc()
    srcs = sources()
    t0 = time.time()
    if verbose:
        _say(f"compiling {len(srcs)} CUDA files for sm_100a into {bdir} (first use only)")

    def compile_one(src: str) -> str:
        obj = os.path.join(bdir, os.path.basename(src)[:-3] + f".{os.getpid()}.o")
        cmd = [nvcc, *NVCC_FLAGS, "-c", src, "-o", obj]
        r = subprocess.run(cmd, capture_output=True, text=True)
        if r.returncode != 0:
            raise BuildError(f"nvcc failed on {src}:\n{r.stdout}\n{r.stderr}")
        if verbose:
            _say(f"  compiled {os.path.basename(src)} ({time.time() - t0:.0f} s)")
        return obj

    with ThreadPoolExecutor(max_workers=min(8, len(srcs))) as pool:
        objs = list(pool.map(compile_one, srcs))
    tmp_lib = lib + f".{os.getpid()}.tmp"
    r = subprocess.run([nvcc, "-shared", "-o", tmp_lib, *objs, "-gencode",
                        "arch=compute_100a,code=sm_100a"], capture_output=True, text=True)
    for o in objs:
        try:
            os.remove(o)
        except OSError:
            pass
    if r.returncode != 0:
        raise BuildError(f"linking failed:\n{r.stdout}\n{r.stderr}")
    os.replace(tmp_lib, lib)
    with open(stamp, "w") as f:
        f.write(digest)
    if verbose:
        _say(f"built {LIB_NAME} in {time.time() - t0:.0f} s")
    return lib
