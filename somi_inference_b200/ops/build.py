"""Builds the CUDA kernels of `csrc/` into one shared library, in-tree, with nvcc.

The library is compiled for sm_100a only and loaded with ctypes; there is no
other implementation behind it.  It is rebuilt when the sources' hash changes.
Compilation happens at the first use (a few files, compiled in parallel) and
prints a line per file to stderr meanwhile.

A part that brings kernels of its own (a mixer or feed-forward outside this package) builds them
the same way with `build_library(its folder, a library name)`: its `.cu` files may include the
headers of `csrc/` (`common.cuh` for `SOMI_API`, `launch_pdl` and `launch_status`), and it loads
the result with ctypes and launches on the current stream.
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


def sources(src_dir: str = CSRC) -> list[str]:
    return sorted(os.path.join(src_dir, f) for f in os.listdir(src_dir) if f.endswith(".cu"))


def _digest(src_dir: str, include_dirs: tuple[str, ...]) -> str:
    h = hashlib.sha256(" ".join(NVCC_FLAGS).encode())
    for d in (src_dir, *include_dirs):
        for f in sorted(os.listdir(d)):
            if f.endswith((".cu", ".cuh", ".h")) and (d == src_dir or not f.endswith(".cu")):
                h.update(f.encode())
                with open(os.path.join(d, f), "rb") as fh:
                    h.update(fh.read())
    return h.hexdigest()


def _build_dir(src_dir: str) -> str:
    d = os.path.join(src_dir, "_build")
    try:
        os.makedirs(d, exist_ok=True)
        probe = os.path.join(d, f".w{os.getpid()}")
        with open(probe, "w"):
            pass
        os.remove(probe)
        return d
    except OSError:
        tag = "" if src_dir == CSRC else "_" + hashlib.sha256(src_dir.encode()).hexdigest()[:10]
        d = os.path.join(tempfile.gettempdir(), f"somi_b200_build_{os.getuid()}{tag}")
        os.makedirs(d, exist_ok=True)
        return d


def _say(msg: str) -> None:
    print(f"[somi_inference_b200] {msg}", file=sys.stderr, flush=True)


def build(force: bool = False, verbose: bool = True) -> str:
    """Compile the engine's kernels if needed; return the path of the shared library."""
    return build_library(CSRC, LIB_NAME, force=force, verbose=verbose)


def build_library(src_dir: str, lib_name: str, include_dirs: tuple[str, ...] = (),
                  force: bool = False, verbose: bool = True) -> str:
    """Compile every `.cu` file of `src_dir` into the shared library `lib_name` (in
    `src_dir/_build`, or a temporary folder where that cannot be written) if its stamp does not
    match the sources; return its path.  The headers of this package's `csrc/` are on the include
    path, with those of `include_dirs`."""
    src_dir = os.path.abspath(src_dir)
    include_dirs = tuple(os.path.abspath(d) for d in include_dirs)
    if src_dir != CSRC and CSRC not in include_dirs:
        include_dirs = (*include_dirs, CSRC)
    bdir = _build_dir(src_dir)
    lib = os.path.join(bdir, lib_name)
    stamp = os.path.join(bdir, "stamp.txt")
    digest = _digest(src_dir, include_dirs)
    if not force and os.path.isfile(lib) and os.path.isfile(stamp):
        with open(stamp) as f:
            if f.read().strip() == digest:
                return lib
    nvcc = _nvcc()
    srcs = sources(src_dir)
    if not srcs:
        raise BuildError(f"no .cu files in {src_dir}")
    includes = [flag for d in include_dirs for flag in ("-I", d)]
    t0 = time.time()
    if verbose:
        _say(f"compiling {len(srcs)} CUDA files for sm_100a into {bdir} (first use only)")

    def compile_one(src: str) -> str:
        obj = os.path.join(bdir, os.path.basename(src)[:-3] + f".{os.getpid()}.o")
        cmd = [nvcc, *NVCC_FLAGS, *includes, "-c", src, "-o", obj]
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
        _say(f"built {lib_name} in {time.time() - t0:.0f} s")
    return lib
