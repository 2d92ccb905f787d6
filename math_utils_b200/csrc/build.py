"""Builds the CUDA kernels of this library into one shared object for sm_100a.

The sources under this folder are compiled with nvcc at the first call that
needs them and whenever a source changed since (a hash of the sources and of
the flags is kept beside the objects).  The library lands next to the sources;
if that folder cannot be written to, in a per-user folder under the system's
temporary directory.  Nothing here needs a GPU: nvcc cross-compiles.
"""
from __future__ import annotations

import concurrent.futures
import hashlib
import os
import shutil
import subprocess
import sys
import tempfile
import time

HERE = os.path.dirname(os.path.abspath(__file__))
LIB_NAME = "libmu_b200_kernels.so"
NVCC_FLAGS = [
    "-gencode", "arch=compute_100a,code=sm_100a", "-lineinfo", "-O3", "-std=c++17",
    "-Xcompiler", "-fPIC", "-Xcompiler", "-fvisibility=hidden",
]   # no fast-math: exp, tanh and erf keep their full accuracy


class BuildError(RuntimeError):
    pass


def _say(msg: str) -> None:
    print(f"[math_utils_b200 build] {msg}", file=sys.stderr, flush=True)


def sources():
    return sorted(f for f in os.listdir(HERE) if f.endswith(".cu"))


def _headers():
    return sorted(f for f in os.listdir(HERE) if f.endswith((".cuh", ".h")))


def source_hash() -> str:
    h = hashlib.sha256()
    h.update(" ".join(NVCC_FLAGS).encode())
    for name in sources() + _headers():
        h.update(name.encode())
        with open(os.path.join(HERE, name), "rb") as f:
            h.update(f.read())
    return h.hexdigest()[:24]


def find_nvcc() -> str:
    for cand in (os.environ.get("MU_B200_NVCC"), shutil.which("nvcc"),
                 os.path.join(os.environ.get("CUDA_HOME", "/usr/local/cuda"), "bin", "nvcc")):
        if cand and os.path.exists(cand):
            return cand
    raise BuildError("nvcc was not found (PATH, CUDA_HOME, /usr/local/cuda): the CUDA kernels of "
                     "math_utils_b200 cannot be built, and there is no other implementation to fall back to")


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


def _locations(tag: str):
    """(folder of the library, folder of the objects)."""
    in_tree = os.path.join(HERE, "_build")
    if _writable(HERE) and _writable(in_tree):
        return HERE, in_tree
    base = os.path.join(tempfile.gettempdir(), f"math_utils_b200_{os.getuid()}_{tag}")
    os.makedirs(base, exist_ok=True)
    return base, base


def library_path(build_if_needed: bool = True, verbose: bool = True) -> str:
    """Path of an up-to-date kernel library, building it first if needed."""
    tag = source_hash()
    lib_dir, obj_dir = _locations(tag)
    lib = os.path.join(lib_dir, LIB_NAME)
    stamp = os.path.join(obj_dir, "stamp")
    if os.path.exists(lib) and os.path.exists(stamp):
        with open(stamp) as f:
            if f.read().strip() == tag:
                return lib
    # a library shipped without its stamp folder but made from these very sources
    side_stamp = lib + ".stamp"
    if os.path.exists(lib) and os.path.exists(side_stamp):
        with open(side_stamp) as f:
            if f.read().strip() == tag:
                return lib
    if not build_if_needed:
        raise BuildError(f"{lib} is missing or older than its sources")
    _build(lib, obj_dir, tag, verbose)
    return lib


def _compile_one(nvcc: str, src: str, obj: str) -> float:
    t0 = time.time()
    cmd = [nvcc] + NVCC_FLAGS + ["-I", HERE, "-c", os.path.join(HERE, src), "-o", obj]
    proc = subprocess.run(cmd, capture_output=True, text=True)
    if proc.returncode != 0:
        raise BuildError(f"nvcc failed on {src}:\n{proc.stdout}\n{proc.stderr}")
    return time.time() - t0


def _build(lib: str, obj_dir: str, tag: str, verbose: bool) -> None:
    nvcc = find_nvcc()
    srcs = sources()
    if verbose:
        _say(f"compiling {len(srcs)} CUDA files for sm_100a with {nvcc} (first call, or a source changed)")
    objs = [os.path.join(obj_dir, s[:-3] + f".{tag}.o") for s in srcs]
    t0 = time.time()
    workers = max(1, min(len(srcs), os.cpu_count() or 1))
    with concurrent.futures.ThreadPoolExecutor(workers) as pool:
        futures = {pool.submit(_compile_one, nvcc, s, o): s for s, o in zip(srcs, objs)}
        for fut in concurrent.futures.as_completed(futures):
            took = fut.result()
            if verbose:
                _say(f"  {futures[fut]} done in {took:.1f}s ({time.time() - t0:.1f}s since start)")
    tmp = lib + f".{os.getpid()}.tmp"
    proc = subprocess.run([nvcc, "-shared", "-o", tmp] + objs, capture_output=True, text=True)
    if proc.returncode != 0:
        raise BuildError(f"linking {lib} failed:\n{proc.stdout}\n{proc.stderr}")
    os.replace(tmp, lib)
    for path in (os.path.join(obj_dir, "stamp"), lib + ".stamp"):
        with open(path, "w") as f:
            f.write(tag)
    # objects of older source versions are of no further use
    for name in os.listdir(obj_dir):
        if name.endswith(".o") and f".{tag}." not in name:
            try:
                os.remove(os.path.join(obj_dir, name))
            except OSError:
                pass
    if verbose:
        _say(f"built {lib} in {time.time() - t0:.1f}s")


if __name__ == "__main__":
    print(library_path())
