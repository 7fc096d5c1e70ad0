"""In-tree build of ``libapproxtorch_b200.so`` (hand-written CUDA for sm_100a, no torch headers).

    python -m approxtorch_b200.build [--force] [--verbose]

Each ``csrc/*.cu`` is compiled with ``nvcc -gencode arch=compute_100a,code=sm_100a`` into
``csrc/_obj/`` and linked into ``approxtorch_b200/lib/libapproxtorch_b200.so``, which the Python
binding loads with ctypes.  nvcc cross-compiles, so no GPU is needed to build.
"""

from __future__ import annotations

import concurrent.futures
import glob
import os
import shutil
import subprocess
import sys

PKG = os.path.dirname(os.path.abspath(__file__))
SRC_DIR = os.path.join(PKG, "csrc")
OBJ_DIR = os.path.join(SRC_DIR, "_obj")
LIB_DIR = os.path.join(PKG, "lib")
LIB_PATH = os.path.join(LIB_DIR, "libapproxtorch_b200.so")
HEADER = os.path.join(os.path.dirname(PKG), "include", "approxtorch_b200.h")

ARCH_FLAGS = ["-gencode", "arch=compute_100a,code=sm_100a"]


def _nvcc() -> str:
    cand = os.path.join(os.environ.get("CUDA_HOME", "/usr/local/cuda"), "bin", "nvcc")
    if os.path.exists(cand):
        return cand
    found = shutil.which("nvcc")
    if not found:
        raise RuntimeError("nvcc not found: the CUDA toolkit is required to build approxtorch_b200")
    return found


def _host_compiler_flags() -> list[str]:
    return ["-ccbin", "/usr/bin/g++"] if os.path.exists("/usr/bin/g++") else []


def sources() -> list[str]:
    return sorted(glob.glob(os.path.join(SRC_DIR, "*.cu")))


def _stale(target: str, deps: list[str]) -> bool:
    if not os.path.exists(target):
        return True
    t = os.path.getmtime(target)
    return any(os.path.getmtime(d) > t for d in deps)


def build_library(force: bool = False, verbose: bool = False) -> str:
    """Compile (if stale) and return the path of the shared library.

    Safe to call from several processes at once (every rank of a torchrun job imports the package): the
    build runs under an exclusive file lock, and the library is linked under a temporary name and moved into
    place atomically, so no process ever opens a half-written file."""
    import fcntl
    os.makedirs(LIB_DIR, exist_ok=True)
    with open(os.path.join(LIB_DIR, ".build.lock"), "w") as lock:
        fcntl.flock(lock, fcntl.LOCK_EX)
        try:
            return _build_locked(force, verbose)
        finally:
            fcntl.flock(lock, fcntl.LOCK_UN)


def _build_locked(force: bool, verbose: bool) -> str:
    srcs = sources()
    headers = glob.glob(os.path.join(SRC_DIR, "*.cuh")) + [HEADER]
    os.makedirs(OBJ_DIR, exist_ok=True)
    os.makedirs(LIB_DIR, exist_ok=True)
    nvcc = _nvcc()
    common = [nvcc, "-std=c++17", "-O3", "-lineinfo", *ARCH_FLAGS, *_host_compiler_flags(),
              "-Xcompiler", "-fPIC", "-Xptxas", "-v" if verbose else "-O3"]
    jobs = []
    for src in srcs:
        obj = os.path.join(OBJ_DIR, os.path.basename(src)[:-3] + ".o")
        if force or _stale(obj, [src] + headers):
            jobs.append((src, obj))

    def compile_one(job):
        src, obj = job
        proc = subprocess.run(common + ["-c", src, "-o", obj], capture_output=True, text=True)
        return src, proc

    with concurrent.futures.ThreadPoolExecutor(max_workers=min(8, max(1, len(jobs)))) as pool:
        for src, proc in pool.map(compile_one, jobs):
            if verbose or proc.returncode != 0:
                sys.stderr.write(f"--- {os.path.basename(src)}\n{proc.stdout}{proc.stderr}\n")
            if proc.returncode != 0:
                raise RuntimeError(f"nvcc failed on {src}")
    objs = [os.path.join(OBJ_DIR, os.path.basename(s)[:-3] + ".o") for s in srcs]
    if force or jobs or _stale(LIB_PATH, objs):
        tmp = f"{LIB_PATH}.{os.getpid()}.tmp"
        link = [nvcc, "-shared", *ARCH_FLAGS, *_host_compiler_flags(), "-o", tmp, *objs, "-lcudart"]
        proc = subprocess.run(link, capture_output=True, text=True)
        if proc.returncode != 0:
            sys.stderr.write(proc.stdout + proc.stderr)
            if os.path.exists(tmp):
                os.remove(tmp)
            raise RuntimeError("link of libapproxtorch_b200.so failed")
        os.replace(tmp, LIB_PATH)
    return LIB_PATH


if __name__ == "__main__":
    print(build_library(force="--force" in sys.argv, verbose="--verbose" in sys.argv))
