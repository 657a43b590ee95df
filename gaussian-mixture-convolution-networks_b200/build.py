"""Builds libgmc_b200.so (the C-ABI library) from csrc/*.cu with nvcc for sm_100a.

Run as a script or call build(). Objects are compiled in parallel and only when a source or header
is newer than the object; the shared object lands next to the Python package in gmc/_lib/.
"""
import concurrent.futures
import os
import subprocess
import sys

HERE = os.path.dirname(os.path.abspath(__file__))
CSRC = os.path.join(HERE, "csrc")
INCLUDE = os.path.join(os.path.dirname(HERE), "include")
OUT_DIR = os.path.join(HERE, "gmc", "_lib")
BUILD_DIR = os.path.join(HERE, "build")
LIB_PATH = os.path.join(OUT_DIR, "libgmc_b200.so")

NVCC = os.environ.get("NVCC", "/usr/local/cuda/bin/nvcc")
ARCH_FLAGS = ["-gencode", "arch=compute_100a,code=sm_100a"]
COMMON_FLAGS = ["-O3", "-std=c++17", "-lineinfo", "-Xcompiler", "-fPIC", "-I", INCLUDE, "-I", CSRC]
# Fast-math is applied per file: kernels whose integer results must be bit-exact (Morton codes) are
# compiled with IEEE arithmetic and without FMA contraction.
FAST_MATH = ["--use_fast_math"]
IEEE_FILES = {"lbvh.cu", "mhem_fit.cu", "convolution_fitting.cu"}


def _sources():
    return sorted(f for f in os.listdir(CSRC) if f.endswith(".cu"))


def _headers_mtime():
    newest = 0.0
    for d in (CSRC, INCLUDE):
        for f in os.listdir(d):
            if f.endswith((".cuh", ".h")):
                newest = max(newest, os.path.getmtime(os.path.join(d, f)))
    return newest


CHECKED_LIB_PATH = os.path.join(OUT_DIR, "libgmc_b200_checked.so")


def _compile(src, verbose, bounds_check=False):
    obj = os.path.join(BUILD_DIR + ("_checked" if bounds_check else ""), src[:-3] + ".o")
    src_path = os.path.join(CSRC, src)
    if os.path.exists(obj) and os.path.getmtime(obj) >= max(os.path.getmtime(src_path), _headers_mtime()):
        return obj
    flags = list(COMMON_FLAGS)
    if bounds_check:
        flags += ["-DGMC_BOUNDS_CHECK"]
    if src in IEEE_FILES:
        flags += ["--fmad=false"]
    else:
        flags += FAST_MATH
    if verbose:
        flags += ["-Xptxas", "-v"]
    cmd = [NVCC] + ARCH_FLAGS + flags + ["-c", src_path, "-o", obj]
    res = subprocess.run(cmd, capture_output=True, text=True)
    if res.returncode != 0:
        raise RuntimeError(f"nvcc failed for {src}:\n{res.stdout}\n{res.stderr}")
    if verbose:
        print(res.stderr)
    return obj


def build(verbose: bool = False, bounds_check: bool = False) -> str:
    """bounds_check=True builds libgmc_b200_checked.so instead: the same sources with -DGMC_BOUNDS_CHECK (indices read from
    data are range-checked on the device; used by the tests in place of a memory checker)."""
    lib_path = CHECKED_LIB_PATH if bounds_check else LIB_PATH
    os.makedirs(OUT_DIR, exist_ok=True)
    os.makedirs(BUILD_DIR + ("_checked" if bounds_check else ""), exist_ok=True)
    srcs = _sources()
    with concurrent.futures.ThreadPoolExecutor(max_workers=min(8, len(srcs))) as pool:
        objs = list(pool.map(lambda s: _compile(s, verbose, bounds_check), srcs))
    if (not os.path.exists(lib_path)) or any(os.path.getmtime(o) > os.path.getmtime(lib_path) for o in objs):
        cmd = [NVCC] + ARCH_FLAGS + ["-shared", "-o", lib_path] + objs + ["-lcudart"]
        res = subprocess.run(cmd, capture_output=True, text=True)
        if res.returncode != 0:
            raise RuntimeError(f"link failed:\n{res.stdout}\n{res.stderr}")
    return lib_path


if __name__ == "__main__":
    print(build(verbose="-v" in sys.argv, bounds_check="--checked" in sys.argv))
