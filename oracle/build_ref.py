"""TEST INFRASTRUCTURE. Builds the REFERENCE's own native sources (CPU path) into oracle/_ref/libgmc_ref.so.

The sources are compiled where they lie in the reference checkout (nothing is copied): `lbvh/bvh.cu`,
`convolution_fitting/Tree.cu`, `evaluate_inversed/parallel_implementation.cu`, `CpuSynchronisationPoint.cpp`, and the
header-only template bodies of `bvh_mhem_fit` and `convolution_fitting` through oracle/ref_entry.cu, which adds plain-C
entry points.  The third-party headers the reference expects beside its tree (glm, gcem, yamc: empty clone targets
there, none installed) are replaced by the small stand-ins in oracle/ref_shims/.  nvcc compiles the .cu files, so their
host code is built the way the reference builds it (no host fast-math for .cu units; its CPU launcher is OpenMP).

The recipe needs the reference checkout (path in GMC_REFERENCE_ROOT, default /root/reference); where that is absent
the prebuilt library is used as it is.
"""
import concurrent.futures
import os
import subprocess
import sysconfig

HERE = os.path.dirname(os.path.abspath(__file__))
OUT_DIR = os.path.join(HERE, "_ref")
LIB_PATH = os.path.join(OUT_DIR, "libgmc_ref.so")
SHIMS = os.path.join(HERE, "ref_shims")
ENTRY = os.path.join(HERE, "ref_entry.cu")


def reference_ext_dir():
    root = os.environ.get("GMC_REFERENCE_ROOT", "/root/reference")
    d = os.path.join(root, "src", "gmc", "cpp", "extensions")
    return d if os.path.isdir(d) else None


def available() -> bool:
    return os.path.exists(LIB_PATH)


def _torch_dirs():
    import torch
    base = os.path.dirname(torch.__file__)
    inc = os.path.join(base, "include")
    return [inc, os.path.join(inc, "torch", "csrc", "api", "include")], os.path.join(base, "lib")


def _units(ext):
    # (object name, source, extra defines)
    units = [
        ("ref_bvh.o", os.path.join(ext, "lbvh", "bvh.cu"), []),
        ("ref_tree.o", os.path.join(ext, "convolution_fitting", "Tree.cu"), []),
        ("ref_eval_cpu.o", os.path.join(ext, "evaluate_inversed", "parallel_implementation.cu"), []),
    ]
    for part in ("COMMON", "LBVH", "MHEM_FWD", "MHEM_BWD", "CONVFIT_FWD", "CONVFIT_BWD", "EVAL"):
        units.append(("entry_%s.o" % part.lower(), ENTRY, ["-DREF_PART_" + part]))
    return units


def build(force: bool = False, jobs: int = 0) -> str:
    """Returns the library path; builds it when the reference checkout is present and the library is stale."""
    ext = reference_ext_dir()
    if ext is None:
        if not os.path.exists(LIB_PATH):
            raise FileNotFoundError("no reference checkout and no prebuilt " + LIB_PATH)
        return LIB_PATH
    deps = [ENTRY] + [os.path.join(r, f) for r, _, fs in os.walk(SHIMS) for f in fs]
    newest = max(os.path.getmtime(p) for p in deps)
    if not force and os.path.exists(LIB_PATH) and os.path.getmtime(LIB_PATH) >= newest:
        return LIB_PATH
    os.makedirs(OUT_DIR, exist_ok=True)
    incs, torch_lib = _torch_dirs()
    common = ["-std=c++17", "-O2", "--expt-extended-lambda", "--expt-relaxed-constexpr", "-DNDEBUG",
              "-DGPE_LIMIT_N_REDUCTION", "-gencode", "arch=compute_100a,code=sm_100a",
              "-Xcompiler", "-fopenmp,-fPIC", "-w", "-I" + SHIMS, "-I" + ext] + ["-I" + i for i in incs]

    def compile_unit(unit):
        obj, src, defs = unit
        out = os.path.join(OUT_DIR, obj)
        if not force and os.path.exists(out) and os.path.getmtime(out) >= max(newest, os.path.getmtime(src)):
            return out
        subprocess.run(["nvcc"] + common + defs + ["-c", src, "-o", out], check=True)
        return out

    jobs = jobs or max(1, min(6, (os.cpu_count() or 2) - 1))
    with concurrent.futures.ThreadPoolExecutor(jobs) as pool:
        objs = list(pool.map(compile_unit, _units(ext)))
    sync_obj = os.path.join(OUT_DIR, "ref_sync.o")
    subprocess.run(["g++", "-std=c++17", "-O2", "-fPIC", "-I" + SHIMS, "-I" + ext, "-c",
                    os.path.join(ext, "CpuSynchronisationPoint.cpp"), "-o", sync_obj], check=True)
    subprocess.run(["nvcc", "-shared", "-o", LIB_PATH] + objs + [sync_obj] +
                   ["-Xcompiler", "-fopenmp", "-L" + torch_lib, "-ltorch", "-ltorch_cpu", "-lc10",
                    "-Xlinker", "-rpath," + torch_lib], check=True)
    return LIB_PATH


if __name__ == "__main__":
    print(build(force=True))
