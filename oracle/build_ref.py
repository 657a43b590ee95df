"""TEST INFRASTRUCTURE. Builds the REFERENCE's own native sources (CPU path) into two libraries under oracle/_ref/:
libgmc_ref_fit.so (LBVH, BVH-MHEM fit, evaluation) and libgmc_ref_convfit.so (convolution fitting).

Two libraries because the reference builds these as separate extension modules (bvh_mhem_fit/binding.py:11-20 links
lbvh/bvh.cu, convolution_fitting/binding.py:10-19 links Tree.cu) and relies on it: lbvh/building.h and
convolution_fitting/building.h (likewise the two morton_code.h) define the same inline functions
(lbvh::kernels::determine_range, find_split, lbvh::sort_morton_codes) with different bodies under the same include
guard. Linked into one object the linker keeps one body for both users and the convolution tree silently gets the
other variant (it differs for leaves with equal Morton codes).

The sources are compiled where they lie in the reference checkout (nothing is copied): `lbvh/bvh.cu`,
`convolution_fitting/Tree.cu`, `evaluate_inversed/parallel_implementation.cu`, `CpuSynchronisationPoint.cpp`, and the
header-only template bodies of `bvh_mhem_fit` and `convolution_fitting` through oracle/ref_entry.cu, which adds plain-C
entry points.  The third-party headers the reference expects beside its tree (glm, gcem, yamc: empty clone targets
there, none installed) are replaced by the small stand-ins in oracle/ref_shims/.  nvcc compiles the .cu files, so their
host code is built the way the reference builds it (no host fast-math for .cu units; its CPU launcher is OpenMP).

The recipe needs the reference checkout (its path comes from GMC_REFERENCE_ROOT or the default below); where that is
absent the prebuilt library is used as it is.
"""
import concurrent.futures
import os
import subprocess
import sysconfig

HERE = os.path.dirname(os.path.abspath(__file__))
OUT_DIR = os.path.join(HERE, "_ref")
LIB_FIT = os.path.join(OUT_DIR, "libgmc_ref_fit.so")
LIB_CONVFIT = os.path.join(OUT_DIR, "libgmc_ref_convfit.so")
LIB_PATH = LIB_FIT
SHIMS = os.path.join(HERE, "ref_shims")
ENTRY = os.path.join(HERE, "ref_entry.cu")


def reference_ext_dir():
    root = os.environ.get("GMC_REFERENCE_ROOT", "/root/reference")
    d = os.path.join(root, "src", "gmc", "cpp", "extensions")
    return d if os.path.isdir(d) else None


def available() -> bool:
    return os.path.exists(LIB_FIT) and os.path.exists(LIB_CONVFIT)


def _torch_dirs():
    import torch
    base = os.path.dirname(torch.__file__)
    inc = os.path.join(base, "include")
    return [inc, os.path.join(inc, "torch", "csrc", "api", "include")], os.path.join(base, "lib")


FIT_PARTS = ("LBVH", "MHEM_FWD", "MHEM_BWD", "EVAL")
CONVFIT_PARTS = ("CONVFIT_FWD", "CONVFIT_BWD")


def _units(ext):
    # (object name, source, extra defines, library)
    units = [
        ("ref_bvh.o", os.path.join(ext, "lbvh", "bvh.cu"), [], "fit"),
        ("ref_eval_cpu.o", os.path.join(ext, "evaluate_inversed", "parallel_implementation.cu"), [], "fit"),
        ("ref_tree.o", os.path.join(ext, "convolution_fitting", "Tree.cu"), [], "convfit"),
        ("entry_common.o", ENTRY, ["-DREF_PART_COMMON"], "both"),
    ]
    for part in FIT_PARTS:
        units.append(("entry_%s.o" % part.lower(), ENTRY, ["-DREF_PART_" + part], "fit"))
    for part in CONVFIT_PARTS:
        units.append(("entry_%s.o" % part.lower(), ENTRY, ["-DREF_PART_" + part], "convfit"))
    return units


def build(force: bool = False, jobs: int = 0) -> str:
    """Returns the library path; builds it when the reference checkout is present and the library is stale."""
    ext = reference_ext_dir()
    if ext is None:
        if not available():
            raise FileNotFoundError("no reference checkout and no prebuilt libraries under " + OUT_DIR)
        return LIB_PATH
    deps = [ENTRY, os.path.abspath(__file__)] + [os.path.join(r, f) for r, _, fs in os.walk(SHIMS) for f in fs]
    newest = max(os.path.getmtime(p) for p in deps)
    if not force and available() and min(os.path.getmtime(LIB_FIT), os.path.getmtime(LIB_CONVFIT)) >= newest:
        return LIB_PATH
    os.makedirs(OUT_DIR, exist_ok=True)
    incs, torch_lib = _torch_dirs()
    common = ["-std=c++17", "-O2", "--expt-extended-lambda", "--expt-relaxed-constexpr", "-DNDEBUG",
              "-DGPE_LIMIT_N_REDUCTION", "-gencode", "arch=compute_100a,code=sm_100a",
              "-Xcompiler", "-fopenmp,-fPIC", "-w", "-I" + SHIMS, "-I" + ext] + ["-I" + i for i in incs]

    def compile_unit(unit):
        obj, src, defs, _ = unit
        out = os.path.join(OUT_DIR, obj)
        if not force and os.path.exists(out) and os.path.getmtime(out) >= max(newest, os.path.getmtime(src)):
            return out
        subprocess.run(["nvcc"] + common + defs + ["-c", src, "-o", out], check=True)
        return out

    jobs = jobs or max(1, min(6, (os.cpu_count() or 2) - 1))
    units = _units(ext)
    with concurrent.futures.ThreadPoolExecutor(jobs) as pool:
        objs = list(pool.map(compile_unit, units))
    sync_obj = os.path.join(OUT_DIR, "ref_sync.o")
    subprocess.run(["g++", "-std=c++17", "-O2", "-fPIC", "-I" + SHIMS, "-I" + ext, "-c",
                    os.path.join(ext, "CpuSynchronisationPoint.cpp"), "-o", sync_obj], check=True)
    for which, path in (("fit", LIB_FIT), ("convfit", LIB_CONVFIT)):
        mine = [o for o, u in zip(objs, units) if u[3] in (which, "both")]
        # -Bsymbolic: calls inside a library bind to that library's own definitions whatever else the process has loaded
        subprocess.run(["nvcc", "-shared", "-o", path] + mine + [sync_obj] +
                       ["-Xcompiler", "-fopenmp", "-L" + torch_lib, "-ltorch", "-ltorch_cpu", "-lc10",
                        "-Xlinker", "-Bsymbolic", "-Xlinker", "-rpath," + torch_lib], check=True)
    old = os.path.join(OUT_DIR, "libgmc_ref.so")
    if os.path.exists(old):
        os.remove(old)
    return LIB_PATH


if __name__ == "__main__":
    print(build(force=True))
