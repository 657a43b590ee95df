"""TEST INFRASTRUCTURE. Builds the CPU oracle (oracle/cpu/*.c, *.cpp) into oracle/_build/liboracle.so with gcc/g++.

The reference's own native sources are built separately by oracle/build_ref.py into oracle/_ref/.
"""
import os
import subprocess

HERE = os.path.dirname(os.path.abspath(__file__))
SRC = os.path.join(HERE, "cpu")
OUT_DIR = os.path.join(HERE, "_build")
LIB_PATH = os.path.join(OUT_DIR, "liboracle.so")

# x86-64-v3 (AVX2 + FMA) instead of -march=native: the object built on one machine is also run on another.
# -ffast-math -fno-finite-math-only are the reference's own host flags
# (src/gmc/cpp/extensions/compile_flags.py:15); the Morton stage is compiled without them.
FAST = ["-O3", "-march=x86-64-v3", "-fopenmp", "-fPIC", "-ffast-math", "-fno-finite-math-only"]
IEEE = ["-O2", "-march=x86-64-v3", "-fopenmp", "-fPIC", "-ffp-contract=off"]
IEEE_FILES = {"lbvh.cpp", "mhem_fit.cpp", "convolution_fitting.cpp"}


def build(force: bool = False) -> str:
    os.makedirs(OUT_DIR, exist_ok=True)
    srcs = sorted(f for f in os.listdir(SRC) if f.endswith((".c", ".cpp")))
    newest = max(os.path.getmtime(os.path.join(SRC, f)) for f in os.listdir(SRC))
    if not force and os.path.exists(LIB_PATH) and os.path.getmtime(LIB_PATH) >= newest:
        return LIB_PATH
    objs = []
    for s in srcs:
        obj = os.path.join(OUT_DIR, s.rsplit(".", 1)[0] + ".o")
        cc = "g++" if s.endswith(".cpp") else "gcc"
        flags = IEEE if s in IEEE_FILES else FAST
        if s.endswith(".cpp"):
            flags = flags + ["-std=c++17"]
        subprocess.run([cc] + flags + ["-c", os.path.join(SRC, s), "-o", obj], check=True)
        objs.append(obj)
    subprocess.run(["g++", "-shared", "-fopenmp", "-o", LIB_PATH] + objs + ["-lm"], check=True)
    return LIB_PATH


if __name__ == "__main__":
    print(build(force=True))
