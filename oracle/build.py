"""Build recipe for the CPU oracle shared library (test infrastructure).

    python -m oracle.build

compiles oracle/cider_oracle.c with gcc into oracle/libcider_oracle.so.  The
flags matter for parity: -ffp-contract=off keeps gcc from fusing anything the
source did not fuse explicitly with fmaf(), and no -ffast-math / -march flag is
given so that the library built on one x86-64 machine runs on another (the hot
loops carry target_clones for AVX2 / AVX-512 dispatch at load time).

The reference's own implementation of the path is Metal + Objective-C++ against
MLX's Metal backend (CMakeLists.txt:3,42-46); it cannot be compiled with gcc, so
there is no oracle/_ref build.
"""
import os
import subprocess
import sys

HERE = os.path.dirname(os.path.abspath(__file__))
SRC = os.path.join(HERE, "cider_oracle.c")
OUT = os.path.join(HERE, "libcider_oracle.so")

FLAGS = ["-O3", "-fPIC", "-shared", "-fopenmp", "-ffp-contract=off",
         "-fno-fast-math", "-Wall", "-Wno-unknown-pragmas"]


def build(force: bool = False) -> str:
    if (not force and os.path.exists(OUT)
            and os.path.getmtime(OUT) >= os.path.getmtime(SRC)):
        return OUT
    cmd = ["gcc", *FLAGS, SRC, "-o", OUT, "-lm"]
    subprocess.run(cmd, check=True)
    return OUT


if __name__ == "__main__":
    print(build(force="--force" in sys.argv))
