"""Build libcider_b200.so (sm_100a only) with nvcc, in-tree.

    python -m cider_b200.csrc.build [--force] [--verbose]

nvcc cross-compiles without a GPU.  The arch is passed as an explicit -gencode
so that tcgen05 / TMA instructions (sm_100a features) are accepted.
"""
import os
import subprocess
import sys

HERE = os.path.dirname(os.path.abspath(__file__))
ROOT = os.path.dirname(os.path.dirname(HERE))
SOURCES = ["api.cu", "quantize.cu", "gemm_generic.cu", "gemm_tc.cu", "gemv.cu", "sdpa_decode.cu",
           "noalloc.cu", "decoder_glue.cu", "host_pipeline.cu"]
HEADERS = ["common.cuh", os.path.join(ROOT, "include", "cider_b200.h")]
OUT_DIR = os.path.join(os.path.dirname(HERE), "lib")
OUT = os.path.join(OUT_DIR, "libcider_b200.so")

NVCC_FLAGS = [
    "-gencode", "arch=compute_100a,code=sm_100a", "-lineinfo", "-O3", "-std=c++17",
    "-Xcompiler", "-fPIC",
    "-shared", "-cudart", "static",
]


def _stale() -> bool:
    if not os.path.exists(OUT):
        return True
    t = os.path.getmtime(OUT)
    deps = [os.path.join(HERE, s) for s in SOURCES] + [h if os.path.isabs(h) else os.path.join(HERE, h) for h in HEADERS]
    deps.append(os.path.abspath(__file__))
    return any(os.path.getmtime(d) > t for d in deps)


def build(force: bool = False, verbose: bool = False) -> str:
    if not force and not _stale():
        return OUT
    os.makedirs(OUT_DIR, exist_ok=True)
    nvcc = os.environ.get("NVCC", "nvcc")
    cmd = [nvcc, *NVCC_FLAGS]
    if verbose:
        cmd += ["-Xptxas", "-v"]
    cmd += [os.path.join(HERE, s) for s in SOURCES] + ["-o", OUT]
    subprocess.run(cmd, check=True)
    return OUT


if __name__ == "__main__":
    print(build(force="--force" in sys.argv, verbose="--verbose" in sys.argv))
