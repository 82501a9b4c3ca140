"""Build libcider_b200.so (sm_100a only) with nvcc, in-tree.

    python -m cider_b200.csrc.build [--force] [--verbose]

nvcc cross-compiles without a GPU.  The arch is passed as an explicit -gencode
so that tcgen05 / TMA instructions (sm_100a features) are accepted.  Each source
is compiled to an object file of its own (in parallel, only when it or a header
is newer than its object) and the objects are linked into the shared library.
"""
import os
import subprocess
import sys
from concurrent.futures import ThreadPoolExecutor

HERE = os.path.dirname(os.path.abspath(__file__))
ROOT = os.path.dirname(os.path.dirname(HERE))
SOURCES = ["api.cu", "quantize.cu", "gemm_generic.cu", "gemm_tc.cu", "gemv.cu", "sdpa_decode.cu",
           "noalloc.cu", "decoder_glue.cu", "host_pipeline.cu", "peer_reduce.cu"]
HEADERS = ["common.cuh", os.path.join(ROOT, "include", "cider_b200.h"),
           os.path.join(ROOT, "include", "cider_b200_testing.h")]
OUT_DIR = os.path.join(os.path.dirname(HERE), "lib")
OBJ_DIR = os.path.join(OUT_DIR, "obj")
OUT = os.path.join(OUT_DIR, "libcider_b200.so")

NVCC_FLAGS = ["-gencode", "arch=compute_100a,code=sm_100a", "-lineinfo", "-O3", "-std=c++17",
              "-Xcompiler", "-fPIC"]
LINK_FLAGS = ["-gencode", "arch=compute_100a,code=sm_100a", "-shared", "-cudart", "static", "-Xcompiler", "-fPIC"]


def _header_paths():
    return [h if os.path.isabs(h) else os.path.join(HERE, h) for h in HEADERS]


def _newer_than(target: str, deps) -> bool:
    if not os.path.exists(target):
        return True
    t = os.path.getmtime(target)
    return any(os.path.getmtime(d) > t for d in deps)


def build(force: bool = False, verbose: bool = False) -> str:
    os.makedirs(OBJ_DIR, exist_ok=True)
    nvcc = os.environ.get("NVCC", "nvcc")
    common = _header_paths() + [os.path.abspath(__file__)]
    jobs = []
    for s in SOURCES:
        src = os.path.join(HERE, s)
        obj = os.path.join(OBJ_DIR, s[:-3] + ".o")
        if force or _newer_than(obj, [src] + common):
            cmd = [nvcc, *NVCC_FLAGS] + (["-Xptxas", "-v"] if verbose else []) + ["-c", src, "-o", obj]
            jobs.append(cmd)

    def run(cmd):
        r = subprocess.run(cmd, capture_output=True, text=True)
        return cmd, r

    if jobs:
        with ThreadPoolExecutor(max_workers=min(len(jobs), os.cpu_count() or 4)) as ex:
            for cmd, r in ex.map(run, jobs):
                if verbose or r.returncode != 0:
                    sys.stderr.write(r.stdout + r.stderr)
                if r.returncode != 0:
                    raise subprocess.CalledProcessError(r.returncode, cmd)
    objs = [os.path.join(OBJ_DIR, s[:-3] + ".o") for s in SOURCES]
    if jobs or _newer_than(OUT, objs):
        subprocess.run([nvcc, *LINK_FLAGS, *objs, "-o", OUT], check=True)
    return OUT


if __name__ == "__main__":
    print(build(force="--force" in sys.argv, verbose="--verbose" in sys.argv))
