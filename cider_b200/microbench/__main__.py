import os
import subprocess
import sys

HERE = os.path.dirname(os.path.abspath(__file__))
NAMES = ["mma_rate", "hbm_stream", "tmem_ld_rate"]


def build(name: str) -> str:
    src, exe = os.path.join(HERE, name + ".cu"), os.path.join(HERE, name)
    if not os.path.exists(exe) or os.path.getmtime(exe) < os.path.getmtime(src):
        subprocess.run([os.environ.get("NVCC", "nvcc"), "-gencode", "arch=compute_100a,code=sm_100a", "-O3",
                        "-std=c++17", "-o", exe, src], check=True)
    return exe


def main():
    names = sys.argv[1:] or NAMES
    for n in names:
        if n not in NAMES:
            raise SystemExit(f"unknown micro-benchmark {n!r}; choose from {NAMES}")
        exe = build(n)
        print(f"# {n}", flush=True)
        subprocess.run([exe], check=True)


if __name__ == "__main__":
    main()
