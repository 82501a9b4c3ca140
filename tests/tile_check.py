"""Helper run as a subprocess by test_gpu_parity.py::test_forced_tile_kernels.

    python tile_check.py TILE [BN]

The tensor-core GEMM picks its tile shape from the problem size; the testing
setter cider_testing_set_tile forces the single-CTA 128-row kernel (TILE 128,
optionally with its N tile BN) or the CTA-pair kernel (TILE 2) so that each can
be checked on shapes the heuristic would not give it (ragged M / N / K tails,
fewer tiles than SMs).  A process of its own, so that the process-wide override
cannot leak into other tests.  Prints one line per case and exits non-zero on the
first mismatch with the CPU oracle.
"""
import os
import sys

import numpy as np
import torch

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
sys.path.insert(0, ROOT)
sys.path.insert(0, os.path.dirname(os.path.abspath(__file__)))

import oracle  # noqa: E402
from cider_b200 import _lib, ops  # noqa: E402
from conftest import make_activations, make_weight  # noqa: E402

SHAPES = [(256, 256, 128), (300, 1000, 1008), (129, 257, 144), (8, 8, 128), (1024, 768, 2560),
          (513, 520, 4096), (2048, 2560, 640), (33, 1004, 256), (700, 4100, 384)]


def main():
    lib = _lib.load()
    lib.cider_set_gemm_backend(2)
    tile = int(sys.argv[1]) if len(sys.argv) > 1 else 0
    bn = int(sys.argv[2]) if len(sys.argv) > 2 else 0
    assert lib.cider_testing_set_tile(tile, bn) == 0
    dev = "cuda:0"
    for (M, N, K) in SHAPES:
        rng = np.random.default_rng(M + N + K)
        a = rng.integers(-128, 128, (M, K), dtype=np.int8)
        b = rng.integers(-128, 128, (N, K), dtype=np.int8)
        c = ops.int8_matmul_int32(torch.from_numpy(a).to(dev), torch.from_numpy(b).to(dev)).cpu().numpy()
        ok1 = np.array_equal(c, oracle.c_int8_matmul_int32(a, b))
        x = make_activations(M, K, seed=M)
        wq, sw = oracle.np_quantize_weight_int8(make_weight(N, K, seed=N))
        bias = (rng.standard_normal(N) * 0.05).astype(np.float16)
        y = ops.perchannel_linear(torch.from_numpy(x).to(dev), torch.from_numpy(wq).to(dev),
                                  torch.from_numpy(sw).to(dev), torch.from_numpy(bias).to(dev)).cpu().numpy()
        ok2 = M == 1 or np.array_equal(y, oracle.c_perchannel_linear(x, wq, sw, bias))
        print((M, N, K), "int32", "ok" if ok1 else "MISMATCH", "linear", "ok" if ok2 else "MISMATCH", flush=True)
        if not (ok1 and ok2):
            return 1
    import ctypes
    st = ctypes.c_uint(0)
    lib.cider_device_status(st)
    print("device status", st.value)
    return 0 if st.value == 0 else 2


if __name__ == "__main__":
    sys.exit(main())
