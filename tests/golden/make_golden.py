"""Generate the golden fixtures in this directory from the reference itself.

Run where the reference checkout is available:

    python tests/golden/make_golden.py /path/to/cider

What can be taken from the reference:

* its numpy weight-quantization helpers (cider/ops.py:73-116, cider/nn.py:34-59)
  import and run anywhere once ``mlx`` is stubbed (only type annotations and
  module-level imports touch it) -> ``weight_quant.npz``;
* its only correctness test, benchmarks/test_bitexact.py:19-58, draws its
  operands from ``np.random.seed(42)`` / ``randint(-128, 128)`` and compares with
  an int64 numpy matmul.  Those operands regenerate bit-identically anywhere, so
  the fixture stores the shapes and a SHA-256 of each expected int32 product
  computed exactly as the test computes it -> ``bitexact_int32.json``.

Nothing else on the path has a test or vector in the reference (its GPU kernels
are Metal and its primitives' eval_cpu throws), so there is nothing else to
record.  Reference sources are read, never copied.
"""
import hashlib
import importlib.util
import json
import os
import sys
import types

import numpy as np

HERE = os.path.dirname(os.path.abspath(__file__))


def load_reference(root: str):
    mx_core = types.ModuleType("mlx.core")
    mx_core.array = object
    mx_core.Stream = object
    mx_nn = types.ModuleType("mlx.nn")
    mx_nn.Module = type("Module", (), {})
    mx_nn.Linear = type("Linear", (mx_nn.Module,), {})
    mx_nn.QuantizedLinear = type("QuantizedLinear", (mx_nn.Module,), {})
    mlx = types.ModuleType("mlx")
    mlx.core, mlx.nn = mx_core, mx_nn
    sys.modules.update({"mlx": mlx, "mlx.core": mx_core, "mlx.nn": mx_nn})
    pkg = os.path.join(root, "cider")
    spec = importlib.util.spec_from_file_location(
        "cider", os.path.join(pkg, "__init__.py"), submodule_search_locations=[pkg])
    mod = importlib.util.module_from_spec(spec)
    sys.modules["cider"] = mod
    spec.loader.exec_module(mod)
    import cider.nn
    import cider.ops
    return mod


# shapes of benchmarks/test_bitexact.py:19-35, (M, K, N)
BITEXACT_SHAPES = [
    (1, 2, 2), (2, 4, 2), (1, 128, 128), (1, 4096, 4096), (4, 2048, 2048),
    (16, 4096, 4096), (32, 4096, 4096), (64, 4096, 4096), (128, 4096, 4096),
    (16, 4096, 8192), (16, 8192, 4096), (64, 2048, 4096), (7, 513, 1025),
    (33, 4097, 4095),
]


def bitexact_operands(M, K, N):
    np.random.seed(42)
    a = np.random.randint(-128, 128, (M, K), dtype=np.int8)
    b = np.random.randint(-128, 128, (N, K), dtype=np.int8)
    return a, b


def main(root: str):
    ref = load_reference(root)
    rng = np.random.default_rng(1234)
    out = {}
    # per-channel int8, incl. an all-zero row and exact-tie values
    w = (rng.standard_normal((24, 96)) * 0.02).astype(np.float32)
    w[3] = 0.0
    w[5, :8] = np.array([0.5, 1.5, 2.5, -0.5, -1.5, -2.5, 127.0, -127.0], np.float32)
    out["pc_w"] = w
    out["pc_q"], out["pc_scale"] = ref.ops.quantize_weight_int8(w)
    # fp16 input as a converted checkpoint would provide it
    w16 = (rng.standard_normal((16, 128)) * 0.02).astype(np.float16)
    out["pc16_w"] = w16
    out["pc16_q"], out["pc16_scale"] = ref.ops.quantize_weight_int8(w16)
    # per-group
    for gs in (64, 128, 256):
        wg = (rng.standard_normal((12, 512)) * 0.02).astype(np.float32)
        wg[2, :gs] = 0.0
        out[f"pg{gs}_w"] = wg
        out[f"pg{gs}_q"], out[f"pg{gs}_scale"] = ref.nn._symmetric_quantize_pergroup(wg, gs)
    # packed int4, [K, N]
    w4 = (rng.standard_normal((64, 20)) * 0.02).astype(np.float32)
    w4[:, 4] = 0.0
    out["w4_w"] = w4
    out["w4_packed"], out["w4_scale"] = ref.ops.pack_weight_int4(w4)
    np.savez_compressed(os.path.join(HERE, "weight_quant.npz"), **out)

    recs = []
    for (M, K, N) in BITEXACT_SHAPES:
        a, b = bitexact_operands(M, K, N)
        c = (a.astype(np.int64) @ b.astype(np.int64).T).astype(np.int32)
        recs.append({"M": M, "K": K, "N": N,
                     "sha256": hashlib.sha256(c.tobytes()).hexdigest(),
                     "c00": int(c[0, 0]), "c_last": int(c[-1, -1])})
    with open(os.path.join(HERE, "bitexact_int32.json"), "w") as f:
        json.dump({"source": "benchmarks/test_bitexact.py:19-58", "seed": 42,
                   "cases": recs}, f, indent=1)
    print("wrote", sorted(out), len(recs), "bitexact cases")


if __name__ == "__main__":
    if len(sys.argv) != 2:
        sys.exit("usage: python make_golden.py <path of a checkout of the reference (Mininglamp-AI/cider)>")
    main(sys.argv[1])
