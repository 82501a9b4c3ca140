"""ctypes binding of libcider_b200.so (the C ABI declared in include/cider_b200.h).

This is the only place the shared library is loaded.  There is no CPU fallback:
if the library cannot be loaded the import fails loudly, exactly as the
reference's ``_load_ext`` does (cider/ops.py:31-47).
"""
from __future__ import annotations

import ctypes
import os
from ctypes import c_char_p, c_float, c_int, c_int64, c_size_t, c_void_p, POINTER, c_uint

_HERE = os.path.dirname(os.path.abspath(__file__))
DEFAULT_LIB = os.path.join(_HERE, "lib", "libcider_b200.so")

OK = 0
E_INVALID, E_SHAPE, E_WORKSPACE, E_ALIGNMENT, E_CUDA, E_UNSUPPORTED, E_DEVICE = -1, -2, -3, -4, -5, -6, -7
F32, F16 = 0, 1
OP_PERCHANNEL, OP_PERGROUP, OP_W4A8, OP_W4A8_ROWS, OP_W4A8_ROWS_INT8COPY = 1, 2, 3, 4, 5

# name -> (restype, argtypes); also the list the symbol-export test walks
SIGNATURES = {
    "cider_version": (c_int, []),
    "cider_last_error": (c_char_p, []),
    "cider_device_supported": (c_int, [c_int]),
    "cider_workspace_bytes": (c_size_t, [c_int, c_int64, c_int64, c_int64]),
    "cider_quantize_per_token": (c_int, [c_void_p, c_int64, c_int64, c_int64, c_void_p, c_void_p, c_void_p]),
    "cider_row_absmax": (c_int, [c_void_p, c_int64, c_int64, c_int64, c_void_p, c_void_p]),
    "cider_quantize_given_amax": (c_int, [c_void_p, c_int64, c_int64, c_int64, c_void_p, c_void_p, c_void_p,
                                          c_void_p]),
    "cider_int8_matmul_int32": (c_int, [c_void_p, c_void_p, c_void_p, c_int64, c_int64, c_int64, c_void_p]),
    "cider_perchannel_linear": (c_int, [c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_int64, c_int64,
                                        c_int64, c_void_p, c_size_t, c_void_p]),
    "cider_perchannel_linear_noalloc": (c_int, [c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_int64,
                                                c_int64, c_int64, c_void_p]),
    "cider_perchannel_linear_host": (c_int, [c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_int64, c_int64,
                                             c_int64, c_int64, c_void_p]),
    "cider_pergroup_linear": (c_int, [c_void_p, c_void_p, c_void_p, c_int, c_void_p, c_void_p, c_int64,
                                      c_int64, c_int64, c_int, c_void_p, c_size_t, c_void_p]),
    "cider_w4a8_linear": (c_int, [c_void_p, c_void_p, c_void_p, c_int, c_int, c_void_p, c_int64, c_int64,
                                  c_int64, c_void_p, c_size_t, c_void_p]),
    "cider_w4a8_repack": (c_int, [c_void_p, c_void_p, c_int64, c_int64, c_void_p]),
    "cider_w4a8_linear_nk4": (c_int, [c_void_p, c_void_p, c_void_p, c_int, c_int, c_void_p, c_int64, c_int64,
                                      c_int64, c_void_p, c_size_t, c_void_p]),
    "cider_linear_prequantized": (c_int, [c_void_p, c_void_p, c_void_p, c_void_p, c_int, c_int, c_void_p,
                                          c_void_p, c_int64, c_int64, c_int64, c_void_p]),
    "cider_rmsnorm_quant": (c_int, [c_void_p, c_void_p, c_float, c_int64, c_int64, c_void_p, c_void_p,
                                    c_void_p, c_void_p]),
    "cider_sdpa_decode": (c_int, [c_void_p, c_void_p, c_void_p, c_void_p, c_int64, c_int64, c_int64, c_int64,
                                  c_int64, c_int64, c_float, c_void_p, c_size_t, c_void_p, c_void_p]),
    "cider_quantize_heads": (c_int, [c_void_p, c_int64, c_int64, c_int64, c_int64, c_void_p, c_void_p, c_void_p]),
    "cider_silu_mul_quant": (c_int, [c_void_p, c_int64, c_int64, c_void_p, c_void_p, c_void_p]),
    "cider_swiglu_linear_prequantized": (c_int, [c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p,
                                                 c_int64, c_int64, c_int64, c_void_p]),
    "cider_quantize_consume_amax": (c_int, [c_void_p, c_int64, c_int64, c_int64, c_void_p, c_void_p, c_void_p, c_void_p]),
    "cider_sdpa_decode_tickets": (c_int, [c_void_p, c_void_p, c_void_p, c_void_p, c_int64, c_int64, c_int64,
                                          c_int64, c_int64, c_int64, c_float, c_void_p, c_size_t, c_void_p,
                                          c_void_p, c_void_p]),
    "cider_sdpa_decode_fused": (c_int, [c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_int64, c_float,
                                        c_void_p, c_void_p, c_void_p, c_int64, c_int64, c_int64, c_int64, c_int64,
                                        c_int64, c_float, c_void_p, c_size_t, c_void_p, c_void_p, c_void_p]),
    "cider_add_rmsnorm_quant": (c_int, [c_void_p, c_void_p, c_void_p, c_float, c_int64, c_int64, c_void_p,
                                        c_void_p, c_void_p, c_void_p]),
    "cider_qk_norm_rope_append": (c_int, [c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_int64,
                                          c_void_p, c_int64, c_float, c_void_p, c_void_p, c_void_p, c_int64,
                                          c_int64, c_int64, c_int64, c_int64, c_int64, c_void_p]),
    "cider_silu_mul": (c_int, [c_void_p, c_void_p, c_int64, c_int64, c_void_p]),
    "cider_linear_m1_fused": (c_int, [c_void_p, c_int, c_void_p, c_void_p, c_float, c_void_p, c_void_p, c_void_p,
                                      c_int, c_int, c_void_p, c_void_p, c_int64, c_int64, c_void_p]),
    "cider_sdpa_decode_workspace_bytes": (c_size_t, [c_int64, c_int64, c_int64, c_int64, c_int64]),
    "cider_device_status": (c_int, [POINTER(c_uint)]),
    "cider_clear_device_status": (c_int, []),
    "cider_set_gemm_backend": (c_int, [c_int]),
    "cider_testing_set_tile": (c_int, [c_int, c_int]),
    "cider_testing_last_gemm_kernel": (c_char_p, []),
    "cider_testing_set_sdpa_kernel": (c_int, [c_int]),
    "cider_set_programmatic_launch": (c_int, [c_int]),
    "cider_peer_max_bytes": (c_size_t, [c_size_t]),
    "cider_peer_alloc": (c_int, [c_size_t, POINTER(c_void_p), c_void_p]),
    "cider_peer_open": (c_int, [c_void_p, POINTER(c_void_p)]),
    "cider_peer_close": (c_int, [c_void_p]),
    "cider_peer_free": (c_int, [c_void_p]),
    "cider_peer_reset": (c_int, [c_void_p, c_void_p]),
    "cider_allreduce_f16": (c_int, [c_void_p, c_void_p, c_int64, c_int, c_int, POINTER(c_void_p), c_size_t,
                                    c_int64, c_void_p]),
    "cider_allreduce_add_rmsnorm_quant": (c_int, [c_void_p, c_void_p, c_void_p, c_float, c_int64, c_int64, c_void_p,
                                                  c_void_p, c_void_p, c_int, c_int, POINTER(c_void_p), c_size_t,
                                                  c_int64, c_void_p]),
    "cider_testing_allreduce_norm_emulated": (c_int, [POINTER(c_void_p), POINTER(c_void_p), c_void_p, c_float,
                                                      c_int64, c_int64, POINTER(c_void_p), POINTER(c_void_p),
                                                      POINTER(c_void_p), c_int, POINTER(c_void_p), c_size_t,
                                                      c_void_p]),
    "cider_testing_allreduce_emulated": (c_int, [POINTER(c_void_p), POINTER(c_void_p), c_int64, c_int,
                                                 POINTER(c_void_p), c_size_t, c_int64, c_int, c_void_p]),
}

_lib = None


class CiderError(RuntimeError):
    """A C-ABI call returned a non-zero status."""

    def __init__(self, code: int, message: str):
        super().__init__(f"cider_b200 error {code}: {message}")
        self.code = code


def lib_path() -> str:
    return os.environ.get("CIDER_B200_LIB", DEFAULT_LIB)


def load() -> ctypes.CDLL:
    """Load the library (once).  Raises RuntimeError when it is missing."""
    global _lib
    if _lib is not None:
        return _lib
    path = lib_path()
    if not os.path.exists(path):
        raise RuntimeError(
            f"cider_b200 CUDA library not found at {path}. Build it with "
            "`python -m cider_b200.csrc.build` (needs nvcc); there is no CPU fallback.")
    lib = ctypes.CDLL(path)
    for name, (res, args) in SIGNATURES.items():
        fn = getattr(lib, name)  # AttributeError if the symbol is not exported
        fn.restype = res
        fn.argtypes = args
    _lib = lib
    return lib


def last_error() -> str:
    return load().cider_last_error().decode("utf-8", "replace")


def check(code: int) -> None:
    """Map a status code to the exception class the reference would raise:
    std::invalid_argument -> ValueError, everything else -> RuntimeError."""
    if code == OK:
        return
    msg = last_error()
    if code in (E_INVALID, E_SHAPE, E_ALIGNMENT):
        raise ValueError(f"cider_b200: {msg}")
    raise CiderError(code, msg)
