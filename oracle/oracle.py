"""Python face of the CPU oracle (test infrastructure, never on the product path).

Two independent restatements of the reference semantics live here:

* ``c_*``  - thin ctypes wrappers over oracle/cider_oracle.c (fast, OpenMP, the
  one the GPU parity tests and the timed CPU baseline use);
* ``np_*`` - a numpy restatement used to cross-check the C code on small cases.

Parity pinning: the raw integer GEMM is pinned by the reference's own bit-exact
test (benchmarks/test_bitexact.py:19-58) and the weight-quant helpers by
fixtures generated from the reference's numpy code (tests/golden).  Everything
else (activation quant, fused dequant, MV, W4A8) has no test in the reference:
"parity unpinned", restated from the Metal sources cited at each function.
"""
from __future__ import annotations

import ctypes
import os

import numpy as np

from . import build as _build

__all__ = [
    "lib", "num_threads", "set_num_threads",
    "c_quantize_per_token", "c_int8_matmul_int32", "c_perchannel_linear",
    "c_dequant_perchannel", "c_pergroup_linear", "c_w4a8_linear", "c_unpack_w4",
    "c_rmsnorm", "c_sdpa_decode",
    "np_round_half_away", "np_quantize_per_token", "np_int8_matmul_int32",
    "np_perchannel_linear", "np_pergroup_linear", "np_w4a8_linear",
    "np_unpack_w4", "np_quantize_weight_int8", "np_quantize_weight_pergroup",
    "np_pack_weight_int4", "np_pack_weight_int4_pergroup",
]

_lib = None


def lib() -> ctypes.CDLL:
    global _lib
    if _lib is None:
        path = _build.OUT
        if not os.path.exists(path):
            path = _build.build()
        _lib = ctypes.CDLL(path)
        _lib.cider_oracle_version.restype = ctypes.c_int
        _lib.cider_oracle_num_threads.restype = ctypes.c_int
    return _lib


def num_threads() -> int:
    return int(lib().cider_oracle_num_threads())


def set_num_threads(n: int) -> None:
    """OpenMP threads of the following oracle calls (0 or less: leave as is)."""
    f = lib().cider_oracle_set_num_threads
    f.argtypes = [ctypes.c_int]
    f.restype = None
    f(int(n))


def _p(a: np.ndarray):
    return a.ctypes.data_as(ctypes.c_void_p)


def _c(a, dtype) -> np.ndarray:
    a = np.ascontiguousarray(a)
    assert a.dtype == dtype, (a.dtype, dtype)
    return a


_i64 = ctypes.c_int64


# ----------------------------------------------------------------- C wrappers

def c_quantize_per_token(x: np.ndarray):
    """S1: fp16 [M,K] -> (int8 [M,K], fp32 [M]).  w8a8_quantize.metal:34-86."""
    x = _c(x, np.float16)
    M, K = x.shape
    q = np.empty((M, K), np.int8)
    s = np.empty((M,), np.float32)
    lib().cider_oracle_quantize_per_token(_p(x), _i64(M), _i64(K), _i64(K), _p(q), _p(s))
    return q, s


def c_int8_matmul_int32(a: np.ndarray, b: np.ndarray) -> np.ndarray:
    """S2: int8 [M,K] x int8 [N,K]^T -> int32 [M,N].  w8a8_matmul.metal:301-453."""
    a = _c(a, np.int8)
    b = _c(b, np.int8)
    M, K = a.shape
    N = b.shape[0]
    assert b.shape[1] == K
    c = np.empty((M, N), np.int32)
    lib().cider_oracle_int8_matmul_int32(_p(a), _p(b), _p(c), _i64(M), _i64(N), _i64(K))
    return c


def c_perchannel_linear(x, w, sw, bias=None) -> np.ndarray:
    """S3 (M>1) / S5 (M==1).  w8a8_matmul.metal:63-81, w8a8_int8_mv.metal:34-69."""
    x = _c(x, np.float16)
    w = _c(w, np.int8)
    sw = _c(sw, np.float32)
    M, K = x.shape
    N = w.shape[0]
    assert w.shape[1] == K and sw.shape == (N,)
    y = np.empty((M, N), np.float16)
    b = None if bias is None else _c(bias, np.float16)
    lib().cider_oracle_perchannel_linear(_p(x), _p(w), _p(sw),
                                         _p(b) if b is not None else None,
                                         _p(y), _i64(M), _i64(N), _i64(K))
    return y


def c_dequant_perchannel(acc, sa, sw, bias=None) -> np.ndarray:
    acc = _c(acc, np.int32)
    sa = _c(sa, np.float32)
    sw = _c(sw, np.float32)
    M, N = acc.shape
    y = np.empty((M, N), np.float16)
    b = None if bias is None else _c(bias, np.float16)
    lib().cider_oracle_dequant_perchannel(_p(acc), _p(sa), _p(sw),
                                          _p(b) if b is not None else None,
                                          _p(y), _i64(M), _i64(N))
    return y


def c_pergroup_linear(x, w, sw, group_size, bias=None) -> np.ndarray:
    """S4 (M>1) / S6 (M==1); sw is [K/gs, N], any float dtype (upcast to fp32)."""
    x = _c(x, np.float16)
    w = _c(w, np.int8)
    sw = np.ascontiguousarray(np.asarray(sw).astype(np.float32))
    M, K = x.shape
    N = w.shape[0]
    assert K % group_size == 0 and sw.shape == (K // group_size, N)
    y = np.empty((M, N), np.float16)
    b = None if bias is None else _c(bias, np.float16)
    lib().cider_oracle_pergroup_linear(_p(x), _p(w), _p(sw),
                                       _p(b) if b is not None else None, _p(y),
                                       _i64(M), _i64(N), _i64(K), _i64(group_size))
    return y


def c_unpack_w4(packed: np.ndarray) -> np.ndarray:
    """S7 unpack: [K/2,N] uint8 -> int8 [N,K].  w4a8_matmul.metal:47-70."""
    packed = _c(packed, np.uint8)
    K2, N = packed.shape
    w = np.empty((N, 2 * K2), np.int8)
    lib().cider_oracle_unpack_w4(_p(packed), _p(w), _i64(N), _i64(2 * K2))
    return w


def c_w4a8_linear(x, packed, sw, group_size=0) -> np.ndarray:
    """S7.  group_size 0: sw [N] (reference); >0: sw [K/gs,N] (extension)."""
    x = _c(x, np.float16)
    packed = _c(packed, np.uint8)
    sw = np.ascontiguousarray(np.asarray(sw).astype(np.float32))
    M, K = x.shape
    N = packed.shape[1]
    assert packed.shape[0] * 2 == K
    if group_size == 0:
        assert sw.shape == (N,)
    else:
        assert sw.shape == (K // group_size, N)
    y = np.empty((M, N), np.float16)
    lib().cider_oracle_w4a8_linear(_p(x), _p(packed), _p(sw), _p(y), _i64(M),
                                   _i64(N), _i64(K), _i64(group_size))
    return y


def c_rmsnorm(x, w, eps: float) -> np.ndarray:
    x = _c(x, np.float16)
    w = _c(w, np.float16)
    M, K = x.shape
    y = np.empty_like(x)
    lib().cider_oracle_rmsnorm(_p(x), _p(w), _p(y), _i64(M), _i64(K), ctypes.c_float(eps))
    return y


def c_sdpa_decode(q, kc, vc, T: int, scale: float) -> np.ndarray:
    """q [B,Hq,D]; kc/vc [B,Hkv,Tcap,D] fp16; attends to the first T positions."""
    q = _c(q, np.float16)
    kc = _c(kc, np.float16)
    vc = _c(vc, np.float16)
    B, Hq, D = q.shape
    _, Hkv, Tcap, _ = kc.shape
    out = np.empty_like(q)
    lib().cider_oracle_sdpa_decode(_p(q), _p(kc), _p(vc), _p(out), _i64(B), _i64(Hq),
                                   _i64(Hkv), _i64(D), _i64(T), _i64(Tcap),
                                   ctypes.c_float(scale))
    return out


# ------------------------------------------------------- numpy restatement

def np_round_half_away(v: np.ndarray) -> np.ndarray:
    """Metal round(): half away from zero (np.round is half-to-even).  Written
    with an exact fractional part: floor(|v| + 0.5) in fp32 would round the
    largest float below 0.5 up to 1."""
    a = np.abs(v)
    fl = np.floor(a)
    return np.sign(v) * (fl + ((a - fl) >= np.float32(0.5)))


def np_quantize_per_token(x: np.ndarray):
    xf = x.astype(np.float32)
    amax = np.max(np.abs(xf), axis=1) if xf.shape[1] else np.zeros(xf.shape[0], np.float32)
    s = (amax / np.float32(127.0)).astype(np.float32)
    s[s == 0] = np.float32(1.0)
    inv = (np.float32(1.0) / s).astype(np.float32)
    v = (xf * inv[:, None]).astype(np.float32)
    q = np.clip(np_round_half_away(v), -128, 127).astype(np.int8)
    return q, s


def np_int8_matmul_int32(a: np.ndarray, b: np.ndarray) -> np.ndarray:
    # exact: every partial sum is an integer far below 2^53
    return (a.astype(np.float64) @ b.astype(np.float64).T).astype(np.int64).astype(np.int32)


def _fma32(a, b, c):
    """fp32 fused multiply-add emulated in extended precision (a*b is exact)."""
    r = a.astype(np.longdouble) * b.astype(np.longdouble) + c.astype(np.longdouble)
    return r.astype(np.float32)


def np_perchannel_linear(x, w, sw, bias=None):
    M = x.shape[0]
    N = w.shape[0]
    b = np.zeros(N, np.float32) if bias is None else bias.astype(np.float32)
    if M == 1:
        dot = (w.astype(np.float64) @ x[0].astype(np.float64)).astype(np.float32)
        return _fma32(sw.astype(np.float32), dot, b).astype(np.float16)[None, :]
    q, sa = np_quantize_per_token(x)
    acc = np_int8_matmul_int32(q, w)
    t = (acc.astype(np.float32) * sa[:, None]).astype(np.float32)
    return _fma32(t, np.broadcast_to(sw.astype(np.float32), t.shape),
                  np.broadcast_to(b, t.shape)).astype(np.float16)


def np_pergroup_linear(x, w, sw, group_size, bias=None):
    M, K = x.shape
    N = w.shape[0]
    G = K // group_size
    sw = sw.astype(np.float32)
    b = np.zeros(N, np.float32) if bias is None else bias.astype(np.float32)
    if M == 1:
        acc = np.zeros(N, np.float64)
        for g in range(G):
            sl = slice(g * group_size, (g + 1) * group_size)
            acc += sw[g].astype(np.float64) * (w[:, sl].astype(np.float64) @ x[0, sl].astype(np.float64))
        return (acc.astype(np.float32) + b).astype(np.float16)[None, :]
    q, sa = np_quantize_per_token(x)
    accf = np.zeros((M, N), np.float32)
    for g in range(G):
        sl = slice(g * group_size, (g + 1) * group_size)
        acc = np_int8_matmul_int32(q[:, sl], w[:, sl]).astype(np.float32)
        accf = _fma32(acc, np.broadcast_to(sw[g], acc.shape), accf)
    return _fma32(accf, np.broadcast_to(sa[:, None], accf.shape),
                  np.broadcast_to(b, accf.shape)).astype(np.float16)


def np_unpack_w4(packed: np.ndarray) -> np.ndarray:
    K2, N = packed.shape
    w = np.empty((2 * K2, N), np.int8)
    w[0::2] = (packed >> 4).astype(np.int8) - 8
    w[1::2] = (packed & 15).astype(np.int8) - 8
    return np.ascontiguousarray(w.T)  # [N, K]


def np_w4a8_linear(x, packed, sw, group_size=0):
    w = np_unpack_w4(packed)
    M, K = x.shape
    q, sa = np_quantize_per_token(x)
    sw = sw.astype(np.float32)
    if group_size == 0:
        acc = np_int8_matmul_int32(q, w).astype(np.float32)
        return ((acc * sa[:, None]).astype(np.float32) * sw[None, :]).astype(np.float32).astype(np.float16)
    accf = np.zeros((M, w.shape[0]), np.float32)
    for g in range(K // group_size):
        sl = slice(g * group_size, (g + 1) * group_size)
        acc = np_int8_matmul_int32(q[:, sl], w[:, sl]).astype(np.float32)
        accf = _fma32(acc, np.broadcast_to(sw[g], acc.shape), accf)
    return (accf * sa[:, None]).astype(np.float32).astype(np.float16)


# ---- S8: offline weight quantization (cider/ops.py:73-116, cider/nn.py:34-59)

def np_quantize_weight_int8(w: np.ndarray):
    w = w.astype(np.float32)
    scale = np.max(np.abs(w), axis=1) / 127.0
    scale = np.where(scale == 0, 1.0, scale)
    q = np.clip(np.round(w / scale[:, None]), -128, 127).astype(np.int8)
    return q, scale.astype(np.float32)


def np_quantize_weight_pergroup(w: np.ndarray, group_size: int):
    N, K = w.shape
    G = K // group_size
    wr = w.astype(np.float32).reshape(N, G, group_size)
    scale = np.max(np.abs(wr), axis=2) / 127.0
    scale = np.where(scale == 0, 1.0, scale)
    q = np.clip(np.round(wr / scale[:, :, None]), -128, 127).astype(np.int8).reshape(N, K)
    return q, scale.astype(np.float32)  # [N, G]; callers transpose to [G, N]


def np_pack_weight_int4(w_kn: np.ndarray, zero_point: int = 8):
    w = w_kn.astype(np.float32)
    scale = np.max(np.abs(w), axis=0) / 7.0
    scale = np.where(scale == 0, 1.0, scale)
    q = np.clip(np.round(w / scale[None, :]) + zero_point, 0, 15).astype(np.uint8)
    return (q[0::2] << 4) | q[1::2], scale.astype(np.float32)


def np_pack_weight_int4_pergroup(w_kn: np.ndarray, group_size: int, scale_dtype=np.float16):
    """Group-wise int4 (extension): scales [K/gs, N] rounded to ``scale_dtype``
    BEFORE quantizing, so the stored scale is the one the weights were divided by."""
    K, N = w_kn.shape
    G = K // group_size
    w = w_kn.astype(np.float32).reshape(G, group_size, N)
    scale = (np.max(np.abs(w), axis=1) / 7.0).astype(scale_dtype)
    scale = np.where(scale == 0, scale_dtype(1.0), scale)
    q = np.clip(np.round(w / scale.astype(np.float32)[:, None, :]) + 8, 0, 15).astype(np.uint8).reshape(K, N)
    return (q[0::2] << 4) | q[1::2], scale
