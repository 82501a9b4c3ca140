"""cider_b200.ops - low-level operator API over torch CUDA tensors.

Same names, argument order and error behaviour as the reference's ``cider.ops``
(cider/ops.py), with ``mx.array`` -> ``torch.Tensor`` and ``mx.Stream`` ->
``torch.cuda.Stream``.  The reference returns lazy graph nodes; here the kernels
are enqueued on the given (or current) CUDA stream right away.  Everything runs
in hand-written sm_100a kernels behind the C ABI of include/cider_b200.h; torch
only provides device memory and streams.
"""
from __future__ import annotations

import functools
import inspect
from pathlib import Path
from typing import Optional

import numpy as np
import torch

from . import _lib

__all__ = [
    "is_available", "kernel_dir", "quantize_weight_int8", "pack_weight_int4",
    "perchannel_linear", "pergroup_linear", "w4a8_linear", "int8_matmul_int32",
    "quantize_per_token", "linear_prequantized", "rmsnorm_quant", "sdpa_decode",
    "quantize_weight_int8_pergroup", "pack_weight_int4_pergroup",
    "add_rmsnorm", "qk_norm_rope_append", "silu_mul", "linear_m1_fused",
    "interleave_gate_up", "swiglu_linear_prequantized", "quantize_consume_amax",
    "row_absmax", "quantize_given_amax", "sdpa_decode_fused",
]


# -- kernel directory (vestigial: the reference compiles Metal sources found
#    there at first use, cider/ops.py:19-24; the CUDA kernels are built ahead
#    of time, the directory now just holds their sources)
_KERNEL_DIR: Optional[str] = None


def kernel_dir() -> str:
    """Absolute path of the bundled kernel sources."""
    global _KERNEL_DIR
    if _KERNEL_DIR is None:
        _KERNEL_DIR = str(Path(__file__).parent / "csrc")
    return _KERNEL_DIR


# -- hardware gate (cider/ops.py:52-68: Apple M5+ and extension importable)
def is_available() -> bool:
    """True when a compute-capability-10.x GPU is present and the CUDA library loads."""
    try:
        if not torch.cuda.is_available():
            return False
        lib = _lib.load()
        return bool(lib.cider_device_supported(torch.cuda.current_device()))
    except Exception:
        return False


# -- offline weight quantisation (host side, numpy; cider/ops.py:73-116)
def quantize_weight_int8(w: np.ndarray) -> tuple:
    """Per-output-channel symmetric int8: ``w`` [N,K] -> (int8 [N,K], fp32 scale [N])."""
    w = np.asarray(w).astype(np.float32)
    scale = np.abs(w).max(axis=1) / 127.0
    scale = np.where(scale == 0, 1.0, scale)
    q = np.clip(np.round(w / scale[:, None]), -128, 127).astype(np.int8)
    return q, scale.astype(np.float32)


def quantize_weight_int8_pergroup(w: np.ndarray, group_size: int) -> tuple:
    """Per-group symmetric int8 (cider/nn.py:34-59): [N,K] -> (int8 [N,K], fp32 [N, K/gs])."""
    w = np.asarray(w).astype(np.float32)
    n, k = w.shape
    assert k % group_size == 0, f"K={k} not divisible by group_size={group_size}"
    blocks = w.reshape(n, k // group_size, group_size)
    scale = np.abs(blocks).max(axis=2) / 127.0
    scale = np.where(scale == 0, 1.0, scale)
    q = np.clip(np.round(blocks / scale[:, :, None]), -128, 127).astype(np.int8).reshape(n, k)
    return q, scale.astype(np.float32)


def pack_weight_int4(w: np.ndarray, zero_point: int = 8) -> tuple:
    """Per-column symmetric int4, two values per byte: ``w`` [K,N] ->
    (uint8 [K/2,N] with the even k in the high nibble, fp32 scale [N])."""
    k, _ = w.shape
    assert k % 2 == 0, f"K must be even, got {k}"
    w = np.asarray(w).astype(np.float32)
    scale = np.abs(w).max(axis=0) / 7.0
    scale = np.where(scale == 0, 1.0, scale)
    q = np.clip(np.round(w / scale[None, :]) + zero_point, 0, 15).astype(np.uint8)
    return (q[0::2] << 4) | q[1::2], scale.astype(np.float32)


def pack_weight_int4_pergroup(w: np.ndarray, group_size: int = 64, scale_dtype=np.float16) -> tuple:
    """Group-wise int4 (not in the reference, whose W4A8 scales are per column):
    ``w`` [K,N] -> (uint8 [K/2,N], scales [K/gs,N] in ``scale_dtype``).  The scale is
    rounded to its storage type before the weights are divided by it."""
    k, n = w.shape
    assert k % group_size == 0 and k % 2 == 0
    blocks = np.asarray(w).astype(np.float32).reshape(k // group_size, group_size, n)
    scale = (np.abs(blocks).max(axis=1) / 7.0).astype(scale_dtype)
    scale = np.where(scale == 0, scale_dtype(1.0), scale)
    q = np.clip(np.round(blocks / scale.astype(np.float32)[:, None, :]) + 8, 0, 15)
    q = q.astype(np.uint8).reshape(k, n)
    return (q[0::2] << 4) | q[1::2], scale


# -- helpers ----------------------------------------------------------------
def _stream_scoped(fn):
    """Run an op whose ``stream`` argument names a stream other than the current one
    entirely on that stream: outputs, workspace and dtype / layout temporaries come from
    torch's caching allocator, which ties a block to the stream that is current when it is
    allocated, so allocating on the current stream and launching on another would let the
    allocator hand the workspace to the next allocation while the kernels still use it.
    ``stream`` first waits for the work already queued on the current stream (the inputs
    may have been produced there).  The returned tensors belong to ``stream``: order later
    work after it (``wait_stream``) before using them elsewhere."""
    sig = inspect.signature(fn)

    @functools.wraps(fn)
    def wrapper(*args, **kwargs):
        bound = sig.bind(*args, **kwargs)
        stream = bound.arguments.get("stream")
        if stream is None:
            return fn(*args, **kwargs)
        cur = torch.cuda.current_stream(stream.device)
        if stream == cur:
            return fn(*args, **kwargs)
        stream.wait_stream(cur)
        bound.arguments["stream"] = None
        with torch.cuda.stream(stream):
            return fn(*bound.args, **bound.kwargs)

    return wrapper


def _stream_ptr(x: torch.Tensor, stream) -> int:
    if stream is None:
        stream = torch.cuda.current_stream(x.device)
    return int(stream.cuda_stream)


def _need_cuda(name: str, *tensors) -> None:
    dev = None
    for t in tensors:
        if t is None:
            continue
        if not isinstance(t, torch.Tensor) or not t.is_cuda:
            raise RuntimeError(
                f"cider_b200.{name}: expected CUDA tensors; there is no CPU implementation")
        if dev is None:
            dev = t.device
        elif t.device != dev:
            raise ValueError(f"cider_b200.{name}: tensors are on different devices")


def _as(t: torch.Tensor, dtype) -> torch.Tensor:
    if t.dtype != dtype:
        t = t.to(dtype)
    return t.contiguous()


def _ptr(t: Optional[torch.Tensor]):
    return None if t is None else t.data_ptr()


def _workspace(x: torch.Tensor, nbytes: int) -> Optional[torch.Tensor]:
    if nbytes == 0:
        return None
    return torch.empty(nbytes, dtype=torch.uint8, device=x.device)


def _scale_tag(t: torch.Tensor) -> int:
    return _lib.F16 if t.dtype == torch.float16 else _lib.F32


# -- primitive API ------------------------------------------------------------
@_stream_scoped
def perchannel_linear(x, w, scale_w, bias=None, stream=None):
    """W8A8 per-channel linear, ``y = dequant(quant_a(x) @ w_int8^T) + bias``
    (cider/ops.py:121-148).  x [M,K] fp16/bf16, w [N,K] int8, scale_w [N] fp32,
    bias [N] or None.  Returns [M,N] in x's dtype.  M == 1 takes the
    matrix-vector path that does not quantise x."""
    _need_cuda("perchannel_linear", x, w, scale_w, bias)
    if x.dim() != 2 or w.dim() != 2:
        raise ValueError("perchannel_linear: x and w must be 2-D")
    out_dtype = x.dtype
    xh, wq, sw = _as(x, torch.float16), _as(w, torch.int8), _as(scale_w, torch.float32)
    b = None if bias is None else _as(bias, torch.float16)
    M, K = xh.shape
    N = wq.shape[0]
    if wq.shape[1] != K or sw.numel() != N or (b is not None and b.numel() != N):
        raise ValueError(f"perchannel_linear: shape mismatch x{tuple(x.shape)} w{tuple(w.shape)} "
                         f"scale_w{tuple(scale_w.shape)}")
    lib = _lib.load()
    y = torch.empty((M, N), dtype=torch.float16, device=x.device)
    with torch.cuda.device(x.device):
        nbytes = lib.cider_workspace_bytes(_lib.OP_PERCHANNEL, M, N, K)
        ws = _workspace(xh, nbytes)
        _lib.check(lib.cider_perchannel_linear(xh.data_ptr(), wq.data_ptr(), sw.data_ptr(), _ptr(b),
                                               y.data_ptr(), M, N, K, _ptr(ws), nbytes,
                                               _stream_ptr(x, stream)))
    return y if out_dtype == torch.float16 else y.to(out_dtype)


def perchannel_linear_host(x_host, w, scale_w, bias=None, out=None, chunk_rows=0, stream=None):
    """``perchannel_linear`` for a HOST activation tensor (fp16, contiguous; pinned
    memory for full speed) and a host result: the rows are uploaded, multiplied and
    downloaded in overlapping chunks (``cider_perchannel_linear_host``).  w, scale_w,
    bias are CUDA tensors.  ``out`` is an optional [M,N] fp16 CPU tensor (pinned for
    full speed); the call returns it after the device has finished writing it."""
    if x_host.is_cuda or x_host.dtype != torch.float16 or x_host.dim() != 2 or not x_host.is_contiguous():
        raise ValueError("perchannel_linear_host: x_host must be a contiguous 2-D fp16 CPU tensor")
    _need_cuda("perchannel_linear_host", w, scale_w, bias)
    wq, sw = _as(w, torch.int8), _as(scale_w, torch.float32)
    b = None if bias is None else _as(bias, torch.float16)
    M, K = x_host.shape
    N = wq.shape[0]
    if wq.shape[1] != K or sw.numel() != N or (b is not None and b.numel() != N):
        raise ValueError(f"perchannel_linear_host: shape mismatch x{tuple(x_host.shape)} w{tuple(w.shape)}")
    if out is None:
        out = torch.empty((M, N), dtype=torch.float16, pin_memory=True)
    elif out.is_cuda or out.dtype != torch.float16 or tuple(out.shape) != (M, N) or not out.is_contiguous():
        raise ValueError("perchannel_linear_host: out must be a contiguous [M,N] fp16 CPU tensor")
    lib = _lib.load()
    with torch.cuda.device(w.device):
        st = torch.cuda.current_stream(w.device) if stream is None else stream
        _lib.check(lib.cider_perchannel_linear_host(x_host.data_ptr(), wq.data_ptr(), sw.data_ptr(), _ptr(b),
                                                    out.data_ptr(), M, N, K, int(chunk_rows), int(st.cuda_stream)))
        st.synchronize()
    return out


@_stream_scoped
def pergroup_linear(x, w, scale_w, group_size, bias=None, new_bias=None, stream=None):
    """W8A8 per-group linear (cider/ops.py:161-209).  scale_w is [K/group_size, N]
    (physically transposed), fp32 or fp16; group_size in {64,128,256}.
    ``new_bias`` is accepted and ignored, as in the reference's kernels."""
    _need_cuda("pergroup_linear", x, w, scale_w, bias)
    if x.dim() != 2 or w.dim() != 2:
        raise ValueError("pergroup_linear: x and w must be 2-D")
    out_dtype = x.dtype
    xh, wq = _as(x, torch.float16), _as(w, torch.int8)
    sw = scale_w.contiguous() if scale_w.dtype == torch.float16 else _as(scale_w, torch.float32)
    b = None if bias is None else _as(bias, torch.float16)
    M, K = xh.shape
    N = wq.shape[0]
    gs = int(group_size)
    if gs not in (64, 128, 256):
        raise ValueError(f"pergroup_linear: group_size must be 64, 128, or 256 (got {gs})")
    if wq.shape[1] != K or K % gs != 0 or tuple(sw.shape) != (K // gs, N):
        raise ValueError(f"pergroup_linear: shape mismatch x{tuple(x.shape)} w{tuple(w.shape)} "
                         f"scale_w{tuple(scale_w.shape)} group_size={gs}")
    lib = _lib.load()
    y = torch.empty((M, N), dtype=torch.float16, device=x.device)
    with torch.cuda.device(x.device):
        nbytes = lib.cider_workspace_bytes(_lib.OP_PERGROUP, M, N, K)
        ws = _workspace(xh, nbytes)
        _lib.check(lib.cider_pergroup_linear(xh.data_ptr(), wq.data_ptr(), sw.data_ptr(), _scale_tag(sw),
                                             _ptr(b), y.data_ptr(), M, N, K, gs, _ptr(ws), nbytes,
                                             _stream_ptr(x, stream)))
    return y if out_dtype == torch.float16 else y.to(out_dtype)


@_stream_scoped
def w4a8_linear(x, packed_w, scale_w, stream=None, group_size: int = 0):
    """W4A8 linear (cider/ops.py:212-235).  packed_w [K/2,N] uint8; scale_w [N]
    fp32 (reference) or, with ``group_size`` > 0, [K/group_size, N] fp16/fp32."""
    _need_cuda("w4a8_linear", x, packed_w, scale_w)
    if x.dim() != 2 or packed_w.dim() != 2:
        raise ValueError("w4a8_linear: x and packed_w must be 2-D")
    out_dtype = x.dtype
    xh, pw = _as(x, torch.float16), _as(packed_w, torch.uint8)
    gs = int(group_size)
    if gs == 0:
        sw = _as(scale_w, torch.float32)
    else:
        sw = scale_w.contiguous() if scale_w.dtype == torch.float16 else _as(scale_w, torch.float32)
    M, K = xh.shape
    N = pw.shape[1]
    if pw.shape[0] * 2 != K:
        raise ValueError(f"w4a8_linear: packed_w has {pw.shape[0]} rows, expected K/2 = {K // 2}")
    want = (N,) if gs == 0 else (K // max(gs, 1), N)
    if tuple(sw.shape) != want:
        raise ValueError(f"w4a8_linear: scale_w shape {tuple(sw.shape)}, expected {want}")
    lib = _lib.load()
    y = torch.empty((M, N), dtype=torch.float16, device=x.device)
    with torch.cuda.device(x.device):
        nbytes = lib.cider_workspace_bytes(_lib.OP_W4A8, M, N, K)
        ws = _workspace(xh, nbytes)
        _lib.check(lib.cider_w4a8_linear(xh.data_ptr(), pw.data_ptr(), sw.data_ptr(), _scale_tag(sw), gs,
                                         y.data_ptr(), M, N, K, _ptr(ws), nbytes, _stream_ptr(x, stream)))
    return y if out_dtype == torch.float16 else y.to(out_dtype)


@_stream_scoped
def w4a8_repack(packed_w, stream=None):
    """One-time repack of the reference's packed int4 weights [K/2, N] (N contiguous)
    into rows [N, K/2] (K contiguous, same nibble convention) for ``w4a8_linear_rows``."""
    _need_cuda("w4a8_repack", packed_w)
    pw = _as(packed_w, torch.uint8)
    kp, N = pw.shape
    out = torch.empty((N, kp), dtype=torch.uint8, device=pw.device)
    lib = _lib.load()
    with torch.cuda.device(pw.device):
        _lib.check(lib.cider_w4a8_repack(pw.data_ptr(), out.data_ptr(), N, 2 * kp, _stream_ptr(pw, stream)))
    return out


@_stream_scoped
def w4a8_linear_rows(x, w_rows, scale_w, stream=None, group_size: int = 0, int8_scratch: bool = False):
    """``w4a8_linear`` on weights repacked by ``w4a8_repack`` ([N, K/2] uint8): the
    same results with no weight scratch - the GEMM expands the nibbles in its
    shared-memory stage, a decode-sized call streams the packed rows.
    ``int8_scratch=True`` lends the call N*K more bytes of workspace: beyond decode sizes
    the weights are then expanded by a pass of their own and the int8 kernels run on the
    copy (memory for time; the same bits)."""
    _need_cuda("w4a8_linear_rows", x, w_rows, scale_w)
    if x.dim() != 2 or w_rows.dim() != 2:
        raise ValueError("w4a8_linear_rows: x and w_rows must be 2-D")
    out_dtype = x.dtype
    xh, pw = _as(x, torch.float16), _as(w_rows, torch.uint8)
    gs = int(group_size)
    if gs == 0:
        sw = _as(scale_w, torch.float32)
    else:
        sw = scale_w.contiguous() if scale_w.dtype == torch.float16 else _as(scale_w, torch.float32)
    M, K = xh.shape
    N = pw.shape[0]
    if pw.shape[1] * 2 != K:
        raise ValueError(f"w4a8_linear_rows: w_rows has {pw.shape[1]} bytes per row, expected K/2 = {K // 2}")
    want = (N,) if gs == 0 else (K // max(gs, 1), N)
    if tuple(sw.shape) != want:
        raise ValueError(f"w4a8_linear_rows: scale_w shape {tuple(sw.shape)}, expected {want}")
    lib = _lib.load()
    y = torch.empty((M, N), dtype=torch.float16, device=x.device)
    with torch.cuda.device(x.device):
        nbytes = lib.cider_workspace_bytes(_lib.OP_W4A8_ROWS_INT8COPY if int8_scratch else _lib.OP_W4A8_ROWS,
                                           M, N, K)
        ws = _workspace(xh, nbytes)
        _lib.check(lib.cider_w4a8_linear_nk4(xh.data_ptr(), pw.data_ptr(), sw.data_ptr(), _scale_tag(sw), gs,
                                             y.data_ptr(), M, N, K, _ptr(ws), nbytes, _stream_ptr(x, stream)))
    return y if out_dtype == torch.float16 else y.to(out_dtype)


@_stream_scoped
def int8_matmul_int32(a, b, stream=None):
    """Raw int8 x int8 -> int32 matmul, bit-exact (cider/ops.py:238-255).
    a [M,K] int8, b [N,K] int8 (weight layout) -> [M,N] int32."""
    _need_cuda("int8_matmul_int32", a, b)
    if a.dim() != 2 or b.dim() != 2:
        raise ValueError("int8_matmul_int32: a and b must be 2-D")
    aq, bq = _as(a, torch.int8), _as(b, torch.int8)
    M, K = aq.shape
    N = bq.shape[0]
    if bq.shape[1] != K:
        raise ValueError(f"int8_matmul_int32: K mismatch a{tuple(a.shape)} b{tuple(b.shape)}")
    lib = _lib.load()
    c = torch.empty((M, N), dtype=torch.int32, device=a.device)
    with torch.cuda.device(a.device):
        _lib.check(lib.cider_int8_matmul_int32(aq.data_ptr(), bq.data_ptr(), c.data_ptr(), M, N, K,
                                               _stream_ptr(a, stream)))
    return c


# -- pieces of the path exposed on their own (no counterpart in cider.ops; the
#    reference keeps them inside its primitives)
@_stream_scoped
def quantize_per_token(x, stream=None):
    """Per-token activation quantisation: x [M,K] fp16 -> (int8 [M,K], fp32 [M])."""
    _need_cuda("quantize_per_token", x)
    if x.dim() != 2:
        raise ValueError("quantize_per_token: x must be 2-D")
    xh = x if x.dtype == torch.float16 else x.to(torch.float16)
    if xh.stride(1) != 1 and xh.shape[1] > 1:
        xh = xh.contiguous()
    M, K = xh.shape
    ldx = xh.stride(0) if M > 1 else max(K, 1)
    if ldx < K:
        xh, ldx = xh.contiguous(), K
    q = torch.empty((M, K), dtype=torch.int8, device=x.device)
    s = torch.empty((M,), dtype=torch.float32, device=x.device)
    lib = _lib.load()
    with torch.cuda.device(x.device):
        _lib.check(lib.cider_quantize_per_token(xh.data_ptr(), M, K, ldx, q.data_ptr(), s.data_ptr(),
                                                _stream_ptr(x, stream)))
    return q, s


@_stream_scoped
def row_absmax(x, stream=None):
    """Row absmax of x [M,K] (fp16) -> fp32 [M]: the first half of the quantiser, for a
    tensor-parallel rank that holds a K-slice of the activation."""
    _need_cuda("row_absmax", x)
    xh = _as(x, torch.float16)
    M, K = xh.shape
    amax = torch.empty((M,), dtype=torch.float32, device=x.device)
    lib = _lib.load()
    with torch.cuda.device(x.device):
        _lib.check(lib.cider_row_absmax(xh.data_ptr(), M, K, K, amax.data_ptr(), _stream_ptr(x, stream)))
    return amax


@_stream_scoped
def quantize_given_amax(x, amax, stream=None):
    """Per-token quantiser with a given row absmax (fp32 [M], at least the row's own):
    (int8 [M,K], fp32 scale [M] = amax/127, 0 -> 1)."""
    _need_cuda("quantize_given_amax", x, amax)
    xh, am = _as(x, torch.float16), _as(amax, torch.float32)
    M, K = xh.shape
    if am.numel() != M:
        raise ValueError("quantize_given_amax: amax must have one value per row")
    q = torch.empty((M, K), dtype=torch.int8, device=x.device)
    s = torch.empty((M,), dtype=torch.float32, device=x.device)
    lib = _lib.load()
    with torch.cuda.device(x.device):
        _lib.check(lib.cider_quantize_given_amax(xh.data_ptr(), M, K, K, am.data_ptr(), q.data_ptr(), s.data_ptr(),
                                                 _stream_ptr(x, stream)))
    return q, s


@_stream_scoped
def linear_prequantized(a_int8, scale_a, w, scale_w, group_size: int = 0, bias=None, stream=None):
    """GEMM + dequant epilogue on already-quantised activations."""
    _need_cuda("linear_prequantized", a_int8, scale_a, w, scale_w, bias)
    aq, sa, wq = _as(a_int8, torch.int8), _as(scale_a, torch.float32), _as(w, torch.int8)
    gs = int(group_size)
    if gs == 0:
        sw = _as(scale_w, torch.float32)
    else:
        sw = scale_w.contiguous() if scale_w.dtype == torch.float16 else _as(scale_w, torch.float32)
    b = None if bias is None else _as(bias, torch.float16)
    M, K = aq.shape
    N = wq.shape[0]
    if wq.shape[1] != K or sa.numel() != M:
        raise ValueError("linear_prequantized: shape mismatch")
    y = torch.empty((M, N), dtype=torch.float16, device=aq.device)
    lib = _lib.load()
    with torch.cuda.device(aq.device):
        _lib.check(lib.cider_linear_prequantized(aq.data_ptr(), sa.data_ptr(), wq.data_ptr(), sw.data_ptr(),
                                                 _scale_tag(sw), gs, _ptr(b), y.data_ptr(), M, N, K,
                                                 _stream_ptr(aq, stream)))
    return y


@_stream_scoped
def rmsnorm_quant(x, weight, eps: float, want_fp16: bool = True, stream=None):
    """RMSNorm fused with the per-token quantiser.  Returns (y fp16 or None, q int8, scale)."""
    _need_cuda("rmsnorm_quant", x, weight)
    xh, wh = _as(x, torch.float16), _as(weight, torch.float16)
    M, K = xh.shape
    y = torch.empty_like(xh) if want_fp16 else None
    q = torch.empty((M, K), dtype=torch.int8, device=x.device)
    s = torch.empty((M,), dtype=torch.float32, device=x.device)
    lib = _lib.load()
    with torch.cuda.device(x.device):
        _lib.check(lib.cider_rmsnorm_quant(xh.data_ptr(), wh.data_ptr(), float(eps), M, K, _ptr(y),
                                           q.data_ptr(), s.data_ptr(), _stream_ptr(x, stream)))
    return y, q, s


@_stream_scoped
def sdpa_decode(q, k_cache, v_cache, length: int, scale: float, stream=None, length_dev=None, out=None,
                workspace=None, tickets=None):
    """Single-query attention over an fp16 KV cache.  q [B,Hq,D]; caches
    [B,Hkv,Tcap,D]; attends to the first ``length`` positions, or to the first
    ``length_dev[0]`` (int32 device tensor <= length) when given.  Returns [B,Hq,D].
    ``tickets``: an int32 device tensor of B*Hkv zeros lent by the caller turns the two
    launches (partial + combine) into one; it is zero again when the call is done."""
    _need_cuda("sdpa_decode", q, k_cache, v_cache)
    qh, kc, vc = _as(q, torch.float16), k_cache, v_cache
    if kc.dtype != torch.float16 or vc.dtype != torch.float16 or not kc.is_contiguous() or not vc.is_contiguous():
        raise ValueError("sdpa_decode: caches must be contiguous fp16 [B,Hkv,Tcap,D]")
    B, Hq, D = qh.shape
    _, Hkv, Tcap, _ = kc.shape
    if out is None:
        out = torch.empty_like(qh)
    lib = _lib.load()
    with torch.cuda.device(q.device):
        nbytes = lib.cider_sdpa_decode_workspace_bytes(B, Hq, Hkv, D, int(length))
        ws = workspace if workspace is not None else torch.empty(max(nbytes, 16), dtype=torch.uint8,
                                                                 device=q.device)
        if ws.numel() < nbytes:
            raise ValueError("sdpa_decode: workspace too small")
        if tickets is not None:
            if tickets.dtype != torch.int32 or tickets.numel() < B * Hkv or not tickets.is_cuda:
                raise ValueError("sdpa_decode: tickets must be an int32 CUDA tensor of at least B*Hkv zeros")
            _lib.check(lib.cider_sdpa_decode_tickets(qh.data_ptr(), kc.data_ptr(), vc.data_ptr(), out.data_ptr(),
                                                     B, Hq, Hkv, D, int(length), Tcap, float(scale),
                                                     ws.data_ptr(), ws.numel(), _ptr(length_dev),
                                                     tickets.data_ptr(), _stream_ptr(q, stream)))
        else:
            _lib.check(lib.cider_sdpa_decode(qh.data_ptr(), kc.data_ptr(), vc.data_ptr(), out.data_ptr(), B, Hq,
                                             Hkv, D, int(length), Tcap, float(scale), ws.data_ptr(), ws.numel(),
                                             _ptr(length_dev), _stream_ptr(q, stream)))
    return out


@_stream_scoped
def sdpa_decode_fused(qkv, q_norm_w, k_norm_w, inv_freq, axis, pos3, eps, k_cache, v_cache, length: int, scale: float,
                      nq: int, nkv: int, length_dev=None, tickets=None, stream=None):
    """One decode step's attention with its prologue folded in: qkv [B, (nq + 2 nkv) * 128] is the
    raw projection output of ONE new token per sequence; per-head q / k RMSNorm, rope (position
    ids pos3[:, 0]), append of the new key / value at cache position ``length - 1`` (or
    ``length_dev[0] - 1``) and single-query attention over the first ``length`` positions, in one
    launch (two without ``tickets``).  The bits of ``qk_norm_rope_append`` + ``sdpa_decode``."""
    _need_cuda("sdpa_decode_fused", qkv, k_cache, v_cache)
    B = qkv.shape[0]
    D = k_cache.shape[-1]
    Tcap = k_cache.shape[-2]
    out = torch.empty((B, nq, D), dtype=torch.float16, device=qkv.device)
    lib = _lib.load()
    with torch.cuda.device(qkv.device):
        nbytes = lib.cider_sdpa_decode_workspace_bytes(B, nq, nkv, D, int(length))
        ws = torch.empty(max(nbytes, 16), dtype=torch.uint8, device=qkv.device)
        _lib.check(lib.cider_sdpa_decode_fused(qkv.data_ptr(), q_norm_w.data_ptr(), k_norm_w.data_ptr(),
                                               inv_freq.data_ptr(), axis.data_ptr(), pos3.data_ptr(), pos3.stride(0),
                                               float(eps), k_cache.data_ptr(), v_cache.data_ptr(), out.data_ptr(),
                                               B, nq, nkv, D, int(length), Tcap, float(scale), ws.data_ptr(),
                                               ws.numel(), _ptr(length_dev), _ptr(tickets), _stream_ptr(qkv, stream)))
    return out


@_stream_scoped
def add_rmsnorm(x, delta, weight, eps: float, want_fp16: bool = True, want_int8: bool = False, stream=None):
    """x <- x + delta in place (delta may be None), then RMSNorm of the sum.  Returns
    (y fp16 or None, q int8 or None, scale or None)."""
    _need_cuda("add_rmsnorm", x, delta, weight)
    if x.dtype != torch.float16 or not x.is_contiguous() or x.dim() != 2:
        raise ValueError("add_rmsnorm: x must be a contiguous 2-D fp16 tensor (updated in place)")
    M, K = x.shape
    d = None if delta is None else _as(delta, torch.float16)
    wh = _as(weight, torch.float16)
    y = torch.empty_like(x) if want_fp16 else None
    q = torch.empty((M, K), dtype=torch.int8, device=x.device) if want_int8 else None
    s = torch.empty((M,), dtype=torch.float32, device=x.device) if want_int8 else None
    lib = _lib.load()
    with torch.cuda.device(x.device):
        _lib.check(lib.cider_add_rmsnorm_quant(x.data_ptr(), _ptr(d), wh.data_ptr(), float(eps), M, K, _ptr(y),
                                               _ptr(q), _ptr(s), _stream_ptr(x, stream)))
    return y, q, s


@_stream_scoped
def qk_norm_rope_append(qkv, q_norm_w, k_norm_w, inv_freq, axis, pos3, base, eps, q_out, k_cache, v_cache,
                        B: int, T: int, nq: int, nkv: int, base_dev=None, stream=None):
    """Per-head q/k RMSNorm + rope + KV append (see cider_qk_norm_rope_append).
    pos3: int32 device tensor [3, T]; base: first cache position (host int), or
    base_dev: int32 device tensor holding it."""
    _need_cuda("qk_norm_rope_append", qkv, pos3, q_out, k_cache, v_cache)
    D = k_cache.shape[-1]
    Tcap = k_cache.shape[-2]
    lib = _lib.load()
    with torch.cuda.device(qkv.device):
        _lib.check(lib.cider_qk_norm_rope_append(qkv.data_ptr(), q_norm_w.data_ptr(), k_norm_w.data_ptr(),
                                                 inv_freq.data_ptr(), axis.data_ptr(), pos3.data_ptr(),
                                                 pos3.stride(0), _ptr(base_dev), int(base), float(eps),
                                                 q_out.data_ptr(), k_cache.data_ptr(), v_cache.data_ptr(),
                                                 B, T, nq, nkv, D, Tcap, _stream_ptr(qkv, stream)))
    return q_out


@_stream_scoped
def silu_mul(gate_up, stream=None):
    """SwiGLU on a fused [M, 2*inter] gate/up tensor -> [M, inter]."""
    _need_cuda("silu_mul", gate_up)
    gu = _as(gate_up, torch.float16)
    M, two = gu.shape
    act = torch.empty((M, two // 2), dtype=torch.float16, device=gu.device)
    lib = _lib.load()
    with torch.cuda.device(gu.device):
        _lib.check(lib.cider_silu_mul(gu.data_ptr(), act.data_ptr(), M, two // 2, _stream_ptr(gu, stream)))
    return act


@_stream_scoped
def quantize_heads(a, stream=None):
    """Per-token quantiser of an attention output ``a`` [B, heads, T, D] (contiguous):
    returns (q [B*T, heads*D] int8, scale [B*T] fp32), row (b, t) being the
    concatenation of its heads - the same as quantising
    ``a.transpose(1, 2).reshape(B*T, heads*D)`` without making that copy."""
    _need_cuda("quantize_heads", a)
    if a.dim() != 4:
        raise ValueError("quantize_heads: a must be [B, heads, T, D]")
    ah = _as(a, torch.float16)
    B, Hh, T, D = ah.shape
    q = torch.empty((B * T, Hh * D), dtype=torch.int8, device=ah.device)
    s = torch.empty((B * T,), dtype=torch.float32, device=ah.device)
    lib = _lib.load()
    with torch.cuda.device(ah.device):
        _lib.check(lib.cider_quantize_heads(ah.data_ptr(), B, Hh, T, D, q.data_ptr(), s.data_ptr(),
                                            _stream_ptr(ah, stream)))
    return q, s


@_stream_scoped
def silu_mul_quant(gate_up, stream=None):
    """SwiGLU on a fused [M, 2*inter] gate/up tensor followed by the per-token
    quantiser, in one pass: returns (q [M, inter] int8, scale [M] fp32) of
    ``silu_mul(gate_up)`` without materialising it."""
    _need_cuda("silu_mul_quant", gate_up)
    gu = _as(gate_up, torch.float16)
    M, two = gu.shape
    q = torch.empty((M, two // 2), dtype=torch.int8, device=gu.device)
    s = torch.empty((M,), dtype=torch.float32, device=gu.device)
    lib = _lib.load()
    with torch.cuda.device(gu.device):
        _lib.check(lib.cider_silu_mul_quant(gu.data_ptr(), M, two // 2, q.data_ptr(), s.data_ptr(),
                                            _stream_ptr(gu, stream)))
    return q, s


def interleave_gate_up(w, scale_w=None, bias=None, block: int = 32):
    """Rows of a fused [gate ; up] projection ([2*inter, K], gate rows first) reordered into blocks
    of ``block`` gate rows followed by their ``block`` up rows - the layout
    ``swiglu_linear_prequantized`` takes.  The per-row scales and the bias follow.  Works on
    numpy arrays and torch tensors alike (indexing only)."""
    n = w.shape[0]
    inter = n // 2
    if n % 2 or inter % block:
        raise ValueError(f"interleave_gate_up: {n} rows are not two halves of whole blocks of {block}")
    r = np.arange(n)
    b, wi = r // (2 * block), r % (2 * block)
    idx = np.where(wi < block, b * block + wi, inter + b * block + wi - block)
    if isinstance(w, torch.Tensor):
        tidx = torch.from_numpy(idx).to(w.device)
        take = lambda t: None if t is None else t.index_select(0, tidx.to(t.device)).contiguous()
    else:
        take = lambda t: None if t is None else np.ascontiguousarray(t[idx])
    return take(w), take(scale_w), take(bias)


@_stream_scoped
def swiglu_linear_prequantized(a_int8, scale_a, w_interleaved, scale_w_interleaved, bias_interleaved=None,
                               rowmax=None, stream=None):
    """The fused gate/up projection with the SwiGLU in the GEMM's epilogue: returns
    (act [M, N/2] fp16, rowmax [M] fp32) with act = half(half(silu(g)) * u) of the fp16 linear
    outputs and rowmax[m] = max |act[m, :]|.  Weights, scales and bias in the
    ``interleave_gate_up`` layout.  ``rowmax`` (zeroed, reused between calls) may be passed in;
    ``quantize_consume_amax`` turns the pair into the next linear's int8 input and zeroes it again."""
    _need_cuda("swiglu_linear_prequantized", a_int8, scale_a, w_interleaved, scale_w_interleaved, bias_interleaved)
    a, sa = _as(a_int8, torch.int8), _as(scale_a, torch.float32)
    w, sw = _as(w_interleaved, torch.int8), _as(scale_w_interleaved, torch.float32)
    b = None if bias_interleaved is None else _as(bias_interleaved, torch.float16)
    M, K = a.shape
    N = w.shape[0]
    if w.shape[1] != K or sw.numel() != N or sa.numel() != M:
        raise ValueError("swiglu_linear_prequantized: shape mismatch")
    act = torch.empty((M, N // 2), dtype=torch.float16, device=a.device)
    if rowmax is None:
        rowmax = torch.zeros((M,), dtype=torch.float32, device=a.device)
    lib = _lib.load()
    with torch.cuda.device(a.device):
        _lib.check(lib.cider_swiglu_linear_prequantized(a.data_ptr(), sa.data_ptr(), w.data_ptr(), sw.data_ptr(),
                                                        _ptr(b), act.data_ptr(), rowmax.data_ptr(), M, N, K,
                                                        _stream_ptr(a, stream)))
    return act, rowmax


@_stream_scoped
def quantize_consume_amax(x, amax, stream=None):
    """``quantize_given_amax`` that writes 0 back to ``amax`` once it has been read."""
    _need_cuda("quantize_consume_amax", x, amax)
    xh = _as(x, torch.float16)
    M, K = xh.shape
    q = torch.empty((M, K), dtype=torch.int8, device=xh.device)
    s = torch.empty((M,), dtype=torch.float32, device=xh.device)
    lib = _lib.load()
    with torch.cuda.device(xh.device):
        _lib.check(lib.cider_quantize_consume_amax(xh.data_ptr(), M, K, K, amax.data_ptr(), q.data_ptr(), s.data_ptr(),
                                                   _stream_ptr(xh, stream)))
    return q, s


@_stream_scoped
def linear_m1_fused(x, w, scale_w, group_size: int = 0, bias=None, prologue: str = "plain", delta=None,
                    norm_weight=None, eps: float = 0.0, x_out=None, stream=None):
    """M == 1 linear with a fused activation prologue (see cider_linear_m1_fused).
    prologue: "plain" (x [K]), "silu_mul" (x = [gate | up], length 2K) or
    "add_norm" (x [K] residual, optional ``delta``, RMSNorm weight ``norm_weight``,
    updated residual written to ``x_out``).  Returns y [1, N] fp16."""
    _need_cuda("linear_m1_fused", x, w, scale_w, bias, delta, norm_weight, x_out)
    mode = {"plain": 0, "silu_mul": 1, "add_norm": 2}[prologue]
    wq = _as(w, torch.int8)
    gs = int(group_size)
    sw = _as(scale_w, torch.float32) if (gs == 0 or scale_w.dtype != torch.float16) else scale_w.contiguous()
    N, K = wq.shape
    xh = _as(x, torch.float16).reshape(-1)
    if xh.numel() != (2 * K if mode == 1 else K):
        raise ValueError("linear_m1_fused: activation length does not match the weight")
    y = torch.empty((1, N), dtype=torch.float16, device=x.device)
    lib = _lib.load()
    with torch.cuda.device(x.device):
        _lib.check(lib.cider_linear_m1_fused(xh.data_ptr(), mode, _ptr(delta), _ptr(norm_weight), float(eps),
                                             _ptr(x_out), wq.data_ptr(), sw.data_ptr(), _scale_tag(sw), gs,
                                             _ptr(bias), y.data_ptr(), N, K, _stream_ptr(x, stream)))
    return y
