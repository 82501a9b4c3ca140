"""cider_b200.nn - INT8 / packed-INT4 linear modules (torch.nn.Module).

Mirror of the reference's ``cider.nn`` (cider/nn.py): ``CiderLinear`` (alias
``W8A8Linear``) keeps one int8 copy of the weight plus its scales and dispatches
to ``ops.perchannel_linear`` (group_size 0) or ``ops.pergroup_linear``
(group_size 64/128/256); both pick the GEMM (M > 1) or the matrix-vector kernel
(M == 1) by themselves.  ``W4A8Linear`` holds packed int4 weights.
"""
from __future__ import annotations

import numpy as np
import torch
from torch import nn

from . import ops


# -- backward-compatible no-ops (cider/nn.py:24-30)
def set_mode(mode: str):
    """No-op, kept for backward compatibility."""
    return None


def get_mode() -> str:
    """Always 'auto'."""
    return "auto"


def _symmetric_quantize_pergroup(w_fp: np.ndarray, group_size: int):
    """[N,K] float -> (int8 [N,K], fp32 scales [N, K/group_size]); cider/nn.py:34-59."""
    return ops.quantize_weight_int8_pergroup(w_fp, group_size)


class CiderLinear(nn.Module):
    """Unified INT8 linear (cider/nn.py:63-113).

    Args:
        w_int8: [N,K] int8.
        scale_w: per-channel [N] fp32, or per-group [K/group_size, N] fp32/fp16
            (already physically transposed).
        group_size: 0 = per-channel, 64/128/256 = per-group.
        bias: [N] fp16 or None (zeros).
    """

    def __init__(self, w_int8, scale_w, group_size: int, in_features: int, out_features: int, bias=None):
        super().__init__()
        if group_size == 0:
            self._mode = "per_channel"
        elif group_size in (64, 128, 256):
            self._mode = "per_group"
        else:
            raise ValueError(f"Unsupported group_size={group_size}. Use 0 (per-channel) or 64/128/256.")
        w_int8 = torch.as_tensor(w_int8)
        scale_w = torch.as_tensor(scale_w)
        self.register_buffer("w_int8", w_int8.to(torch.int8).contiguous())
        if scale_w.dtype != torch.float16 or group_size == 0:
            scale_w = scale_w.to(torch.float32)
        self.register_buffer("scale_w", scale_w.contiguous())
        self.group_size = int(group_size)
        self._in_features = int(in_features)
        self._out_features = int(out_features)
        if bias is None:
            bias = torch.zeros(out_features, dtype=torch.float16, device=self.w_int8.device)
        self.register_buffer("bias", torch.as_tensor(bias).to(torch.float16).contiguous())

    def forward(self, x: torch.Tensor) -> torch.Tensor:
        orig_shape = x.shape
        x_2d = x.reshape(-1, self._in_features)
        if self._mode == "per_channel":
            y = ops.perchannel_linear(x_2d, self.w_int8, self.scale_w, self.bias)
        else:
            y = ops.pergroup_linear(x_2d, self.w_int8, self.scale_w, self.group_size, self.bias)
        return y.reshape(*orig_shape[:-1], self._out_features)

    @staticmethod
    def from_float(layer: nn.Module, target_group_size: int = None, scale_dtype=torch.float32) -> "CiderLinear":
        """Build from a float ``nn.Linear`` (per-channel unless ``target_group_size``),
        or from a ``QuantizedLinear`` (dequantise, then symmetric re-quantise:
        per-group when it was 8-bit with group size 64/128/256, else per-channel),
        following cider/nn.py:115-194.  Quantisation runs on the host in numpy."""
        if isinstance(layer, QuantizedLinear):
            bits, gs = layer.bits, layer.group_size
            if target_group_size is not None:
                tgs = target_group_size
            elif bits == 8 and gs in (64, 128, 256):
                tgs = gs
            else:
                tgs = 0
            w_np = layer.dequantize().to(torch.float32).cpu().numpy()
            out_f, in_f = w_np.shape
            lin_bias = layer.bias
            device = layer.scales.device
        elif hasattr(layer, "weight"):
            out_f, in_f = layer.weight.shape
            lin_bias = getattr(layer, "bias", None)
            tgs = target_group_size or 0
            w_np = layer.weight.detach().to(torch.float32).cpu().numpy()
            device = layer.weight.device
        else:
            raise TypeError(f"Unsupported layer: {type(layer)}")
        if tgs == 0:
            w_q, scale = ops.quantize_weight_int8(w_np)
            scale_t = torch.from_numpy(scale)
        else:
            w_q, scale = _symmetric_quantize_pergroup(w_np, tgs)
            scale_t = torch.from_numpy(np.ascontiguousarray(scale.T)).to(scale_dtype)  # [N,ng] -> [ng,N]
        bias = None if lin_bias is None else lin_bias.detach().to(torch.float16).to(device)
        return CiderLinear(torch.from_numpy(w_q).to(device), scale_t.to(device), tgs, in_f, out_f, bias)

    @property
    def input_dims(self) -> int:
        return self._in_features

    @property
    def output_dims(self) -> int:
        return self._out_features

    def extra_repr(self) -> str:
        return f"in={self._in_features}, out={self._out_features}, mode={self._mode}, gs={self.group_size}"


W8A8Linear = CiderLinear  # backward-compatible alias (cider/nn.py:213)


class W4A8Linear(nn.Module):
    """Packed INT4 weight x INT8 activation linear (cider/nn.py:217-241)."""

    def __init__(self, packed_weight, scale, K: int, group_size: int = 0):
        super().__init__()
        self.register_buffer("packed_weight", torch.as_tensor(packed_weight).to(torch.uint8).contiguous())
        scale = torch.as_tensor(scale)
        if group_size == 0 or scale.dtype != torch.float16:
            scale = scale.to(torch.float32)
        self.register_buffer("scale", scale.contiguous())
        self._K = int(K)
        self.group_size = int(group_size)

    def forward(self, x: torch.Tensor) -> torch.Tensor:
        orig_shape = x.shape
        x2 = x.reshape(-1, self._K)
        if self._K % 16 == 0:
            # weights are static: keep a row-major copy ([N, K/2], K contiguous) made on
            # first use, so that decode-sized calls stream the packed bytes
            pw = self.packed_weight
            key = (pw.data_ptr(), pw._version, pw.device)  # rebuilt if the buffer is replaced or written
            if self._rows is None or self._rows_key != key:
                self._rows, self._rows_key = ops.w4a8_repack(pw), key
            rows = self._rows
            y = ops.w4a8_linear_rows(x2, rows, self.scale, group_size=self.group_size)
        else:
            y = ops.w4a8_linear(x2, self.packed_weight, self.scale, group_size=self.group_size)
        return y.reshape(*orig_shape[:-1], self.output_dims)

    _rows = None  # lazily built [N, K/2] copy of packed_weight (not part of the state dict)
    _rows_key = None

    @staticmethod
    def from_weights(w: np.ndarray, zero_point: int = 8, group_size: int = 0, device=None) -> "W4A8Linear":
        """From an fp16/fp32 numpy weight [K,N]; per-column scales unless ``group_size`` > 0."""
        K = w.shape[0]
        if group_size:
            packed, scale = ops.pack_weight_int4_pergroup(w, group_size)
        else:
            packed, scale = ops.pack_weight_int4(w, zero_point)
        dev = device if device is not None else ("cuda" if torch.cuda.is_available() else "cpu")
        return W4A8Linear(torch.from_numpy(packed).to(dev), torch.from_numpy(scale).to(dev), K, group_size)

    @property
    def input_dims(self) -> int:
        return self._K

    @property
    def output_dims(self) -> int:
        return self.packed_weight.shape[1]


class QuantizedLinear(nn.Module):
    """Container for an affine group-quantised weight in the layout of MLX's
    ``nn.QuantizedLinear`` (the second input type of the reference's
    ``CiderLinear.from_float``, cider/nn.py:127-171):
    ``w[n,k] = q[n,k] * scales[n, k // group_size] + biases[n, k // group_size]``
    with ``q`` unsigned ``bits``-bit values packed little-end first into uint32
    words along K.  It only stores and dequantises; it has no forward of its own."""

    def __init__(self, weight, scales, biases, group_size: int, bits: int, bias=None):
        super().__init__()
        self.register_buffer("weight", torch.as_tensor(weight))
        self.register_buffer("scales", torch.as_tensor(scales))
        self.register_buffer("biases", torch.as_tensor(biases))
        self.bias = bias
        self.group_size = int(group_size)
        self.bits = int(bits)

    @staticmethod
    def quantize(w: torch.Tensor, group_size: int = 64, bits: int = 8, bias=None) -> "QuantizedLinear":
        """Affine min/max group quantisation of a float [N,K] weight."""
        N, K = w.shape
        assert K % group_size == 0 and 32 % bits == 0
        wf = w.detach().to(torch.float32).reshape(N, K // group_size, group_size)
        lo, hi = wf.amin(dim=2), wf.amax(dim=2)
        levels = (1 << bits) - 1
        scales = (hi - lo) / levels
        scales = torch.where(scales == 0, torch.ones_like(scales), scales)
        q = torch.clamp(torch.round((wf - lo[:, :, None]) / scales[:, :, None]), 0, levels).to(torch.int64)
        per_word = 32 // bits
        q = q.reshape(N, K // per_word, per_word)
        shifts = torch.arange(per_word, dtype=torch.int64, device=w.device) * bits
        packed = (q << shifts).sum(dim=2).to(torch.int64)
        packed = torch.where(packed >= 2 ** 31, packed - 2 ** 32, packed).to(torch.int32)
        return QuantizedLinear(packed, scales, lo, group_size, bits, bias)

    def dequantize(self) -> torch.Tensor:
        per_word = 32 // self.bits
        words = self.weight.to(torch.int64) & 0xFFFFFFFF
        shifts = torch.arange(per_word, dtype=torch.int64, device=words.device) * self.bits
        q = (words[:, :, None] >> shifts) & ((1 << self.bits) - 1)
        N = q.shape[0]
        q = q.reshape(N, -1, self.group_size).to(torch.float32)
        w = q * self.scales.to(torch.float32)[:, :, None] + self.biases.to(torch.float32)[:, :, None]
        return w.reshape(N, -1)
