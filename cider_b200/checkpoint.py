"""cider_b200.checkpoint - ingestion of already-quantised checkpoints.

The reference reaches its INT8 modules from a "compressed-tensors" pack-quantised
checkpoint (``<layer>.weight_packed`` int32 words, ``<layer>.weight_scale``,
``<layer>.weight_shape``) by way of other formats: its tool rewrites the words
into MLX's affine layout (tools/convert_compressed_tensors_to_mlx.py:105-146)
and ``CiderLinear.from_float`` then dequantises and re-quantises
(cider/nn.py:127-171); the smooth-quant converter dequantises to bf16 first
(vlm_service/convert_qwen3vl_smooth_to_mlx.py:63-72,177-205).  The stored values
are already symmetric integers with per-channel or per-group scales, i.e. exactly
the operands of the W8A8 / W4A8 kernels, so this module builds ``CiderLinear`` /
``W4A8Linear`` from them directly: no fp16 detour, no second rounding.

Layout of the source format (as written by compressed-tensors, little end first):
    weight_packed  int32 [N, ceil(K * bits / 32)]; element k of a row sits in word
                   k // (32 / bits) at bit (k % (32 / bits)) * bits.  Every width is
                   offset binary: stored field = weight + 2^(bits-1), i.e. + 128 for
                   8 bits and + 8 for 4 bits (offset = 1 << (num_bits - 1),
                   tools/convert_compressed_tensors_to_mlx.py:51,140,236-238).
    weight_scale   [N, 1] (per-channel) or [N, K / group_size]
    weight_shape   [2] = (N, K)
A raw variant stores ``<layer>.weight`` as int8 [N, K] next to ``weight_scale``.
Everything here runs on the host with torch ops; nothing touches the GPU until the
modules are moved there.
"""
from __future__ import annotations

from typing import Dict, Optional, Tuple

import torch
from torch import nn

from .nn import CiderLinear, W4A8Linear

_SUFFIXES = ((".weight_packed", "packed"), (".weight_scale", "scale"), (".weight_shape", "shape"),
             (".weight_zero_point", "zero_point"))
_GROUPS = (64, 128, 256)


def unpack_int8_words(packed: torch.Tensor, in_features: int) -> torch.Tensor:
    """int32 [N, W] -> int8 [N, K]: the four bytes of a word are four consecutive k, each
    stored offset binary (byte = weight + 128), so weight = byte - 128 = byte ^ 0x80 read as
    two's complement."""
    if packed.dtype != torch.int32 or packed.dim() != 2:
        raise ValueError("weight_packed must be a 2-D int32 tensor")
    if packed.shape[1] * 4 < in_features:
        raise ValueError(f"weight_packed holds {packed.shape[1] * 4} values per row, need {in_features}")
    b = packed.contiguous().view(torch.uint8).reshape(packed.shape[0], -1)[:, :in_features]
    return (b ^ 0x80).contiguous().view(torch.int8)


def unpack_int4_words(packed: torch.Tensor, in_features: int) -> torch.Tensor:
    """int32 [N, W] -> uint8 [N, K] nibble values 0..15 (stored value = weight + 8)."""
    if packed.dtype != torch.int32 or packed.dim() != 2:
        raise ValueError("weight_packed must be a 2-D int32 tensor")
    if packed.shape[1] * 8 < in_features:
        raise ValueError(f"weight_packed holds {packed.shape[1] * 8} values per row, need {in_features}")
    b = packed.contiguous().view(torch.uint8).reshape(packed.shape[0], -1)  # byte j = k 2j (low), 2j+1 (high)
    nib = torch.stack((b & 0x0F, b >> 4), dim=2).reshape(packed.shape[0], -1)
    return nib[:, :in_features].contiguous()


def _scale_layout(scale: torch.Tensor, N: int, K: int) -> Tuple[torch.Tensor, int]:
    """[N], [N,1] or [N, K/gs] -> (scale in the kernels' layout, group_size)."""
    s = scale.detach()
    if s.dim() == 1:
        s = s[:, None]
    if s.dim() != 2 or s.shape[0] != N:
        raise ValueError(f"weight_scale has shape {tuple(scale.shape)}, expected [{N}, groups]")
    ng = s.shape[1]
    if ng == 1:
        return s[:, 0].to(torch.float32).contiguous(), 0
    if K % ng != 0 or (K // ng) not in _GROUPS:
        raise ValueError(f"unsupported group size {K / ng:g} (K={K}, {ng} scale columns); supported: {_GROUPS}")
    # [N, ng] -> [ng, N], N contiguous: the layout of the per-group kernels; fp16 scales stay fp16
    st = s.t().contiguous()
    return (st if st.dtype == torch.float16 else st.to(torch.float32)), K // ng


def linear_from_compressed(packed: Optional[torch.Tensor], scale: torch.Tensor, shape=None, *, num_bits: int = 8,
                           bias: Optional[torch.Tensor] = None, weight_int8: Optional[torch.Tensor] = None,
                           zero_point: Optional[torch.Tensor] = None) -> nn.Module:
    """One layer of a pack-quantised (or raw int8) checkpoint -> ``CiderLinear`` (8 bit)
    or ``W4A8Linear`` (4 bit) holding exactly the stored integers and scales."""
    if zero_point is not None and bool((zero_point != 0).any()):
        raise ValueError("asymmetric quantisation (non-zero weight_zero_point) is not representable: the "
                         "kernels are symmetric")
    if weight_int8 is not None:
        if weight_int8.dtype != torch.int8 or weight_int8.dim() != 2:
            raise ValueError("raw weight must be int8 [N, K]")
        N, K = weight_int8.shape
        num_bits = 8
    else:
        if packed is None:
            raise ValueError("need weight_packed or a raw int8 weight")
        N = packed.shape[0]
        K = int(shape[1]) if shape is not None else packed.shape[1] * (32 // num_bits)
        if shape is not None and int(shape[0]) != N:
            raise ValueError(f"weight_shape says {int(shape[0])} rows, weight_packed has {N}")
    sw, gs = _scale_layout(scale, N, K)
    if num_bits == 8:
        w = weight_int8.contiguous() if weight_int8 is not None else unpack_int8_words(packed, K)
        return CiderLinear(w, sw, gs, K, N, bias)
    if num_bits == 4:
        if K % 2:
            raise ValueError("4-bit layers need an even K")
        if bias is not None:
            raise ValueError("W4A8Linear has no bias (w4a8_primitive.mm:266-283 takes none)")
        nib = unpack_int4_words(packed, K)  # [N, K], value + 8
        # the reference's packing: [K/2, N] bytes, high nibble = even k (cider/ops.py:96-116)
        rows = (nib[:, 0::2] << 4) | nib[:, 1::2]  # [N, K/2]
        return W4A8Linear(rows.t().contiguous(), sw, K, gs)
    raise ValueError(f"num_bits={num_bits} is not supported (8 or 4)")


def classify_state_dict(state: Dict[str, torch.Tensor]):
    """Split a checkpoint's tensors into quantised layers {base: {part: tensor}} and
    the rest.  A layer is quantised when it has ``weight_packed`` or an int8 ``weight``
    together with ``weight_scale``."""
    layers: Dict[str, Dict[str, torch.Tensor]] = {}
    plain: Dict[str, torch.Tensor] = {}
    for key, t in state.items():
        for suffix, part in _SUFFIXES:
            if key.endswith(suffix):
                layers.setdefault(key[: -len(suffix)], {})[part] = t
                break
        else:
            plain[key] = t
    for base in list(layers):
        parts = layers[base]
        wkey = base + ".weight"
        if "packed" not in parts and wkey in plain and plain[wkey].dtype == torch.int8 and "scale" in parts:
            parts["raw"] = plain.pop(wkey)
        if "scale" not in parts or ("packed" not in parts and "raw" not in parts):
            # not a quantised layer after all: hand the tensors back untouched
            for suffix, part in _SUFFIXES:
                if part in parts:
                    plain[base + suffix] = parts[part]
            del layers[base]
    return layers, plain


def modules_from_state_dict(state: Dict[str, torch.Tensor], num_bits: int = 8):
    """-> ({layer name: CiderLinear | W4A8Linear}, {other key: tensor}).  A layer's
    ``<name>.bias`` is folded into its module."""
    layers, plain = classify_state_dict(state)
    mods: Dict[str, nn.Module] = {}
    for base, parts in sorted(layers.items()):
        bias = plain.pop(base + ".bias", None)
        shape = parts.get("shape")
        mods[base] = linear_from_compressed(parts.get("packed"), parts["scale"],
                                            None if shape is None else shape.tolist(), num_bits=num_bits,
                                            bias=bias, weight_int8=parts.get("raw"),
                                            zero_point=parts.get("zero_point"))
    return mods, plain


def load_compressed_checkpoint(model: nn.Module, state: Dict[str, torch.Tensor], num_bits: int = 8,
                               strict: bool = False) -> dict:
    """Swap the quantised layers of ``state`` into ``model`` (by dotted module name, in
    place) and load the remaining tensors with ``load_state_dict``.  Returns
    ``{"n_quantized", "missing_keys", "unexpected_keys"}``."""
    mods, plain = modules_from_state_dict(state, num_bits)
    for name, mod in mods.items():
        parent_name, _, child = name.rpartition(".")
        parent = model.get_submodule(parent_name) if parent_name else model
        old = getattr(parent, child, None)
        if old is None:
            raise KeyError(f"checkpoint layer {name!r} has no module in the model")
        dev = next((p.device for p in old.parameters()), None) or next((b.device for b in old.buffers()), None)
        setattr(parent, child, mod.to(dev) if dev is not None else mod)
    own = {k for k, _ in model.named_parameters()} | {k for k, _ in model.named_buffers()}
    quantised_prefixes = tuple(n + "." for n in mods)
    res = model.load_state_dict({k: v for k, v in plain.items() if k in own and not k.startswith(quantised_prefixes)},
                                strict=False)
    missing = [k for k in res.missing_keys if not k.startswith(quantised_prefixes)]
    unexpected = [k for k in plain if k not in own]
    if strict and (missing or unexpected):
        raise RuntimeError(f"missing keys {missing}, unexpected keys {unexpected}")
    return {"n_quantized": len(mods), "missing_keys": missing, "unexpected_keys": unexpected}
