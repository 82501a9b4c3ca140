"""cider_b200.convert - one-call model conversion (mirror of cider/convert.py).

``convert_model(model)`` walks the module tree and replaces every
``torch.nn.Linear`` (and ``cider_b200.nn.QuantizedLinear``) by a ``CiderLinear``
in place, returning ``{"n_converted", "elapsed_s"}`` like the reference
(cider/convert.py:50-99).  Containers (ModuleList / Sequential / ModuleDict) are
modules in torch, so the reference's separate list walk (cider/convert.py:35-44)
is covered by the same recursion.
"""
from __future__ import annotations

import gc
import time

from torch import nn

from . import ops
from .nn import CiderLinear, QuantizedLinear

_TARGET_TYPES = (nn.Linear, QuantizedLinear)


def _convert_children(module: nn.Module, counter, target_group_size=None, skip=()):
    for name, child in list(module.named_children()):
        if isinstance(child, _TARGET_TYPES):
            if name in skip:
                continue
            setattr(module, name, CiderLinear.from_float(child, target_group_size))
            counter[0] += 1
            if counter[0] % 28 == 0:
                gc.collect()
        elif isinstance(child, nn.Module):
            _convert_children(child, counter, target_group_size, skip)


# Sibling projections that read the same input and can run as one GEMM.
FUSE_SETS = (("q_proj", "k_proj", "v_proj"), ("gate_proj", "up_proj"))


class FusedProjections(nn.Module):
    """Several ``CiderLinear`` layers over the same input as ONE layer whose output
    channels are their concatenation.  Quantisation is per output channel (and per
    group of K), so the fused layer computes, column for column, exactly what the
    separate layers computed; it is one launch and one pass over the activation
    instead of two or three (the reference explored this for prefill,
    cider/fused_hybrid.py:217-296, by swapping the attention / MLP classes; here the
    children keep their names and calling conventions)."""

    def __init__(self, layers):
        super().__init__()
        first = layers[0]
        gs = first.group_size
        if any(l.group_size != gs or l.input_dims != first.input_dims for l in layers):
            raise ValueError("fused projections need the same input size and group size")
        if gs and any(l.scale_w.dtype != first.scale_w.dtype for l in layers):
            raise ValueError("fused projections need the same scale dtype")
        from .nn import CiderLinear as _CL
        import torch
        self.splits = [l.output_dims for l in layers]
        self.linear = _CL(torch.cat([l.w_int8 for l in layers], dim=0),
                          torch.cat([l.scale_w for l in layers], dim=0 if gs == 0 else 1), gs,
                          first.input_dims, sum(self.splits), torch.cat([l.bias for l in layers], dim=0))
        self._x, self._key, self._parts, self._left = None, None, None, 0

    def reset(self):
        """Forget the cached projection (and let go of the activation it belongs to)."""
        self._x, self._key, self._parts, self._left = None, None, None, 0

    def project(self, x, index: int):
        """Output of child ``index`` for input ``x``; the fused GEMM runs once per
        distinct input, the other children of the group pick up their slices.

        The cache is keyed on the input's address, version counter, shape, strides and
        dtype, and it HOLDS the input tensor for as long as it is valid: while that
        reference lives the allocator cannot hand the address to another activation, so
        an equal key means the same bytes.  The cache is dropped when every child has
        been served, and ``fuse_projections`` also drops it before and after every
        forward of the parent module, which bounds its life to one forward even in a
        model that calls only some of the children."""
        key = (x.data_ptr(), x._version, tuple(x.shape), tuple(x.stride()), x.dtype, x.device)
        if self._parts is None or self._key != key:
            self._parts = self.linear(x).split(self.splits, dim=-1)
            self._x, self._key, self._left = x, key, len(self.splits)
        out = self._parts[index]
        self._left -= 1
        if self._left <= 0:  # every child has been served: do not keep the activation alive
            self.reset()
        return out


class FusedSlice(nn.Module):
    """Stands where one of the fused layers stood; ``forward(x)`` returns that layer's
    output.  Holds the group without registering it (the parent owns it)."""

    def __init__(self, group: FusedProjections, index: int):
        super().__init__()
        object.__setattr__(self, "_group", group)
        self.index = index

    def forward(self, x):
        return self._group.project(x, self.index)

    @property
    def output_dims(self) -> int:
        return self._group.splits[self.index]


def fuse_projections(model: nn.Module, sets=FUSE_SETS) -> int:
    """Fuse, in place, every group of sibling ``CiderLinear`` children named as in
    ``sets`` (q/k/v and gate/up by default).  Returns the number of groups fused."""
    n = 0
    for parent in list(model.modules()):
        for names in sets:
            kids = [getattr(parent, nm, None) for nm in names]
            if not all(isinstance(k, CiderLinear) for k in kids):
                continue
            try:
                group = FusedProjections(kids)
            except ValueError:
                continue
            setattr(parent, "fused_" + "_".join(nm.split("_")[0] for nm in names), group)
            # one forward of the parent is the cache's scope
            parent.register_forward_pre_hook(lambda _m, _args, g=group: g.reset())
            parent.register_forward_hook(lambda _m, _args, _out, g=group: g.reset())
            for i, nm in enumerate(names):
                setattr(parent, nm, FusedSlice(group, i))
            n += 1
    return n


def convert_model(model: nn.Module, *, verbose: bool = True, target_group_size: int = None,
                  skip=(), fuse: bool = False) -> dict:
    """Convert all Linear / QuantizedLinear layers to CiderLinear, in place.

    ``target_group_size`` (None = per-channel for float layers), ``skip`` (child
    names to leave alone, e.g. ``("lm_head",)``) and ``fuse`` (run q/k/v and gate/up
    siblings as one GEMM each, see ``fuse_projections``) are additions; with their
    defaults the behaviour is the reference's.
    """
    if not ops.is_available():
        raise RuntimeError(
            "W8A8 INT8 tensor-core kernels not available. Requires an sm_100 (B200) GPU and the "
            "built cider_b200 CUDA library.")
    t0 = time.perf_counter()
    counter = [0]
    _convert_children(model, counter, target_group_size, tuple(skip))
    n_fused = fuse_projections(model) if fuse else 0
    elapsed = time.perf_counter() - t0
    stats = {"n_converted": counter[0], "elapsed_s": elapsed}
    if fuse:
        stats["n_fused_groups"] = n_fused
    if verbose:
        print(f"[cider] Converted {counter[0]} layers to CiderLinear in {elapsed:.1f}s")
    return stats
