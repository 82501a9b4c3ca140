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


def convert_model(model: nn.Module, *, verbose: bool = True, target_group_size: int = None,
                  skip=()) -> dict:
    """Convert all Linear / QuantizedLinear layers to CiderLinear, in place.

    ``target_group_size`` (None = per-channel for float layers) and ``skip`` (child
    names to leave alone, e.g. ``("lm_head",)``) are additions; with their
    defaults the behaviour is the reference's.
    """
    if not ops.is_available():
        raise RuntimeError(
            "W8A8 INT8 tensor-core kernels not available. Requires an sm_100 (B200) GPU and the "
            "built cider_b200 CUDA library.")
    t0 = time.perf_counter()
    counter = [0]
    _convert_children(model, counter, target_group_size, tuple(skip))
    elapsed = time.perf_counter() - t0
    stats = {"n_converted": counter[0], "elapsed_s": elapsed}
    if verbose:
        print(f"[cider] Converted {counter[0]} layers to CiderLinear in {elapsed:.1f}s")
    return stats
