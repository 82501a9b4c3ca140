"""cider_b200 - INT8 tensor-core quantised linear layers for NVIDIA B200 (sm_100a).

Drop-in for the public surface of the reference's ``cider`` package
(cider/__init__.py:42-57), over torch CUDA tensors:

    import cider_b200 as cider
    cider.convert_model(model)        # every nn.Linear -> CiderLinear, in place

When no B200 / CUDA library is available ``is_available()`` is False,
``convert_model`` becomes a warning no-op and the primitives are not exported -
the same degraded surface as the reference off Apple M5 (cider/__init__.py:58-75).
"""

__version__ = "0.1.0"

from .ops import is_available

if is_available():
    from .convert import convert_model
    from .nn import CiderLinear, W4A8Linear, W8A8Linear, QuantizedLinear, get_mode, set_mode
    from .ops import (
        int8_matmul_int32,
        kernel_dir,
        pack_weight_int4,
        perchannel_linear,
        pergroup_linear,
        quantize_weight_int8,
        w4a8_linear,
    )

    __all__ = [
        "convert_model", "set_mode", "get_mode", "CiderLinear", "W8A8Linear", "W4A8Linear",
        "QuantizedLinear", "perchannel_linear", "w4a8_linear", "pergroup_linear",
        "int8_matmul_int32", "quantize_weight_int8", "pack_weight_int4", "is_available",
        "kernel_dir",
    ]
else:
    def convert_model(*args, **kwargs):
        """No-op on unsupported hardware."""
        import warnings
        warnings.warn(
            "cider_b200.convert_model() is a no-op: the INT8 kernels need an sm_100 (B200) GPU. "
            "Model will use standard torch inference.", RuntimeWarning, stacklevel=2)

    def set_mode(*args, **kwargs):
        pass

    def get_mode():
        return "unavailable"

    __all__ = ["convert_model", "set_mode", "get_mode", "is_available"]
