"""feather_ops for B200: the quantized matmul family of woct0rdho/feather-ops on sm_100a.

Same Python surface as the reference package (`feather_ops/__init__.py:18-31` there): `scaled_mm_hip`,
the int8 ConvRot functions and the 3x3 conv, all running hand-written tcgen05 kernels through
`torch.ops.feather_ops.*`. Importing the package loads the native extension and fails loudly when it has
not been built: there is no CPU or eager fallback for the kernels.
"""

import sys

import torch  # noqa: F401  the extension links against libtorch, so torch has to be loaded first

# `python -m feather_ops_b200._build` imports this package before it runs the build script: that one entry has to get
# through without the extension, everything else fails loudly.
_BUILDING = "feather_ops_b200._build" in getattr(sys, "orig_argv", [])

try:
    from . import _C  # noqa: F401  registers torch.ops.feather_ops.{scaled_mm,int8_scaled_mm,convrot_quantize,conv2d_3x3}
except ImportError as exc:  # pragma: no cover - depends on the build state
    if not _BUILDING:
        raise ImportError(
            "feather_ops_b200._C is not built (or failed to load): run `python -m feather_ops_b200._build` "
            "(needs nvcc and g++, no GPU). The kernels have no fallback path."
        ) from exc

if not _BUILDING or "feather_ops_b200._C" in sys.modules:
    from .conv2d import conv3x3_prepacked, prepack_conv2d_weight_3x3
    from .conv2d_module import Conv2d
    from .int8_convrot import (
        convrot_int8_dgrad,
        convrot_int8_linear,
        dequantize_convrot_weight,
        int8_scaled_mm,
        int8_scaled_mm_plain,
        prepack_int8_weight,
        quantize_convrot_activation,
        quantize_convrot_weight,
        unpack_int8_weight,
    )
    from .scaled_mm import prepack_b_for_scaled_mm, scaled_mm_hip

    __all__ = [
        "Conv2d",
        "conv3x3_prepacked",
        "convrot_int8_dgrad",
        "convrot_int8_linear",
        "dequantize_convrot_weight",
        "int8_scaled_mm",
        "int8_scaled_mm_plain",
        "prepack_b_for_scaled_mm",
        "prepack_conv2d_weight_3x3",
        "prepack_int8_weight",
        "quantize_convrot_activation",
        "quantize_convrot_weight",
        "scaled_mm_hip",
        "unpack_int8_weight",
    ]
