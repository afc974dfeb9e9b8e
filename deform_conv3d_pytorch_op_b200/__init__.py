"""B200 (sm_100a) deformable convolution: drop-in for the operator API of lshiwjx/deform_conv3d_pytorch_op.

Modules ``ConvOffset3d`` / ``ConvOffset2d`` / ``Conv2d`` / ``Conv3d`` (aliases ``DeformConv3d`` / ``DeformConv2d``) over the
autograd Functions ``ConvOffset3dFunction`` / ``ConvOffset2dFunction`` / ``Conv2dFunction``; the reference's
FFI call surface is in :mod:`legacy_ops`; all arithmetic runs in ``csrc/libdcn.so`` (C ABI: ``include/dcn.h``).
"""
from ._lib import DcnError, LIB_PATH
from .functions import (Conv2dFunction, Conv3dFunction, ConvOffset2dFunction, ConvOffset3dFunction,
                        DeformLayerFunction, LegacyConvOffset2dFunction)
from .modules import (Conv2d, Conv3d, ConvOffset2d, ConvOffset3d, DeformConv2d, DeformConv3d, DeformLayer2d,
                      DeformLayer3d, LegacyConvOffset2d)
from .legacy_ops import conv2d_op, deform_conv2d_double_op, deform_conv2d_op, deform_conv3d_op
from .ops import Op, check_status

__all__ = [
    "DcnError", "LIB_PATH", "Op", "check_status",
    "ConvOffset3dFunction", "ConvOffset2dFunction", "Conv2dFunction", "Conv3dFunction", "DeformLayerFunction", "LegacyConvOffset2dFunction",
    "ConvOffset3d", "ConvOffset2d", "Conv2d", "Conv3d", "DeformConv3d", "DeformConv2d", "DeformLayer3d", "DeformLayer2d", "LegacyConvOffset2d",
    "deform_conv3d_op", "deform_conv2d_op", "deform_conv2d_double_op", "conv2d_op",
]
