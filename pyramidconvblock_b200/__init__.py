"""B200-native (sm_100a) implementation of the PyramidConvBlock hot path.

Public names follow the reference package ``pyramid_dwconv``; ``import pyramid_dwconv`` (the
compatibility package at the repository root) re-exports them.
"""
from .modules import (ConvBlock, OptimizedAdaptiveAvgPool2d, OptimizedBilinearInterp2d, OptimizedDepthwiseConv2d,
                      SimpleGate)
from .nchw import (ConvBlockNCHW, nchw_as_nhwc, nchw_state_dict_from_nhwc, nhwc_as_nchw,
                   nhwc_state_dict_from_nchw)
from .ops import (AdaptiveAvgPool2dFunction, BilinearInterp2dFunction, DepthwiseConv2DFunction, GateFunction,
                  check_device_status)

__all__ = [
    "ConvBlock", "SimpleGate", "OptimizedDepthwiseConv2d", "OptimizedAdaptiveAvgPool2d",
    "OptimizedBilinearInterp2d", "DepthwiseConv2DFunction", "AdaptiveAvgPool2dFunction",
    "BilinearInterp2dFunction", "GateFunction", "check_device_status",
    "ConvBlockNCHW", "nchw_as_nhwc", "nhwc_as_nchw", "nhwc_state_dict_from_nchw", "nchw_state_dict_from_nhwc",
]
