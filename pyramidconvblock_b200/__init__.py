"""B200-native (sm_100a) implementation of the PyramidConvBlock hot path.

Public names follow the reference package ``pyramid_dwconv``; ``import pyramid_dwconv`` (the
compatibility package at the repository root) re-exports them.
"""
from .modules import (ConvBlock, OptimizedAdaptiveAvgPool2d, OptimizedBilinearInterp2d, OptimizedDepthwiseConv2d,
                      SimpleGate)
from .ops import (AdaptiveAvgPool2dFunction, BilinearInterp2dFunction, DepthwiseConv2DFunction, GateFunction,
                  check_device_status)

__all__ = [
    "ConvBlock", "SimpleGate", "OptimizedDepthwiseConv2d", "OptimizedAdaptiveAvgPool2d",
    "OptimizedBilinearInterp2d", "DepthwiseConv2DFunction", "AdaptiveAvgPool2dFunction",
    "BilinearInterp2dFunction", "GateFunction", "check_device_status",
]
