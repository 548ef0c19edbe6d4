"""Compatibility package: ``from pyramid_dwconv import ConvBlock`` keeps working unchanged.

Everything is implemented in ``pyramidconvblock_b200`` (hand-written sm_100a CUDA behind a C ABI);
this package only provides the reference's import paths.
"""
from pyramidconvblock_b200 import (AdaptiveAvgPool2dFunction, BilinearInterp2dFunction, ConvBlock,
                                   DepthwiseConv2DFunction, OptimizedAdaptiveAvgPool2d,
                                   OptimizedBilinearInterp2d, OptimizedDepthwiseConv2d, SimpleGate)

__all__ = ["ConvBlock", "OptimizedDepthwiseConv2d", "DepthwiseConv2DFunction"]
