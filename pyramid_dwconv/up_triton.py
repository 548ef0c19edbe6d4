"""Import path of the reference's bilinear-resize module."""
from pyramidconvblock_b200.modules import OptimizedBilinearInterp2d  # noqa: F401
from pyramidconvblock_b200.ops import BilinearInterp2dFunction  # noqa: F401
