"""Import path of the reference's adaptive-average-pool module."""
from pyramidconvblock_b200.modules import OptimizedAdaptiveAvgPool2d  # noqa: F401
from pyramidconvblock_b200.ops import AdaptiveAvgPool2dFunction  # noqa: F401
