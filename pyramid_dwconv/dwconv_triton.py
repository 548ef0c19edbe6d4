"""Import path of the reference's depthwise-conv module (the name is historical: no Triton here)."""
from pyramidconvblock_b200.modules import OptimizedDepthwiseConv2d  # noqa: F401
from pyramidconvblock_b200.ops import DepthwiseConv2DFunction  # noqa: F401
