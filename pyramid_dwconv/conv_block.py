"""Import path of the reference's conv_block module."""
from pyramidconvblock_b200.modules import ConvBlock, SimpleGate  # noqa: F401
