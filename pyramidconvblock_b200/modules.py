"""nn.Module surface of the reference package, on top of the CUDA kernels.

Constructor signatures, attribute names, parameter shapes/dtypes and the ORDER in which parameters
are created match the reference, so a fixed torch seed yields the same initial weights and a
reference ``state_dict`` loads unchanged (pyramid_dwconv/conv_block.py:6-49,
pyramid_dwconv/dwconv_triton.py:389-426).
"""
import torch
from torch import nn

from .block_function import ConvBlockFunction
from .ops import (AdaptiveAvgPool2dFunction, BilinearInterp2dFunction, DepthwiseConv2DFunction, GateFunction, _pair)


class OptimizedDepthwiseConv2d(nn.Module):
    """Depthwise conv over NHWC input with a [KH,KW,C] weight.

    As in the reference (dwconv_triton.py:410-416) the weight is created in float16 whatever
    ``dtype`` says and initialised with ``kaiming_uniform_``; cast the module afterwards.  ``bias``
    is an extension (the reference has none) and defaults to off, which keeps the parameter set
    identical.
    """

    def __init__(self, channels, kernel_size, stride=1, padding=0, dilation=1, dtype=None, bias=False):
        super().__init__()
        self.channels = channels
        self.kernel_size = _pair(kernel_size)
        self.stride = _pair(stride)
        self.padding = _pair(padding)
        self.dilation = _pair(dilation)
        self.weight = nn.Parameter(torch.empty(self.kernel_size[0], self.kernel_size[1], channels,
                                               dtype=torch.float16))
        nn.init.kaiming_uniform_(self.weight)
        if bias:
            self.bias = nn.Parameter(torch.zeros(channels, dtype=torch.float16))
        else:
            self.register_parameter("bias", None)

    def forward(self, x):
        assert x.dim() == 4 and x.shape[3] == self.channels, "input must be [B,H,W,C] with C == channels"
        return DepthwiseConv2DFunction.apply(x, self.weight, self.stride, self.padding, self.dilation,
                                             self.weight.dtype, self.bias)

    def extra_repr(self):
        return "channels=%d, kernel_size=%s, stride=%s, padding=%s, dilation=%s, bias=%s" % (
            self.channels, self.kernel_size, self.stride, self.padding, self.dilation, self.bias is not None)


class OptimizedAdaptiveAvgPool2d(nn.Module):
    """NHWC adaptive average pool (pyramid_dwconv/avgpool_triton.py:259-268)."""

    def __init__(self, output_size):
        super().__init__()
        self.output_size = _pair(output_size)

    def forward(self, x):
        assert x.dim() == 4, "input must be a 4-D [B,H,W,C] tensor"
        return AdaptiveAvgPool2dFunction.apply(x, self.output_size)


class OptimizedBilinearInterp2d(nn.Module):
    """NHWC bilinear resize (pyramid_dwconv/up_triton.py:127-162).  Like the reference kernel it
    always uses align_corners=False coordinates; asking for True is refused instead of ignored."""

    def __init__(self, output_size, align_corners=False):
        super().__init__()
        if align_corners:
            raise NotImplementedError("only align_corners=False is implemented (the reference ignores the flag)")
        self.output_size = _pair(output_size)
        self.align_corners = align_corners

    def forward(self, x):
        assert x.dim() == 4, "input must be a 4-D [B,H,W,C] tensor"
        return BilinearInterp2dFunction.apply(x, self.output_size)


class SimpleGate(nn.Module):
    """[pool ->] depthwise conv -> x1*(x2/scale) [-> upsample back] (conv_block.py:6-22)."""

    def __init__(self, dim, kernel_size=13, scale_factor=1., bias=False):
        super().__init__()
        self.scale_factor = scale_factor
        self.scale = (dim / 2) ** -0.5
        self.conv_spatial = OptimizedDepthwiseConv2d(dim, kernel_size=kernel_size, padding=kernel_size // 2)

    def forward(self, x):
        B, H, W, C = x.shape
        resized = self.scale_factor != 1.
        if resized:
            x = AdaptiveAvgPool2dFunction.apply(x, (int(H * self.scale_factor), int(W * self.scale_factor)))
        x = self.conv_spatial(x)
        x = GateFunction.apply(x, 1.0 / self.scale)
        if resized:
            x = BilinearInterp2dFunction.apply(x, (H, W))
        return x


class ConvBlock(nn.Module):
    """Linear up-projection, gated large-kernel depthwise branches at several scales, Linear
    out-projection plus a globally pooled Linear branch (conv_block.py:25-49).  [B,H,W,dim] in and out."""

    def __init__(self, dim, bias=False, out_bias=True, kernel_size=9, scales=(1., 1 / 2), inter_ratio=0.5):
        super().__init__()
        inter_dim = int(dim * inter_ratio)
        self.conv_up = nn.Linear(dim, inter_dim, bias=bias)
        self.gates = nn.ModuleList(
            [SimpleGate(inter_dim, kernel_size=kernel_size, scale_factor=s, bias=bias) for s in scales])
        self.conv_out = nn.Linear(inter_dim // 2 * len(scales), dim, bias=out_bias)
        self.conv_pool = nn.Linear(dim, dim, bias=out_bias)

    def forward(self, x):
        dw = [g.conv_spatial for g in self.gates]
        params = [self.conv_up.weight, self.conv_out.weight, self.conv_pool.weight] + [c.weight for c in dw]
        fusable = (x.dim() == 4 and all(p.dtype == x.dtype for p in params)
                   and all(c.bias is None and c.kernel_size[0] == c.kernel_size[1] for c in dw))
        if not fusable:
            return self.forward_unfused(x)
        return ConvBlockFunction.apply(
            x, tuple(g.scale_factor for g in self.gates), self.conv_up.weight, self.conv_up.bias,
            self.conv_out.weight, self.conv_out.bias, self.conv_pool.weight, self.conv_pool.bias,
            *[c.weight for c in dw])

    def forward_unfused(self, x):
        """The same block composed op by op, exactly as the reference writes it."""
        branches_in = self.conv_up(x)
        branches = torch.cat([gate(branches_in) for gate in self.gates], dim=-1)
        pooled = self.conv_pool(x.mean(dim=(1, 2), keepdim=True))
        return self.conv_out(branches) + pooled
