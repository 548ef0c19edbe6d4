"""Helpers for code written against the NCHW form of the block.

The reference ships a second, plain-torch definition of the same block for NCHW tensors
(``ConvBlockT`` / ``SimpleGateT``, pyramid_dwconv/conv_block.py:50-97): 1x1 ``nn.Conv2d`` where the
NHWC block has ``nn.Linear``, a grouped ``nn.Conv2d`` where it has the depthwise module.  Models
built on that form keep logical NCHW shapes.  This module lets them use the CUDA path without a
layout copy:

* an NCHW tensor stored in ``torch.channels_last`` memory format IS an NHWC-contiguous buffer;
  ``nchw_as_nhwc`` returns that view (and only copies when the tensor is stored otherwise);
* ``ConvBlockNCHW`` is ``ConvBlock`` taking and returning logical-NCHW tensors (the result is a
  channels_last view of the NHWC output, again no copy);
* ``nhwc_state_dict_from_nchw`` / ``nchw_state_dict_from_nhwc`` convert the parameters of one form
  into those of the other (1x1 conv weight [O,I,1,1] <-> Linear weight [O,I]; depthwise weight
  [C,1,KH,KW] <-> [KH,KW,C]), so a checkpoint of an NCHW model loads into the NHWC block and back.
"""
from .modules import ConvBlock


def nchw_as_nhwc(x):
    """Logical [B,C,H,W] -> contiguous [B,H,W,C].  Free for channels_last storage, one copy otherwise."""
    if x.dim() != 4:
        raise ValueError("expected a 4-D [B,C,H,W] tensor, got %d dimensions" % x.dim())
    return x.permute(0, 2, 3, 1).contiguous()     # contiguous() is a no-op on a channels_last tensor


def nhwc_as_nchw(y):
    """Contiguous [B,H,W,C] -> logical [B,C,H,W] view in channels_last memory format (never copies)."""
    if y.dim() != 4:
        raise ValueError("expected a 4-D [B,H,W,C] tensor, got %d dimensions" % y.dim())
    return y.permute(0, 3, 1, 2)


def shares_memory_with_nhwc_view(x):
    """True when ``nchw_as_nhwc(x)`` is a view of ``x`` (no copy will be made)."""
    return x.dim() == 4 and x.permute(0, 2, 3, 1).is_contiguous()


class ConvBlockNCHW(ConvBlock):
    """``ConvBlock`` for logical-NCHW tensors: [B,dim,H,W] in, [B,dim,H,W] (channels_last) out.

    Parameters, their order, shapes and ``state_dict`` keys are those of ``ConvBlock``; use
    ``nhwc_state_dict_from_nchw`` to load parameters saved from the NCHW torch form of the block."""

    def forward(self, x):
        return nhwc_as_nchw(super().forward(nchw_as_nhwc(x)))


_POINTWISE = ("conv_up", "conv_out", "conv_pool")


def _is_depthwise_key(key):
    return key.startswith("gates.") and key.endswith(".conv_spatial.weight")


def nhwc_state_dict_from_nchw(state_dict):
    """Parameters of the NCHW form (1x1 / grouped ``nn.Conv2d`` weights) as a ``ConvBlock`` state_dict.
    Keys are the same in both forms; only weight shapes differ.  Tensors keep their dtype."""
    out = {}
    for key, v in state_dict.items():
        if _is_depthwise_key(key):
            if v.dim() != 4 or v.shape[1] != 1:
                raise ValueError("%s: expected a depthwise weight [C,1,KH,KW], got %s" % (key, tuple(v.shape)))
            out[key] = v[:, 0].permute(1, 2, 0).contiguous()                  # [C,KH,KW] -> [KH,KW,C]
        elif key.endswith(".weight") and key.split(".")[0] in _POINTWISE:
            if v.dim() != 4 or v.shape[2:] != (1, 1):
                raise ValueError("%s: expected a 1x1 conv weight [O,I,1,1], got %s" % (key, tuple(v.shape)))
            out[key] = v[:, :, 0, 0].contiguous()
        else:
            out[key] = v
    return out


def nchw_state_dict_from_nhwc(state_dict):
    """Inverse of ``nhwc_state_dict_from_nchw``."""
    out = {}
    for key, v in state_dict.items():
        if _is_depthwise_key(key):
            if v.dim() != 3:
                raise ValueError("%s: expected a depthwise weight [KH,KW,C], got %s" % (key, tuple(v.shape)))
            out[key] = v.permute(2, 0, 1).unsqueeze(1).contiguous()           # [KH,KW,C] -> [C,1,KH,KW]
        elif key.endswith(".weight") and key.split(".")[0] in _POINTWISE:
            if v.dim() != 2:
                raise ValueError("%s: expected a Linear weight [O,I], got %s" % (key, tuple(v.shape)))
            out[key] = v[:, :, None, None].contiguous()
        else:
            out[key] = v
    return out
