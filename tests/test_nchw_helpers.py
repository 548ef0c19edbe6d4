"""Host-side helpers for models written against the NCHW form of the block: layout views that do
not copy, and the parameter conversion between the NCHW (nn.Conv2d-shaped) and NHWC forms, checked
against the oracle's restatement of the reference's NCHW block (pyramid_dwconv/conv_block.py:50-97)."""
import pytest
import torch

from oracle import oracle
from pyramidconvblock_b200 import nchw
from pyramidconvblock_b200.modules import ConvBlock


def _nchw_params(dim, k, scales, bias, seed):
    g = torch.Generator().manual_seed(seed)
    inter = dim // 2
    p = {"conv_up.weight": torch.randn((inter, dim, 1, 1), generator=g, dtype=torch.float64) / dim ** 0.5}
    if bias:
        p["conv_up.bias"] = torch.randn((inter,), generator=g, dtype=torch.float64)
    for i in range(len(scales)):
        p["gates.%d.conv_spatial.weight" % i] = torch.randn((inter, 1, k, k), generator=g, dtype=torch.float64) / k
    p["conv_out.weight"] = torch.randn((dim, inter // 2 * len(scales), 1, 1), generator=g, dtype=torch.float64) / inter ** 0.5
    p["conv_out.bias"] = torch.randn((dim,), generator=g, dtype=torch.float64)
    p["conv_pool.weight"] = torch.randn((dim, dim, 1, 1), generator=g, dtype=torch.float64) / dim ** 0.5
    p["conv_pool.bias"] = torch.randn((dim,), generator=g, dtype=torch.float64)
    return p


@pytest.mark.parametrize("scales,bias", [((1., 0.5), False), ((1., 0.5, 0.25), True), ((0.5,), False)])
def test_converted_parameters_give_the_same_block(scales, bias):
    dim, k = 16, 5
    p_nchw = _nchw_params(dim, k, scales, bias, seed=11)
    x = torch.randn((2, dim, 12, 20), generator=torch.Generator().manual_seed(12), dtype=torch.float64)
    y_nchw = oracle.ref_block_forward_nchw(x, p_nchw, scales)
    p_nhwc = nchw.nhwc_state_dict_from_nchw(p_nchw)
    assert p_nhwc["conv_up.weight"].shape == (dim // 2, dim)
    assert p_nhwc["gates.0.conv_spatial.weight"].shape == (k, k, dim // 2)
    y_nhwc = oracle.ref_block_forward(x.permute(0, 2, 3, 1), p_nhwc, scales)
    torch.testing.assert_close(y_nhwc.permute(0, 3, 1, 2), y_nchw, rtol=1e-12, atol=1e-12)
    back = nchw.nchw_state_dict_from_nhwc(p_nhwc)
    assert back.keys() == p_nchw.keys()
    for key in p_nchw:
        assert back[key].shape == p_nchw[key].shape and torch.equal(back[key], p_nchw[key]), key


def test_converted_state_dict_loads_into_the_module():
    dim, k = 16, 5
    p_nchw = _nchw_params(dim, k, (1., 0.5), False, seed=13)
    m = nchw.ConvBlockNCHW(dim, kernel_size=k)
    assert list(m.state_dict().keys()) == list(ConvBlock(dim, kernel_size=k).state_dict().keys())
    m.load_state_dict(nchw.nhwc_state_dict_from_nchw(p_nchw), strict=True)
    assert m.gates[1].conv_spatial.weight.shape == (k, k, dim // 2)


def test_wrong_shapes_are_refused():
    with pytest.raises(ValueError):
        nchw.nhwc_state_dict_from_nchw({"conv_up.weight": torch.zeros(4, 8)})
    with pytest.raises(ValueError):
        nchw.nhwc_state_dict_from_nchw({"gates.0.conv_spatial.weight": torch.zeros(4, 2, 3, 3)})
    with pytest.raises(ValueError):
        nchw.nchw_state_dict_from_nhwc({"gates.0.conv_spatial.weight": torch.zeros(4, 1, 3, 3)})
    with pytest.raises(ValueError):
        nchw.nchw_as_nhwc(torch.zeros(2, 3, 4))


def test_layout_views_do_not_copy_channels_last_storage():
    x = torch.randn(2, 8, 5, 7).contiguous(memory_format=torch.channels_last)
    v = nchw.nchw_as_nhwc(x)
    assert v.shape == (2, 5, 7, 8) and v.is_contiguous() and v.data_ptr() == x.data_ptr()
    assert nchw.shares_memory_with_nhwc_view(x)
    plain = torch.randn(2, 8, 5, 7)
    assert not nchw.shares_memory_with_nhwc_view(plain)
    c = nchw.nchw_as_nhwc(plain)
    assert c.is_contiguous() and c.data_ptr() != plain.data_ptr() and torch.equal(c, plain.permute(0, 2, 3, 1))
    y = nchw.nhwc_as_nchw(v)
    assert y.shape == x.shape and y.data_ptr() == x.data_ptr() and y.is_contiguous(memory_format=torch.channels_last)


@pytest.mark.gpu
def test_nchw_block_on_gpu_equals_nhwc_block_and_oracle():
    """ConvBlockNCHW on a channels_last tensor: no layout copy, bit-identical to ConvBlock on the NHWC
    view, and within the 16-bit bar of the oracle's NCHW block evaluated in fp32."""
    import numpy as np
    from conftest import assert_close_16bit, draw
    from pyramidconvblock_b200 import ops
    dim, k = 64, 9
    torch.manual_seed(5)
    m = nchw.ConvBlockNCHW(dim, kernel_size=k).to(torch.float16).cuda()
    ref = ConvBlock(dim, kernel_size=k).to(torch.float16).cuda()
    ref.load_state_dict(m.state_dict())
    (x,) = draw([(2, dim, 24, 40)], 21)
    (go,) = draw([(2, dim, 24, 40)], 22)
    xd = x.half().cuda().contiguous(memory_format=torch.channels_last).requires_grad_(True)
    god = go.half().cuda().contiguous(memory_format=torch.channels_last)
    y = m(xd)
    assert y.shape == xd.shape and y.is_contiguous(memory_format=torch.channels_last)
    y.backward(god)
    ops.check_device_status()
    xn = xd.detach().permute(0, 2, 3, 1).requires_grad_(True)
    assert xn.is_contiguous() and xn.data_ptr() == xd.data_ptr()
    yn = ref(xn)
    yn.backward(god.permute(0, 2, 3, 1))
    assert torch.equal(y.detach().permute(0, 2, 3, 1), yn.detach())
    # same kernels on the same memory; a tolerance only because the library GEMMs of the backward pass
    # are not promised to be bitwise repeatable between calls
    torch.testing.assert_close(xd.grad.permute(0, 2, 3, 1), xn.grad, rtol=1e-3, atol=1e-3)
    for (name, p), q in zip(m.named_parameters(), ref.parameters()):
        tol = 1e-3 * max(1.0, float(q.grad.float().abs().max()))
        torch.testing.assert_close(p.grad.float(), q.grad.float(), rtol=1e-3, atol=tol, msg=name)
    p_nchw = nchw.nchw_state_dict_from_nhwc({key: v.detach().float().cpu() for key, v in m.state_dict().items()})
    y_ref = oracle.ref_block_forward_nchw(x.half().float(), p_nchw).numpy()
    assert_close_16bit(y.detach().float().cpu().numpy(), y_ref, "y", rtol=2e-2,
                       atol=2e-3 + 1e-2 * float(np.abs(y_ref).max()))
