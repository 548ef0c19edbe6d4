"""Pins the CPU oracle: against the golden outputs of the unmodified reference
(tests/golden/*.npz, produced by tests/golden/make_golden.py) and against the torch CPU ops the
reference itself uses as comparator.  No GPU needed."""
import numpy as np
import pytest
import torch

from conftest import assert_close_fp32, draw, golden
from oracle import oracle


@pytest.mark.parametrize("name", ["k3", "k9", "k13", "k17"])
def test_dwconv_matches_reference_golden(name):
    g = golden("dwconv_small.npz")
    B, H, W, C, k, seed = [int(v) for v in g[name + ".meta"]]
    x, w, go = draw([(B, H, W, C), (k, k, C), (B, H, W, C)], seed)
    w = w / k
    p = k // 2
    assert_close_fp32(oracle.c_dwconv_fwd(x, w, padding=p), g[name + ".y"], "y")
    assert_close_fp32(oracle.c_dwconv_bwd_input(go, w, (H, W), padding=p), g[name + ".dx"], "dx")
    dw, _ = oracle.c_dwconv_bwd_weight(x, go, k, padding=p)
    assert_close_fp32(dw, g[name + ".dw"], "dw")


def test_dwconv_general_forward_matches_reference_golden():
    g = golden("dwconv_small.npz")
    B, H, W, C, k, seed = [int(v) for v in g["general.meta"]]
    x, w = draw([(B, H, W, C), (k, k, C)], seed)
    w = w / k
    assert_close_fp32(oracle.c_dwconv_fwd(x, w, stride=2, padding=1), g["general.s2p1.y"], "s2p1")
    assert_close_fp32(oracle.c_dwconv_fwd(x, w, padding=4, dilation=2), g["general.d2p4.y"], "d2p4")
    assert_close_fp32(oracle.c_dwconv_fwd(x, w, padding=0), g["general.p0.y"], "p0")


def test_dwconv_half_forward_matches_reference_golden():
    g = golden("dwconv_small.npz")
    B, H, W, C, k, seed = [int(v) for v in g["half.meta"]]
    x, w = draw([(B, H, W, C), (k, k, C)], seed)
    x, w = x.half().float(), (w / k).half().float()
    y = oracle.c_dwconv_fwd(x, w, padding=k // 2)
    # the reference output is fp16: round the oracle the same way, allow one fp16 ulp
    ref = g["half.k9.y"]
    assert np.abs(torch.from_numpy(y).half().float().numpy() - ref).max() <= 2e-3 * max(1.0, np.abs(ref).max())


@pytest.mark.parametrize("name", ["16to8", "16to4", "12x8to6x2"])
def test_pool_matches_reference_golden(name):
    g = golden("pool_small.npz")
    B, H, W, C, oh, ow, seed = [int(v) for v in g[name + ".meta"]]
    x, go = draw([(B, H, W, C), (B, oh, ow, C)], seed)
    assert_close_fp32(oracle.c_pool_fwd(x.numpy(), (oh, ow)), g[name + ".y"], "y")
    assert_close_fp32(oracle.c_pool_bwd(go.numpy(), (H, W)), g[name + ".dx"], "dx")


@pytest.mark.parametrize("name", ["8to16", "6x5to15x11", "4to16"])
def test_upsample_matches_reference_golden(name):
    g = golden("upsample_small.npz")
    B, h, w, C, H, W, seed = [int(v) for v in g[name + ".meta"]]
    (x,) = draw([(B, h, w, C)], seed)
    assert_close_fp32(oracle.c_upsample_fwd(x.numpy(), (H, W)), g[name + ".y"], "y")


def test_block_restatement_matches_reference_golden():
    """ref_block_forward (the torch composition) reproduces the reference ConvBlock run on config 1."""
    g = golden("convblock_cfg1.npz")
    params = {k[len("param."):]: torch.from_numpy(g[k]) for k in g.files if k.startswith("param.")}
    (x,) = draw([(2, 32, 32, 64)], 0)
    (go,) = draw([(2, 32, 32, 64)], 1)
    for dtype in (torch.float64, torch.float32):
        y, dx, grads = oracle.ref_block_forward_backward(x, go, params, dtype=dtype)
        assert_close_fp32(y.numpy(), g["y"], "y %s" % dtype)
        assert_close_fp32(dx.numpy(), g["dx"], "dx %s" % dtype)
        for k, v in grads.items():
            assert_close_fp32(v.numpy(), g["grad." + k], "grad %s %s" % (k, dtype))


@pytest.mark.parametrize("geom", [
    dict(k=(3, 3), stride=1, padding=1, dilation=1),
    dict(k=(5, 3), stride=(2, 1), padding=(2, 0), dilation=1),
    dict(k=(3, 3), stride=2, padding=2, dilation=2),
    dict(k=(7, 7), stride=1, padding=0, dilation=1),
])
def test_c_oracle_matches_torch_conv(geom):
    B, H, W, C = 2, 13, 11, 6
    x, w, b = draw([(B, H, W, C), geom["k"] + (C,), (C,)], 5)
    xt = x.double().requires_grad_(True)
    wt = w.double().requires_grad_(True)
    bt = b.double().requires_grad_(True)
    y = oracle.torch_dwconv(xt, wt, bt, geom["stride"], geom["padding"], geom["dilation"])
    (go,) = draw([tuple(y.shape)], 6)
    y.backward(go.double())
    assert_close_fp32(oracle.c_dwconv_fwd(x, w, b, geom["stride"], geom["padding"], geom["dilation"]), y.detach().numpy())
    assert_close_fp32(oracle.c_dwconv_bwd_input(go, w, (H, W), geom["stride"], geom["padding"], geom["dilation"]),
                      xt.grad.numpy())
    dw, db = oracle.c_dwconv_bwd_weight(x, go, geom["k"], geom["stride"], geom["padding"], geom["dilation"])
    assert_close_fp32(dw, wt.grad.numpy())
    assert_close_fp32(db, bt.grad.numpy())


@pytest.mark.parametrize("sizes", [((16, 16), (8, 8)), ((15, 9), (4, 7)), ((7, 7), (7, 7)), ((5, 6), (9, 8))])
def test_c_oracle_matches_torch_pool_and_upsample(sizes):
    (H, W), (OH, OW) = sizes
    (x,) = draw([(2, H, W, 4)], 7)
    xt = x.double().requires_grad_(True)
    y = oracle.torch_pool(xt, (OH, OW))
    (go,) = draw([tuple(y.shape)], 8)
    y.backward(go.double())
    assert_close_fp32(oracle.c_pool_fwd(x.numpy(), (OH, OW)), y.detach().numpy())
    assert_close_fp32(oracle.c_pool_bwd(go.numpy(), (H, W)), xt.grad.numpy())
    # resize (H,W) -> (OH,OW) in both directions of scale
    xt = x.double().requires_grad_(True)
    y = oracle.torch_upsample(xt, (OH, OW))
    y.backward(go.double())
    assert_close_fp32(oracle.c_upsample_fwd(x.numpy(), (OH, OW)), y.detach().numpy())
    assert_close_fp32(oracle.c_upsample_bwd(go.numpy(), (H, W)), xt.grad.numpy())


def test_known_answers():
    # a centred delta filter is the identity; an all-ones filter is a box sum
    (x,) = draw([(1, 6, 7, 4)], 9)
    w = torch.zeros(5, 5, 4)
    w[2, 2, :] = 1
    assert np.array_equal(oracle.c_dwconv_fwd(x, w, padding=2), x.numpy())
    ones = torch.ones(3, 3, 4)
    box = oracle.c_dwconv_fwd(torch.ones(1, 5, 5, 4), ones, padding=1)
    assert box[0, 2, 2, 0] == 9 and box[0, 0, 0, 0] == 4 and box[0, 0, 2, 0] == 6
    # constants survive pooling and resizing
    const = np.full((1, 9, 7, 2), 3.25, np.float32)
    assert np.allclose(oracle.c_pool_fwd(const, (4, 3)), 3.25)
    assert np.allclose(oracle.c_upsample_fwd(const, (18, 15)), 3.25)


# ---------------------------------------------------------------------------------------------
# Adjoint identities: every backward restatement is the transpose of its forward (which the golden
# vectors above pin to the reference).  <A x, g> == <x, A^T g> up to fp32 output rounding.
# ---------------------------------------------------------------------------------------------
def _dot(a, b):
    return float(np.sum(a.astype(np.float64) * b.astype(np.float64)))


@pytest.mark.parametrize("geom", [
    dict(k=(9, 9), stride=1, padding=4, dilation=1),
    dict(k=(17, 17), stride=1, padding=8, dilation=1),
    dict(k=(5, 3), stride=(2, 1), padding=(0, 2), dilation=1),
    dict(k=(3, 3), stride=2, padding=1, dilation=2),
    dict(k=(7, 7), stride=1, padding=0, dilation=1),
])
def test_c_oracle_conv_backward_is_the_adjoint_of_forward(geom):
    rng = np.random.default_rng(31)
    k = geom["k"]
    x = rng.standard_normal((2, 19, 23, 8)).astype(np.float32)
    w = rng.standard_normal(k + (8,)).astype(np.float32)
    y = oracle.c_dwconv_fwd(x, w, None, geom["stride"], geom["padding"], geom["dilation"])
    g = rng.standard_normal(y.shape).astype(np.float32)
    dx = oracle.c_dwconv_bwd_input(g, w, (19, 23), geom["stride"], geom["padding"], geom["dilation"])
    dw, db = oracle.c_dwconv_bwd_weight(x, g, k, geom["stride"], geom["padding"], geom["dilation"])
    ref = _dot(y, g)
    scale = float(np.sqrt(_dot(y, y) * _dot(g, g)))
    assert abs(_dot(x, dx) - ref) <= 1e-5 * scale          # linear in x
    assert abs(_dot(w, dw) - ref) <= 1e-5 * scale          # and in w
    np.testing.assert_allclose(db, g.astype(np.float64).sum(axis=(0, 1, 2)), rtol=1e-5, atol=1e-4)


@pytest.mark.parametrize("sizes", [((16, 16), (8, 8)), ((15, 9), (4, 7)), ((96, 96), (48, 48)), ((5, 6), (9, 8)),
                                   ((7, 7), (1, 1))])
def test_c_oracle_resample_backward_is_the_adjoint_of_forward(sizes):
    (H, W), (h, w) = sizes
    rng = np.random.default_rng(32)
    big = rng.standard_normal((2, H, W, 4)).astype(np.float32)
    small = rng.standard_normal((2, h, w, 4)).astype(np.float32)
    # pool: [H,W] -> [h,w];  its adjoint maps [h,w] -> [H,W]
    lhs = _dot(oracle.c_pool_fwd(big, (h, w)), small)
    rhs = _dot(big, oracle.c_pool_bwd(small, (H, W)))
    assert abs(lhs - rhs) <= 1e-5 * max(1.0, abs(lhs))
    # upsample: [h,w] -> [H,W];  its adjoint maps [H,W] -> [h,w]
    lhs = _dot(oracle.c_upsample_fwd(small, (H, W)), big)
    rhs = _dot(small, oracle.c_upsample_bwd(big, (h, w)))
    assert abs(lhs - rhs) <= 1e-5 * max(1.0, abs(lhs))


# ---------------------------------------------------------------------------------------------
# Randomised geometry: the C restatement against the torch ops the reference names as its CPU
# equivalent (F.conv2d(groups=C), adaptive_avg_pool2d, bilinear interpolate), forward and backward.
# ---------------------------------------------------------------------------------------------
from hypothesis import given, settings, HealthCheck  # noqa: E402
from hypothesis import strategies as st  # noqa: E402


@settings(max_examples=40, deadline=None, suppress_health_check=list(HealthCheck), derandomize=True)
@given(st.data())
def test_c_oracle_matches_torch_conv_random_geometry(data):
    kh, kw = data.draw(st.integers(1, 7)), data.draw(st.integers(1, 7))
    sh, sw = data.draw(st.integers(1, 3)), data.draw(st.integers(1, 3))
    dh, dw_ = data.draw(st.integers(1, 2)), data.draw(st.integers(1, 2))
    ph, pw = data.draw(st.integers(0, 4)), data.draw(st.integers(0, 4))
    H = data.draw(st.integers(dh * (kh - 1) + 1, 14))
    W = data.draw(st.integers(dw_ * (kw - 1) + 1, 14))
    B, C = data.draw(st.integers(1, 2)), data.draw(st.integers(1, 5))
    seed = data.draw(st.integers(0, 10 ** 6))
    k, s, p, d = (kh, kw), (sh, sw), (ph, pw), (dh, dw_)
    x, w, b = draw([(B, H, W, C), k + (C,), (C,)], seed)
    xt, wt, bt = (t.double().requires_grad_(True) for t in (x, w, b))
    y = oracle.torch_dwconv(xt, wt, bt, s, p, d)
    (go,) = draw([tuple(y.shape)], seed + 1)
    y.backward(go.double())
    assert_close_fp32(oracle.c_dwconv_fwd(x, w, b, s, p, d), y.detach().numpy())
    assert_close_fp32(oracle.c_dwconv_bwd_input(go, w, (H, W), s, p, d), xt.grad.numpy())
    dw, db = oracle.c_dwconv_bwd_weight(x, go, k, s, p, d)
    assert_close_fp32(dw, wt.grad.numpy())
    assert_close_fp32(db, bt.grad.numpy())


@settings(max_examples=40, deadline=None, suppress_health_check=list(HealthCheck), derandomize=True)
@given(st.integers(1, 20), st.integers(1, 20), st.integers(1, 20), st.integers(1, 20), st.integers(0, 10 ** 6))
def test_c_oracle_matches_torch_resample_random_sizes(H, W, OH, OW, seed):
    (x,) = draw([(2, H, W, 3)], seed)
    for torch_op, c_fwd, c_bwd in ((oracle.torch_pool, oracle.c_pool_fwd, oracle.c_pool_bwd),
                                   (oracle.torch_upsample, oracle.c_upsample_fwd, oracle.c_upsample_bwd)):
        xt = x.double().requires_grad_(True)
        y = torch_op(xt, (OH, OW))
        (go,) = draw([tuple(y.shape)], seed + 1)
        y.backward(go.double())
        assert_close_fp32(c_fwd(x.numpy(), (OH, OW)), y.detach().numpy())
        assert_close_fp32(c_bwd(go.numpy(), (H, W)), xt.grad.numpy())
