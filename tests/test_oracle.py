"""CPU tests of the oracle itself: independent properties and the committed golden vectors that the
reference's own device kernels produced (tests/golden/make_golden.py)."""
import dataclasses
import os

import numpy as np
import pytest
import torch
import torch.nn.functional as F

from oracle import oracle as orc
from tests import cases, helpers

GOLDEN = os.path.join(os.path.dirname(__file__), "golden", "reference_vectors.npz")


def _golden_cases():
    d = {c.name: c for c in cases.REFERENCE_RECIPES + cases.CORNERS}
    d["d2_oob_heavy_ref"] = dataclasses.replace(d["d2_oob_heavy"], name="d2_oob_heavy_ref", G=1)
    return d


def test_golden_vectors_from_reference_kernels():
    assert os.path.exists(GOLDEN), "golden vectors missing"
    blob = np.load(GOLDEN)
    table = _golden_cases()
    names = sorted({k.split(".")[0] for k in blob.files})
    assert len(names) >= 10
    for name in names:
        c = table[name]
        out = helpers.run_oracle(c, cases.make_inputs(c))
        tol = 2e-5 if c.dtype == "float32" else 1e-12
        for k in ("y", "dx", "dw", "doff"):
            key = "%s.%s" % (name, k)
            if key not in blob.files:
                continue
            assert out[k].shape == blob[key].shape, key
            assert cases.rel_err(out[k], blob[key]) <= tol, (key, cases.rel_err(out[k], blob[key]))


def test_d3_test_function_known_answer():
    """deform3d/test_function.py recipe, worked by hand: zero offsets, ones weight, dilation 2, pad 1: the taps
    land on input index -1, 1, 3 per axis; only index 1 is inside, so every output equals x[1,1,1] = 2."""
    c = cases.REFERENCE_RECIPES[0]
    out = helpers.run_oracle(c, cases.make_inputs(c))
    assert out["y"].shape == (1, 1, 3, 3, 3)
    # output (l,h,w): taps at o-1+2t; valid where the index is in [0,2]
    x = np.array([[1.0, 1, 1], [2.0, 2, 2], [1.0, 1, 1]])
    exp = np.zeros((3, 3, 3))
    for l in range(3):
        for h in range(3):
            for w in range(3):
                s = 0.0
                for tl in range(3):
                    for th in range(3):
                        for tw in range(3):
                            il, ih, iw = l - 1 + 2 * tl, h - 1 + 2 * th, w - 1 + 2 * tw
                            if 0 <= il < 3 and 0 <= ih < 3 and 0 <= iw < 3:
                                s += x[ih, iw]
                exp[l, h, w] = s
    assert np.array_equal(out["y"][0, 0], exp.astype(np.float32))


@pytest.mark.parametrize("nd", [2, 3])
def test_zero_offsets_equal_plain_convolution(nd):
    rng = np.random.default_rng(1)
    if nd == 3:
        p = orc.Problem(3, 2, 4, 6, (5, 6, 7), (3, 3, 3), (1, 2, 1), (1, 1, 1), (1, 1, 1), 2, 2)
        conv, wshape = F.conv3d, (6, 2, 3, 3, 3)
    else:
        p = orc.Problem(2, 2, 4, 6, (9, 7), (3, 2), (2, 1), (1, 0), (1, 1), 2, 1)
        conv, wshape = F.conv2d, (6, 2, 3, 2)
    x = rng.standard_normal((2, 4) + p.in_size)
    w = rng.standard_normal(wshape)
    b = rng.standard_normal(6)
    off = np.zeros((2, p.offset_channels) + p.out_size)
    dy = rng.standard_normal((2, 6) + p.out_size)
    xt, wt, bt = [torch.from_numpy(a).requires_grad_() for a in (x, w, b)]
    yt = conv(xt, wt, bt, stride=p.stride, padding=p.pad, groups=2)
    yt.backward(torch.from_numpy(dy))
    y = orc.forward(p, x, off, w, b)
    dx, _ = orc.backward_data(p, x, off, w, dy)
    dw = orc.backward_weight(p, x, off, dy)
    assert np.allclose(y, yt.detach().numpy(), atol=1e-12)
    assert np.allclose(dx, xt.grad.numpy(), atol=1e-12)
    assert np.allclose(dw, wt.grad.numpy(), atol=1e-11)
    assert np.allclose(orc.backward_bias(p, dy), bt.grad.numpy(), atol=1e-11)


def test_dilated_zero_offsets_match_torch_on_the_common_region():
    """With dilation > 1 the deformable size rule yields a larger output than the standard rule; the first
    out_std positions per axis use the same taps as torch's dilated convolution."""
    rng = np.random.default_rng(2)
    p = orc.Problem(2, 1, 2, 3, (9, 9), (3, 3), (1, 1), (2, 2), (2, 2), 1, 2)
    x, w = rng.standard_normal((1, 2, 9, 9)), rng.standard_normal((3, 2, 3, 3))
    off = np.zeros((1, p.offset_channels) + p.out_size)
    y = orc.forward(p, x, off, w)
    yt = F.conv2d(torch.from_numpy(x), torch.from_numpy(w), padding=2, dilation=2).numpy()
    assert p.out_size == (11, 11) and yt.shape[-1] == 9
    assert np.allclose(y[..., :9, :9], yt, atol=1e-12)


def test_interior_offsets_match_torchvision():
    torchvision = pytest.importorskip("torchvision")
    rng = np.random.default_rng(3)
    p = orc.Problem(2, 2, 4, 4, (12, 12), (3, 3), (1, 1), (0, 0), (1, 1), 2, 2)
    x, w = rng.standard_normal((2, 4, 12, 12)), rng.standard_normal((4, 2, 3, 3))
    off = rng.uniform(-0.9, 0.9, (2, p.offset_channels) + p.out_size)
    y = orc.forward(p, x, off, w)
    yt = torchvision.ops.deform_conv2d(torch.from_numpy(x), torch.from_numpy(off), torch.from_numpy(w)).numpy()
    # away from the one-pixel border band the two border rules (edge-replicate vs zero padding) agree
    assert np.allclose(y[..., 1:-1, 1:-1], yt[..., 1:-1, 1:-1], atol=1e-12)


def test_plain_conv_path_matches_torch():
    rng = np.random.default_rng(4)
    p = orc.Problem(2, 2, 6, 9, (11, 9), (3, 3), (2, 1), (1, 2), (1, 2), 3, 6, deformable=False, std_size_rule=True)
    x, w = rng.standard_normal((2, 6, 11, 9)), rng.standard_normal((9, 2, 3, 3))
    dy = rng.standard_normal((2, 9) + p.out_size)
    xt, wt = [torch.from_numpy(a).requires_grad_() for a in (x, w)]
    yt = F.conv2d(xt, wt, None, stride=(2, 1), padding=(1, 2), dilation=(1, 2), groups=3)
    assert tuple(yt.shape[2:]) == p.out_size
    yt.backward(torch.from_numpy(dy))
    assert np.allclose(orc.forward(p, x, None, w), yt.detach().numpy(), atol=1e-12)
    assert np.allclose(orc.backward_data(p, x, None, w, dy)[0], xt.grad.numpy(), atol=1e-12)
    assert np.allclose(orc.backward_weight(p, x, None, dy), wt.grad.numpy(), atol=1e-11)


@pytest.mark.parametrize("nd", [2, 3])
def test_fp64_finite_differences(nd):
    """Central differences for all four gradients, away from lattice kinks, pull-back term disabled."""
    rng = np.random.default_rng(5)
    if nd == 2:
        p = orc.Problem(2, 1, 2, 2, (5, 5), (2, 2), (1, 1), (1, 1), (1, 2), 1, 1, oob_offset_grad=False)
    else:
        p = orc.Problem(3, 1, 2, 2, (3, 4, 4), (2, 2, 2), (1, 1, 1), (1, 1, 1), (1, 1, 1), 2, 1, oob_offset_grad=False)
    x = rng.standard_normal((1, 2) + p.in_size)
    w = rng.standard_normal((2, 2 // p.G) + p.kernel)
    off = rng.uniform(0.15, 0.85, (1, p.offset_channels) + p.out_size) + rng.integers(-1, 2, (1, p.offset_channels) + p.out_size)
    dy = rng.standard_normal((1, 2) + p.out_size)
    dx, doff = orc.backward_data(p, x, off, w, dy)
    dw = orc.backward_weight(p, x, off, dy)
    loss = lambda x_, o_, w_: float((orc.forward(p, x_, o_, w_) * dy).sum())
    eps = 1e-6
    for arr, grad, idx in ((x, dx, 0), (off, doff, 1), (w, dw, 2)):
        flat = arr.reshape(-1)
        for e in rng.choice(flat.size, size=min(40, flat.size), replace=False):
            old = flat[e]
            flat[e] = old + eps
            up = loss(x, off, w)
            flat[e] = old - eps
            dn = loss(x, off, w)
            flat[e] = old
            num = (up - dn) / (2 * eps)
            assert abs(num - grad.reshape(-1)[e]) <= 1e-5 + 1e-3 * abs(num), (idx, e, num, grad.reshape(-1)[e])


def test_oob_pullback_term_follows_the_reference_rule():
    """Invalid 3-D samples: -|col| where p_d <= -1, +|col| where p_d >= in[0] (the LENGTH on every axis)."""
    p = orc.Problem(3, 1, 1, 1, (2, 6, 6), (1, 1, 1), (1, 1, 1), (0, 0, 0), (1, 1, 1), 1, 1)
    x = np.ones((1, 1, 2, 6, 6), np.float32)
    w = np.ones((1, 1, 1, 1, 1), np.float32)
    dy = np.full((1, 1) + p.out_size, 3.0, np.float32)
    off = np.zeros((1, 3) + p.out_size, np.float32)
    off[0, 0, 0, 0, 0] = -5.0        # l far below -> invalid, l component gets -|col|
    off[0, 1, 1, 0, 0] = 10.0        # h beyond the input -> invalid; h = 10 >= in[0] = 2 -> +|col| on h
    off[0, 0, 1, 2, 2] = 7.0         # l beyond -> invalid; h = 2 >= in[0] = 2 also gets +|col| although in range
    _, doff = orc.backward_data(p, x, off, w, dy)
    assert doff[0, 0, 0, 0, 0] == -3.0 and doff[0, 1, 0, 0, 0] == 0.0 and doff[0, 2, 0, 0, 0] == 0.0
    assert doff[0, 1, 1, 0, 0] == 3.0 and doff[0, 0, 1, 0, 0] == 0.0
    assert doff[0, 0, 1, 2, 2] == 3.0 and doff[0, 1, 1, 2, 2] == 3.0 and doff[0, 2, 1, 2, 2] == 3.0
    p0 = orc.Problem(3, 1, 1, 1, (2, 6, 6), (1, 1, 1), (1, 1, 1), (0, 0, 0), (1, 1, 1), 1, 1, oob_offset_grad=False)
    _, doff0 = orc.backward_data(p0, x, off, w, dy)
    assert doff0[0, 0, 0, 0, 0] == 0.0 and doff0[0, 1, 1, 0, 0] == 0.0


def test_truncation_and_edge_rule():
    """p in (-1, 0): low = trunc(p) = 0 and high = low, so the value is the edge pixel (weights 1-f and f)."""
    p = orc.Problem(2, 1, 1, 1, (3, 3), (1, 1), (1, 1), (0, 0), (1, 1), 1, 1)
    off = np.zeros((1, 2, 3, 3), np.float32)
    off[0, 0, 0, 0] = -0.5
    off[0, 1, 2, 2] = 0.75           # w = 2.75 >= in-1 -> high = low = 2
    pts, valid, lo, hi = orc.dump_points(p, off[0])
    assert valid[0, 0, 0] == 1 and lo[0, 0, 0, 0] == 0 and hi[0, 0, 0, 0] == 0
    assert valid[0, 0, 8] == 1 and lo[0, 0, 8, 1] == 2 and hi[0, 0, 8, 1] == 2
    x = np.arange(9, dtype=np.float32).reshape(1, 1, 3, 3) + 1
    y = orc.forward(p, x, off, np.ones((1, 1, 1, 1), np.float32))
    assert y[0, 0, 0, 0] == 1.0 and y[0, 0, 2, 2] == 9.0
    off[0, 0, 0, 0] = -1.0           # exactly -1 is invalid
    assert orc.forward(p, x, off, np.ones((1, 1, 1, 1), np.float32))[0, 0, 0, 0] == 0.0
