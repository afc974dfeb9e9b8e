"""The deformable layer (offset-producing convolution + deformable convolution in one library call) against the
composition of its two halves, which the other GPU tests pin to the oracle one by one.

Caller pattern: deform3d/test_model.py:18-30, deform2d/test_model.py:19-31 (a stock convolution produces the
offsets, ``ConvOffset3d`` consumes them).  Gates: fp32 path 1e-4, bf16 path 2e-2 (max|a-b| / max|b|)."""
import numpy as np
import pytest
import torch

from tests import cases

pytestmark = pytest.mark.gpu

TOL_FP32 = 1e-4
TOL_BF16 = 2e-2


def _rel(a, b):
    return cases.rel_err(a.detach().double().cpu().numpy(), b.detach().double().cpu().numpy())


def _stock_conv(ndim):
    return torch.nn.functional.conv3d if ndim == 3 else torch.nn.functional.conv2d


def _make(ndim, N, C, O, size, k, stride, pad, dil, dg, G, seed, offset_std=0.3):
    import deform_conv3d_pytorch_op_b200 as dcn
    torch.manual_seed(seed)
    cls = dcn.DeformLayer3d if ndim == 3 else dcn.DeformLayer2d
    m = cls(C, O, k, stride=stride, padding=pad, dilation=dil, deformable_groups=dg, groups=G, offset_std=offset_std).cuda()
    with torch.no_grad():
        m.conv_offset.bias.uniform_(-0.5, 0.5)
    x = torch.randn((N, C) + tuple(size), device="cuda")
    return m, x


@pytest.mark.parametrize("ndim,N,C,O,size,k,stride,pad,dil,dg,G", [
    (2, 2, 8, 6, (9, 11), 3, 1, 1, 1, 2, 1),
    (2, 1, 4, 4, (7, 7), 3, 2, 2, 2, 4, 2),
    (3, 2, 4, 6, (5, 6, 7), 3, 1, 1, 1, 2, 2),
    (3, 1, 2, 2, (4, 5, 5), (1, 3, 3), (1, 2, 1), (0, 1, 1), 1, 1, 1),
])
def test_layer_equals_its_two_halves_fp32(ndim, N, C, O, size, k, stride, pad, dil, dg, G):
    """Exact precision: offsets from the library's plain-convolution kernel, then the deformable kernels; the
    reference composition is torch's fp32 convolution followed by this package's ConvOffset function (itself
    oracle-checked in test_parity_gpu.py)."""
    import deform_conv3d_pytorch_op_b200 as dcn
    m, x = _make(ndim, N, C, O, size, k, stride, pad, dil, dg, G, seed=11)
    x.requires_grad_(True)
    y = m(x)
    c = m.conv
    fn = dcn.ConvOffset3dFunction if ndim == 3 else dcn.ConvOffset2dFunction
    with torch.backends.cudnn.flags(enabled=True, allow_tf32=False):
        off = _stock_conv(ndim)(x, m.conv_offset.weight, m.conv_offset.bias, stride=c.stride, padding=c.padding)
        ref = fn.apply(x, off, c.weight, c.bias, c.stride, c.padding, c.dilation, c.channel_per_group, c.group)
        assert y.shape == ref.shape
        dy = torch.randn_like(ref)
        params = [x, m.conv_offset.weight, m.conv_offset.bias, c.weight, c.bias]
        want = torch.autograd.grad(ref, params, dy)
    got = torch.autograd.grad(y, params, dy)
    assert _rel(y, ref) <= TOL_FP32
    for name, a, b in zip(("dx", "doffset_weight", "doffset_bias", "dweight", "dbias"), got, want):
        assert _rel(a, b) <= TOL_FP32, name
    # these sizes take the single-kernel forward whose offsets never leave the SM before they are used
    import ctypes
    from deform_conv3d_pytorch_op_b200 import _lib
    op = dcn.Op(x, c.weight, c.stride, c.padding, c.dilation, c.channel_per_group, c.group)
    assert _lib.lib().dcn_layer_launch_count(ctypes.byref(op.p), _lib.PASS_FORWARD) == 1
    assert _lib.lib().dcn_layer_launch_count(ctypes.byref(op.p), _lib.PASS_BACKWARD) == 2     # zero fill + one kernel
    y2, off2 = op.layer_forward(x.detach(), m.conv_offset.weight, m.conv_offset.bias, c.weight, c.bias)
    assert _rel(off2, off) <= 1e-5 and _rel(y2, ref) <= TOL_FP32


@pytest.mark.parametrize("ndim,channels_last", [(2, False), (3, False), (3, True)])
def test_layer_bf16_against_separate_calls_and_fp32(ndim, channels_last):
    """bf16 precision.  (a) the single call equals the two separate library calls (plain convolution, then the
    deformable operator on ITS offsets) up to the order of the floating-point reductions; (b) offsets against the
    fp32 convolution and y against the exact deformable operator evaluated at the layer's own offsets, 2e-2."""
    import deform_conv3d_pytorch_op_b200 as dcn
    size = (12, 13) if ndim == 2 else (4, 9, 10)
    m, x = _make(ndim, 2, 32, 24, size, 3, 1, 1, 1, 2, 1, seed=5)
    m.conv.precision = "bf16"
    if channels_last:
        x = x.contiguous(memory_format=torch.channels_last_3d)
    c = m.conv
    op = dcn.Op(x, c.weight, c.stride, c.padding, c.dilation, c.channel_per_group, c.group, precision="bf16")
    assert op.channels_last == channels_last
    y, off, ws = op.layer_forward(x, m.conv_offset.weight, m.conv_offset.bias, c.weight, c.bias, keep_workspace=True)
    dy = torch.randn_like(y)
    dx, dow, dob, dw, db = op.layer_backward(x, off, m.conv_offset.weight, c.weight, dy, True, True, True, True, True, ws)
    dcn.check_status()
    # (a) the same kernels, called one by one
    xs = x.contiguous() if channels_last else x           # the plain-convolution Op of the offsets is channel-first
    conv = dcn.Conv3dFunction if ndim == 3 else dcn.Conv2dFunction
    off2 = conv.apply(xs, m.conv_offset.weight, m.conv_offset.bias, c.stride, c.padding, 1, 1, "bf16")
    assert _rel(off, off2) <= 1e-6
    y2 = op.forward(x, off, c.weight, c.bias)
    assert _rel(y, y2) <= 1e-6
    dx_m, doff, dw2, db2 = op.backward(x, off, c.weight, dy, True, True, True, True)
    opq = dcn.Op(xs, m.conv_offset.weight, c.stride, c.padding, 1, x.size(1), 1, deformable=False, std_size_rule=True,
                 precision="bf16")
    dx_q, _, dow2, dob2 = opq.backward(xs, None, m.conv_offset.weight, doff, True, False, True, True)
    assert _rel(dw, dw2) <= 1e-5 and _rel(db, db2) <= 1e-5
    # (gates downstream of dOffset are wider: its last bits depend on the order of the slabs' atomics, and a value on a
    # bf16 rounding boundary moves the packed operand of the plain convolution's gradient kernels by one bf16 step)
    assert _rel(dow, dow2) <= 1e-3 and _rel(dob, dob2) <= 1e-4
    assert _rel(dx, dx_m + dx_q) <= 1e-3
    # (b) against fp32 arithmetic
    with torch.backends.cudnn.flags(enabled=True, allow_tf32=False):
        off_ref = _stock_conv(ndim)(xs, m.conv_offset.weight, m.conv_offset.bias, stride=c.stride, padding=c.padding)
    assert _rel(off, off_ref) <= TOL_BF16
    fn = dcn.ConvOffset3dFunction if ndim == 3 else dcn.ConvOffset2dFunction
    y_ref = fn.apply(xs, off, c.weight, c.bias, c.stride, c.padding, c.dilation, c.channel_per_group, c.group, "exact")
    assert _rel(y, y_ref) <= TOL_BF16


def test_layer_module_trains_and_state_dict_names():
    """The module keeps the parameter names of the two-module pattern and its gradients flow to all four."""
    import deform_conv3d_pytorch_op_b200 as dcn
    m, x = _make(3, 1, 8, 8, (3, 6, 6), 3, 1, 1, 1, 1, 1, seed=2)
    assert sorted(m.state_dict().keys()) == ["conv.bias", "conv.weight", "conv_offset.bias", "conv_offset.weight"]
    m(x).square().mean().backward()
    for name, p in m.named_parameters():
        assert p.grad is not None and torch.isfinite(p.grad).all() and p.grad.abs().max() > 0, name


def test_layer_rejects_wrong_offset_weight_shape():
    import deform_conv3d_pytorch_op_b200 as dcn
    m, x = _make(2, 1, 8, 8, (6, 6), 3, 1, 1, 1, 1, 1, seed=2)
    c = m.conv
    op = dcn.Op(x, c.weight, c.stride, c.padding, c.dilation, c.channel_per_group, c.group)
    with pytest.raises(dcn.DcnError):
        op.layer_forward(x, m.conv_offset.weight[:, :4].contiguous(), None, c.weight, None)


def test_layer_at_benchmark_shape_matches_separate_calls():
    """Config-2 shape (256 -> 256 channels, 56 x 56, 4 deformable groups) at batch 4, bf16 path: the shared-memory
    backward-data kernel and the table-driven forward / weight kernels inside the layer call give what the separate
    calls give; offsets against the fp32 convolution within the bf16 gate."""
    import deform_conv3d_pytorch_op_b200 as dcn
    m, x = _make(2, 4, 256, 256, (56, 56), 3, 1, 1, 1, 4, 1, seed=9, offset_std=0.02)
    c = m.conv
    op = dcn.Op(x, c.weight, c.stride, c.padding, c.dilation, c.channel_per_group, c.group, precision="bf16")
    y, off, ws = op.layer_forward(x, m.conv_offset.weight, m.conv_offset.bias, c.weight, c.bias, keep_workspace=True)
    dy = torch.randn_like(y)
    dx, dow, dob, dw, db = op.layer_backward(x, off, m.conv_offset.weight, c.weight, dy, True, True, True, True, True, ws)
    dcn.check_status()
    with torch.backends.cudnn.flags(enabled=True, allow_tf32=False):
        off_ref = torch.nn.functional.conv2d(x, m.conv_offset.weight, m.conv_offset.bias, stride=c.stride, padding=c.padding)
    assert _rel(off, off_ref) <= TOL_BF16
    assert _rel(y, op.forward(x, off, c.weight, c.bias)) <= 1e-6
    dx_m, doff, dw2, db2 = op.backward(x, off, c.weight, dy, True, True, True, True)
    opq = dcn.Op(x, m.conv_offset.weight, c.stride, c.padding, 1, x.size(1), 1, deformable=False, std_size_rule=True,
                 precision="bf16")
    dx_q, _, dow2, dob2 = opq.backward(x, None, m.conv_offset.weight, doff, True, False, True, True)
    assert torch.equal(dw, dw2)                      # ordered split-K: bit for bit
    # dOffset is summed over the 8 channel slabs of a deformable group with floating-point atomics, so two runs differ
    # in its last bits; where such a value sits on a bf16 rounding boundary the packed operand of the plain
    # convolution's gradient kernels moves by one bf16 step (4e-3 of the term), hence the wider gates downstream of it
    assert _rel(db, db2) <= 1e-5 and _rel(dob, dob2) <= 1e-4
    assert _rel(dow, dow2) <= 1e-3
    assert _rel(dx, dx_m + dx_q) <= 1e-3
