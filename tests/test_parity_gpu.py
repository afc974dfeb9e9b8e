"""GPU parity: the CUDA path (through the public Functions, hence through the C ABI) against the CPU
oracle on identical seeded inputs.  Tolerances (max|a-b| / max|b| per tensor):
  exact fp32 path  <= 1e-4 against the float64 oracle (and against the fp32 oracle)
  exact fp64 path  <= 1e-10
  coordinates, validity, corner indices: bit-exact against the fp32 oracle.
"""
import ctypes

import numpy as np
import pytest
import torch

from oracle import oracle as orc
from tests import cases, helpers

pytestmark = pytest.mark.gpu

ALL = cases.REFERENCE_RECIPES + cases.CORNERS + cases.TC_CASES + [cases.BASELINE[1]]
TOL32, TOL64 = 1e-4, 1e-10


@pytest.mark.parametrize("case", ALL, ids=lambda c: c.name)
def test_exact_path_matches_oracle(case):
    tensors = cases.make_inputs(case)
    ours = helpers.run_ours(case, tensors, "exact")
    same = helpers.run_oracle(case, tensors)
    tol = TOL32 if case.dtype == "float32" else TOL64
    for k in same:
        assert ours[k].shape == same[k].shape, k
        assert cases.rel_err(ours[k], same[k]) <= tol, (k, cases.rel_err(ours[k], same[k]))
    if case.dtype == "float32":
        ref64 = helpers.run_oracle(case, tensors, np.float64)
        mask = helpers.lattice_mask(case, tensors[2].numpy()) if case.deformable else None
        for k in ref64:
            a, b = ours[k].astype(np.float64), ref64[k]
            if k == "doff":
                a, b = np.where(mask, 0, a), np.where(mask, 0, b)
            assert cases.rel_err(a, b) <= TOL32, (k, cases.rel_err(a, b))


@pytest.mark.parametrize("case", [c for c in ALL if c.deformable], ids=lambda c: c.name)
def test_coordinates_bit_exact(case):
    import deform_conv3d_pytorch_op_b200 as dcn
    x, w, off, dy, b = cases.make_inputs(case)
    op = dcn.Op(x.cuda(), w.cuda(), case.stride, case.pad, case.dil, case.cpg, case.G)
    p = case.problem()
    offd = off.cuda()
    for n in range(case.N):
        coords, valid, lo, hi = [t.cpu().numpy() for t in op.debug_points(offd, n)]
        rc, rv, rlo, rhi = orc.dump_points(p, np.ascontiguousarray(off[n].numpy()))
        it = np.uint32 if case.dtype == "float32" else np.uint64
        assert np.array_equal(coords.view(it), rc.view(it))          # coordinate bits
        assert np.array_equal(valid, rv)
        assert np.array_equal(lo, rlo) and np.array_equal(hi, rhi)


def test_zero_offsets_equal_plain_convolution():
    import deform_conv3d_pytorch_op_b200 as dcn
    g = torch.Generator().manual_seed(3)
    x = torch.randn(2, 8, 5, 9, 10, generator=g).cuda()
    w = torch.randn(12, 4, 3, 3, 3, generator=g).cuda()
    m = dcn.ConvOffset3d(8, 12, 3, stride=(1, 2, 1), padding=1, channel_per_group=4, groups=2, bias=True).cuda()
    with torch.no_grad():
        m.weight.copy_(w)
    off = torch.zeros(2, m.offset_channels, 5, 5, 10, device="cuda")
    y = m(x, off)
    ref = torch.nn.functional.conv3d(x, w, m.bias, stride=(1, 2, 1), padding=1, groups=2)
    assert cases.rel_err(y.detach().cpu().numpy(), ref.detach().cpu().numpy()) <= 1e-5


def test_plain_conv2d_matches_torch():
    import deform_conv3d_pytorch_op_b200 as dcn
    g = torch.Generator().manual_seed(4)
    x = torch.randn(3, 6, 13, 11, generator=g).cuda().requires_grad_(True)
    m = dcn.Conv2d(6, 9, 3, stride=2, padding=2, dilation=2, groups=3).cuda()
    y = m(x)
    ref = torch.nn.functional.conv2d(x, m.weight, m.bias, stride=2, padding=2, dilation=2, groups=3)
    assert y.shape == ref.shape
    dy = torch.randn_like(ref)
    gx, gw, gb = torch.autograd.grad(ref, [x, m.weight, m.bias], dy)
    hx, hw, hb = torch.autograd.grad(y, [x, m.weight, m.bias], dy)
    for a, b_ in ((y, ref), (hx, gx), (hw, gw), (hb, gb)):
        assert cases.rel_err(a.detach().cpu().numpy(), b_.detach().cpu().numpy()) <= 1e-5


def test_plain_conv3d_matches_torch():
    """The plain-convolution path over three spatial axes (conv2d/lib/conv2d_cuda.cpp:77-290 generalised): the
    torch fp32 convolution is the reference for this floating-point kernel; fp32 gate 1e-5."""
    import deform_conv3d_pytorch_op_b200 as dcn
    g = torch.Generator().manual_seed(5)
    x = torch.randn(2, 6, 7, 9, 8, generator=g).cuda().requires_grad_(True)
    m = dcn.Conv3d(6, 8, (3, 3, 2), stride=(1, 2, 1), padding=(1, 2, 0), dilation=(2, 1, 1), groups=2).cuda()
    y = m(x)
    with torch.backends.cudnn.flags(enabled=True, allow_tf32=False):
        ref = torch.nn.functional.conv3d(x, m.weight, m.bias, stride=(1, 2, 1), padding=(1, 2, 0), dilation=(2, 1, 1),
                                         groups=2)
        assert y.shape == ref.shape
        dy = torch.randn_like(ref)
        gx, gw, gb = torch.autograd.grad(ref, [x, m.weight, m.bias], dy)
    hx, hw, hb = torch.autograd.grad(y, [x, m.weight, m.bias], dy)
    for a, b_ in ((y, ref), (hx, gx), (hw, gw), (hb, gb)):
        assert cases.rel_err(a.detach().cpu().numpy(), b_.detach().cpu().numpy()) <= 1e-5


def test_fp64_gradcheck_like_the_reference():
    """deform2d_double/test_gradient.py:7-53 with torch's gradcheck (pull-back term off: it is not a derivative)."""
    import deform_conv3d_pytorch_op_b200 as dcn
    c = [k for k in cases.REFERENCE_RECIPES if k.name == "d2d_test_gradient"][0]
    x, w, off, dy, b = [t.cuda().requires_grad_(True) for t in cases.make_inputs(c)]
    fn = lambda x_, o_, w_, b_: dcn.ConvOffset2dFunction.apply(x_, o_, w_, b_, c.stride, c.pad, c.dil, c.cpg, c.G)
    assert torch.autograd.gradcheck(fn, (x, off, w, b), eps=1e-6, atol=1e-5, rtol=1e-3, nondet_tol=1e-9)


def test_legacy_ffi_surface_3d():
    """deform3d/test_function.py:36-56 style direct calls with caller-allocated, zero-filled buffers."""
    import deform_conv3d_pytorch_op_b200 as dcn
    c = cases.REFERENCE_RECIPES[0]
    x, w, off, dy, _ = [None if t is None else t.cuda() for t in cases.make_inputs(c)]
    p = c.problem()
    out = torch.zeros((c.N, c.O) + p.out_size, device="cuda")
    columns = torch.zeros(c.C * p.kv, p.ov, device="cuda")
    op = dcn.deform_conv3d_op
    assert op.deform_conv_forward_cuda(x, w, off, columns, out, *c.pad, *c.stride, *c.dil, c.cpg, c.G) == 1
    gi, go, gw = torch.zeros_like(x), torch.zeros_like(off), torch.zeros_like(w)
    assert op.deform_conv_backward_input_offset_cuda(x, w, off, dy, columns, gi, go, *c.pad, *c.stride, *c.dil,
                                                     c.cpg, c.G) == 1
    assert op.deform_conv_backward_weight_cuda(x, off, dy, columns, gw, *c.pad, *c.stride, *c.dil, c.cpg, c.G) == 1
    ref = helpers.run_oracle(c, cases.make_inputs(c))
    for a, k in ((out, "y"), (gi, "dx"), (go, "doff"), (gw, "dw")):
        assert cases.rel_err(a.cpu().numpy(), ref[k]) <= TOL32, k


def test_legacy_ffi_surface_2d_and_conv():
    import deform_conv3d_pytorch_op_b200 as dcn
    table = {c.name: c for c in cases.REFERENCE_RECIPES}
    # fp32 2-D (no dilation / group arguments)
    c = table["d2_test_gradient"]
    x, w, off, dy, _ = [None if t is None else t.cuda() for t in cases.make_inputs(c)]
    p = c.problem()
    out = torch.zeros((c.N, c.O) + p.out_size, device="cuda")
    gi, go, gw = torch.zeros_like(x), torch.zeros_like(off), torch.zeros_like(w)
    op = dcn.deform_conv2d_op
    assert op.deform_conv_forward_cuda(x, w, off, None, out, *c.pad, *c.stride, c.cpg) == 1
    assert op.deform_conv_backward_input_offset_cuda(x, w, off, dy, None, gi, go, *c.pad, *c.stride, c.cpg) == 1
    assert op.deform_conv_backward_weight_cuda(x, off, dy, None, gw, *c.pad, *c.stride, c.cpg) == 1
    ref = helpers.run_oracle(c, cases.make_inputs(c))
    for a, k in ((out, "y"), (gi, "dx"), (go, "doff"), (gw, "dw")):
        assert cases.rel_err(a.cpu().numpy(), ref[k]) <= TOL32, k
    # fp64 2-D
    c = table["d2d_test_gradient"]
    tens = cases.make_inputs(c)
    x, w, off, dy, b = [None if t is None else t.cuda() for t in tens]
    p = c.problem()
    out = torch.zeros((c.N, c.O) + p.out_size, device="cuda", dtype=torch.float64)
    gi, go, gw = torch.zeros_like(x), torch.zeros_like(off), torch.zeros_like(w)
    op = dcn.deform_conv2d_double_op
    assert op.deform_conv_forward_cuda(x, w, off, None, out, *c.pad, *c.stride, *c.dil, c.cpg, c.G) == 1
    assert op.deform_conv_backward_input_offset_cuda(x, w, off, dy, None, gi, go, *c.pad, *c.stride, *c.dil, c.cpg,
                                                     c.G) == 1
    assert op.deform_conv_backward_weight_cuda(x, off, dy, None, gw, *c.pad, *c.stride, *c.dil, c.cpg, c.G) == 1
    ref = helpers.run_oracle(c, (tens[0], tens[1], tens[2], tens[3], None))
    for a, k in ((out, "y"), (gi, "dx"), (go, "doff"), (gw, "dw")):
        assert cases.rel_err(a.cpu().numpy(), ref[k]) <= TOL64, k
    # plain conv2d
    c = table["c2_test_gradient"]
    tens = cases.make_inputs(c)
    x, w, _, dy, b = [None if t is None else t.cuda() for t in tens]
    p = c.problem()
    out = torch.zeros((c.N, c.O) + p.out_size, device="cuda")
    gi, gw = torch.zeros_like(x), torch.zeros_like(w)
    op = dcn.conv2d_op
    assert op.conv_forward_cuda(x, w, None, out, *c.pad, *c.stride, *c.dil, c.G) == 1
    assert op.conv_backward_input_cuda(w, dy, None, gi, *c.pad, *c.stride, *c.dil, c.G) == 1
    assert op.conv_backward_weight_cuda(x, dy, None, gw, *c.pad, *c.stride, *c.dil, c.G) == 1
    ref = helpers.run_oracle(c, (tens[0], tens[1], None, tens[3], None))
    for a, k in ((out, "y"), (gi, "dx"), (gw, "dw")):
        assert cases.rel_err(a.cpu().numpy(), ref[k]) <= TOL32, k


def test_errors_are_loud():
    import deform_conv3d_pytorch_op_b200 as dcn
    x = torch.randn(1, 4, 6, 6, device="cuda")
    w = torch.randn(4, 4, 3, 3, device="cuda")
    bad_off = torch.zeros(1, 18, 5, 5, device="cuda")       # wrong spatial size
    with pytest.raises(dcn.DcnError):
        dcn.ConvOffset2dFunction.apply(x, bad_off, w, None, (1, 1), (1, 1), (1, 1), 4, 1)
    with pytest.raises(dcn.DcnError):                        # input c != kernel c
        dcn.ConvOffset2dFunction.apply(x, bad_off, torch.randn(4, 3, 3, 3, device="cuda"), None, (1, 1), (1, 1),
                                       (1, 1), 4, 1)
    with pytest.raises(dcn.DcnError):                        # CPU tensors are refused: no CPU implementation
        dcn.ConvOffset2dFunction.apply(x.cpu(), torch.zeros(1, 18, 6, 6), w.cpu(), None, (1, 1), (1, 1), (1, 1), 4, 1)
    with pytest.raises(dcn.DcnError):                        # bf16 tensor-core path needs channel multiples of 8
        dcn.ConvOffset2dFunction.apply(x, torch.zeros(1, 18, 6, 6, device="cuda"), w, None, (1, 1), (1, 1), (1, 1),
                                       4, 1, "bf16")
