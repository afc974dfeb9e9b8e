"""BASELINE configurations 2-4 at their full sizes on the GPU:

* bf16 tensor-core path: EVERY sample of y, dX and dOffset and the whole-batch dW against the float64 oracle
  (max|a-b| / max|b| <= 2e-2 per tensor), plus batch additivity of dW as a size-independent property;
* exact path: one full-size sample of each configuration against the float64 oracle (<= 1e-4);
* zero offsets reproduce torch's ordinary convolution where the two size rules agree (dilation 1);
* forward is linear in the weight.
The oracle restates deform3d/lib/deform_conv3d_cuda.cpp:105-158, 186-253 and 278-330 (dW summed over the whole
batch) on the host; the offset gradient leaves out points within 1e-6 of the integer lattice, where the derivative
is one-sided and fp32 / fp64 coordinates may pick different sides."""
import dataclasses

import numpy as np
import pytest
import torch

from oracle import oracle as orc
from tests import cases, helpers

pytestmark = pytest.mark.gpu
TOL = 2e-2
TOL_EXACT = 1e-4


def _op(case, x, w, precision):
    import deform_conv3d_pytorch_op_b200 as dcn
    return dcn.Op(x, w, case.stride, case.pad, case.dil, case.cpg, case.G, precision=precision)


def _status():
    from deform_conv3d_pytorch_op_b200 import _lib
    _lib.check(_lib.lib().dcn_check_status(_lib.current_stream(torch.device("cuda"))), "device status")


def _oracle64(case, x, w, off, dy):
    """The float64 oracle at the coordinates the reference's fp32 arithmetic produces (see
    helpers.offsets_at_fp32_coordinates): among the 10^8 sampling points of a full-size configuration a few round
    onto the validity boundary, where the operator is discontinuous."""
    p = case.problem()
    p.N = x.shape[0]
    x64, w64, dy64 = [t.numpy().astype(np.float64) for t in (x, w, dy)]
    o64 = helpers.offsets_at_fp32_coordinates(case, off.numpy())
    y = orc.forward(p, x64, o64, w64)
    dx, doff = orc.backward_data(p, x64, o64, w64, dy64)
    dw = orc.backward_weight(p, x64, o64, dy64)
    return y, dx, doff, dw


def _compare(case, off, got, ref, tol):
    y, dx, doff, dw = [t.cpu().numpy() for t in got]
    y_ref, dx_ref, doff_ref, dw_ref = ref
    errs = {"y": cases.rel_err(y, y_ref), "dx": cases.rel_err(dx, dx_ref), "dw": cases.rel_err(dw, dw_ref)}
    mask = helpers.lattice_mask(case, off.numpy())
    errs["doff"] = cases.rel_err(np.where(mask, 0, doff.astype(np.float64)), np.where(mask, 0, doff_ref))
    for k, e in errs.items():
        assert e <= tol, (case.name, k, e)
    return errs


@pytest.mark.parametrize("cfg", [2, 3, 4])
def test_full_size_every_sample_against_float64_oracle(cfg):
    case = cases.BASELINE[cfg]
    x, w, off, dy, _ = cases.make_inputs(case)
    xd, wd, od, dyd = x.cuda(), w.cuda(), off.cuda(), dy.cuda()
    op = _op(case, xd, wd, "bf16")
    y, fws = op.forward(xd, od, wd, None, keep_workspace=True)
    dx, doff, dw, _ = op.backward(xd, od, wd, dyd, True, True, True, False, fws)
    torch.cuda.synchronize()
    _status()
    assert all(bool(torch.isfinite(t).all()) for t in (y, dx, doff, dw))
    ref = _oracle64(case, x, w, off, dy)
    _compare(case, off, (y, dx, doff, dw), ref, TOL)
    # the separate entry points (accumulating semantics) give the same tensors
    dx_s, doff_s = op.backward_data(xd, od, wd, dyd)
    dw_s, _ = op.backward_weight(xd, od, dyd)
    _status()
    _compare(case, off, (y, dx_s, doff_s, dw_s), ref, TOL)

    # size-independent property: the weight gradient is additive over the batch
    h = case.N // 2
    parts = []
    for lo, hi in ((0, h), (h, case.N)):
        xs, os_, dys = xd[lo:hi].contiguous(), od[lo:hi].contiguous(), dyd[lo:hi].contiguous()
        ops = _op(case, xs, wd, "bf16")
        parts.append(ops.backward(xs, os_, wd, dys, False, False, True, False, None)[2])
    assert cases.rel_err(dw.cpu().numpy(), (parts[0] + parts[1]).cpu().numpy()) <= 2e-3


@pytest.mark.parametrize("cfg,n", [(2, 1), (3, 1), (4, 2)])
def test_exact_path_full_size_samples_against_float64_oracle(cfg, n):
    """The exact fp32 path (the <= 1e-4 gate; configuration 4 is stated fp32) on full-size samples."""
    case = dataclasses.replace(cases.BASELINE[cfg], N=n)
    x, w, off, dy, _ = cases.make_inputs(case)
    xd, wd, od, dyd = x.cuda(), w.cuda(), off.cuda(), dy.cuda()
    op = _op(case, xd, wd, "exact")
    y = op.forward(xd, od, wd, None)
    dx, doff, dw, _ = op.backward(xd, od, wd, dyd)
    torch.cuda.synchronize()
    _compare(case, off, (y, dx, doff, dw), _oracle64(case, x, w, off, dy), TOL_EXACT)


@pytest.mark.parametrize("cfg", [2, 3])
def test_full_size_zero_offsets_equal_torch_convolution(cfg):
    case = cases.BASELINE[cfg]
    x, w, off, dy, _ = cases.make_inputs(case)
    xd, wd = x.cuda(), w.cuda()
    od = torch.zeros_like(off).cuda()
    y = _op(case, xd, wd, "bf16").forward(xd, od, wd, None)
    conv = torch.nn.functional.conv3d if case.ndim == 3 else torch.nn.functional.conv2d
    ref = conv(xd, wd, None, stride=case.stride, padding=case.pad, groups=case.G)
    assert y.shape == ref.shape
    assert cases.rel_err(y.cpu().numpy(), ref.cpu().numpy()) <= TOL


def test_full_size_forward_is_linear_in_the_weight():
    case = cases.BASELINE[2]
    x, w, off, dy, _ = cases.make_inputs(case)
    xd, od = x.cuda(), off.cuda()
    g = torch.Generator().manual_seed(9)
    w2 = torch.randn(w.shape, generator=g) * w.std()
    wa, wb = w.cuda(), w2.cuda()
    op = _op(case, xd, wa, "bf16")
    ya, yb = op.forward(xd, od, wa, None), op.forward(xd, od, wb, None)
    yc = op.forward(xd, od, 0.5 * wa - 2.0 * wb, None)
    assert cases.rel_err(yc.cpu().numpy(), (0.5 * ya - 2.0 * yb).cpu().numpy()) <= TOL
