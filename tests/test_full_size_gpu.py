"""BASELINE configurations 2-4 at their full sizes on the GPU (bf16 tensor-core path and, for one sample, the
exact path), checked through size-independent properties and against the oracle on one sample:

* per-sample quantities (y, dX, dOffset) of the LAST sample of the full batch equal the oracle run on that sample
  alone (the samples are independent; this also exercises tiles that straddle sample boundaries);
* the weight gradient is additive over the batch: dW(full) = dW(first half) + dW(second half);
* zero offsets reproduce torch's ordinary convolution where the two size rules agree (dilation 1);
* forward is linear in the weight.
Tolerance of the bf16 path: max|a-b| / max|b| <= 2e-2."""
import numpy as np
import pytest
import torch

from oracle import oracle as orc
from tests import cases

pytestmark = pytest.mark.gpu
TOL = 2e-2


def _op(case, x, w, precision):
    import deform_conv3d_pytorch_op_b200 as dcn
    return dcn.Op(x, w, case.stride, case.pad, case.dil, case.cpg, case.G, precision=precision)


@pytest.mark.parametrize("cfg", [2, 3, 4])
def test_full_size_against_oracle_on_one_sample_and_batch_additivity(cfg):
    case = cases.BASELINE[cfg]
    x, w, off, dy, _ = cases.make_inputs(case)
    xd, wd, od, dyd = x.cuda(), w.cuda(), off.cuda(), dy.cuda()
    op = _op(case, xd, wd, "bf16")
    y, fws = op.forward(xd, od, wd, None, keep_workspace=True)
    dx, doff, dw, _ = op.backward(xd, od, wd, dyd, True, True, True, False, fws)
    torch.cuda.synchronize()
    from deform_conv3d_pytorch_op_b200 import _lib
    _lib.check(_lib.lib().dcn_check_status(_lib.current_stream(xd.device)), "device status")
    assert all(bool(torch.isfinite(t).all()) for t in (y, dx, doff, dw))

    # (1) last sample against the float64 oracle on that sample alone
    n = case.N - 1
    p = case.problem()
    p.N = 1
    sl = slice(n, n + 1)
    x1, o1, dy1 = [t[sl].numpy().astype(np.float64) for t in (x, off, dy)]
    w64 = w.numpy().astype(np.float64)
    y_ref = orc.forward(p, x1, o1, w64)
    dx_ref, doff_ref = orc.backward_data(p, x1, o1, w64, dy1)
    assert cases.rel_err(y[sl].cpu().numpy(), y_ref) <= TOL
    assert cases.rel_err(dx[sl].cpu().numpy(), dx_ref) <= TOL
    # offset gradient: leave out points on the integer lattice (one-sided derivative, fp32 vs fp64 coordinates)
    from tests import helpers
    mask = helpers.lattice_mask(case, off[sl].numpy())
    a = np.where(mask, 0, doff[sl].cpu().numpy().astype(np.float64))
    b = np.where(mask, 0, doff_ref)
    assert cases.rel_err(a, b) <= TOL

    # (2) weight gradient is additive over the batch
    h = case.N // 2
    parts = []
    for lo, hi in ((0, h), (h, case.N)):
        xs, os_, dys = xd[lo:hi].contiguous(), od[lo:hi].contiguous(), dyd[lo:hi].contiguous()
        ops = _op(case, xs, wd, "bf16")
        parts.append(ops.backward(xs, os_, wd, dys, False, False, True, False, None)[2])
    assert cases.rel_err(dw.cpu().numpy(), (parts[0] + parts[1]).cpu().numpy()) <= 2e-3


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


def test_exact_path_full_size_sample_matches_fp32_oracle():
    """The exact fp32 path on one full-size sample of configuration 2 against the fp32 oracle (<= 1e-4)."""
    import dataclasses
    case = dataclasses.replace(cases.BASELINE[2], N=1)
    x, w, off, dy, _ = cases.make_inputs(case)
    xd, wd, od, dyd = x.cuda(), w.cuda(), off.cuda(), dy.cuda()
    op = _op(case, xd, wd, "exact")
    y = op.forward(xd, od, wd, None)
    dx, doff, dw, _ = op.backward(xd, od, wd, dyd)
    p = case.problem()
    xn, wn, on, dyn = x.numpy(), w.numpy(), off.numpy(), dy.numpy()
    assert cases.rel_err(y.cpu().numpy(), orc.forward(p, xn, on, wn)) <= 1e-4
    dx_ref, doff_ref = orc.backward_data(p, xn, on, wn, dyn)
    assert cases.rel_err(dx.cpu().numpy(), dx_ref) <= 1e-4
    assert cases.rel_err(doff.cpu().numpy(), doff_ref) <= 1e-4
    assert cases.rel_err(dw.cpu().numpy(), orc.backward_weight(p, xn, on, dyn)) <= 1e-4
