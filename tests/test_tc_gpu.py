"""GPU parity of the bf16 tensor-core path (tcgen05): against the float64 oracle and against the exact fp32
CUDA path, on shapes whose channel counts allow it.  Gate: max|a-b| / max|b| <= 2e-2 per tensor."""
import numpy as np
import pytest
import torch

from tests import cases, helpers

pytestmark = pytest.mark.gpu
TOL_BF16 = 2e-2


def _check_status():
    from deform_conv3d_pytorch_op_b200 import _lib
    _lib.check(_lib.lib().dcn_check_status(_lib.current_stream(torch.device("cuda"))), "device status")


@pytest.mark.parametrize("case", cases.TC_CASES + [cases.BASELINE[1]], ids=lambda c: c.name)
def test_bf16_path_matches_oracle(case):
    tensors = cases.make_inputs(case)
    ours = helpers.run_ours(case, tensors, "bf16")
    _check_status()
    ref64 = helpers.run_oracle(case, tensors, np.float64)
    exact = helpers.run_ours(case, tensors, "exact")
    mask = helpers.lattice_mask(case, tensors[2].numpy())
    for k in ref64:
        a, b, e = ours[k].astype(np.float64), ref64[k], exact[k].astype(np.float64)
        if k == "doff":
            a, b, e = np.where(mask, 0, a), np.where(mask, 0, b), np.where(mask, 0, e)
        assert cases.rel_err(a, b) <= TOL_BF16, (k, "vs float64 oracle", cases.rel_err(a, b))
        assert cases.rel_err(a, e) <= TOL_BF16, (k, "vs exact fp32 path", cases.rel_err(a, e))


def test_bf16_plain_conv2d():
    import deform_conv3d_pytorch_op_b200 as dcn
    g = torch.Generator().manual_seed(7)
    x = torch.randn(2, 32, 17, 13, generator=g).cuda().requires_grad_(True)
    m = dcn.Conv2d(32, 24, 3, stride=1, padding=1, dilation=1, groups=2, precision="bf16").cuda()
    y = m(x)
    ref = torch.nn.functional.conv2d(x, m.weight, m.bias, stride=1, padding=1, groups=2)
    _check_status()
    assert cases.rel_err(y.detach().cpu().numpy(), ref.detach().cpu().numpy()) <= TOL_BF16
    dy = torch.randn_like(ref)
    gx, gw = torch.autograd.grad(ref, [x, m.weight], dy)
    hx, hw = torch.autograd.grad(y, [x, m.weight], dy)
    _check_status()
    assert cases.rel_err(hx.cpu().numpy(), gx.cpu().numpy()) <= TOL_BF16
    assert cases.rel_err(hw.cpu().numpy(), gw.cpu().numpy()) <= TOL_BF16


def test_bf16_is_deterministic_in_forward():
    case = cases.TC_CASES[0]
    tensors = cases.make_inputs(case)
    a = helpers.run_ours(case, tensors, "bf16")["y"]
    b = helpers.run_ours(case, tensors, "bf16")["y"]
    assert np.array_equal(a, b)


@pytest.mark.parametrize("name", ["tc2_dg_groups", "tc3_groups", "tc2_c256"])
def test_separate_bf16_passes_match_fused_backward(name):
    """dcn_backward_data / dcn_backward_weight (accumulate into zeroed buffers) against dcn_backward (overwrite,
    shared scratch, forward's channels-last copy taken over)."""
    import deform_conv3d_pytorch_op_b200 as dcn
    case = {c.name: c for c in cases.TC_CASES}[name]
    x, w, off, dy, b = [None if t is None else t.cuda() for t in cases.make_inputs(case)]
    op = dcn.Op(x, w, case.stride, case.pad, case.dil, case.cpg, case.G, precision="bf16")
    y, fws = op.forward(x, off, w, b, keep_workspace=True)
    dx_f, doff_f, dw_f, db_f = op.backward(x, off, w, dy, True, True, True, True, fws)
    dx_s, doff_s = op.backward_data(x, off, w, dy)
    dw_s, db_s = op.backward_weight(x, off, dy, True, True)
    dx_n, doff_n, dw_n, _ = op.backward(x, off, w, dy, True, True, True, False, None)     # rebuilds the copy itself
    _check_status()
    for a, r in ((dx_f, dx_s), (doff_f, doff_s), (dw_f, dw_s), (db_f, db_s), (dx_n, dx_s), (dw_n, dw_s)):
        assert cases.rel_err(a.cpu().numpy(), r.cpu().numpy()) <= 1e-3
