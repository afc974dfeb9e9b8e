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


def test_bf16_plain_conv3d():
    """Plain 3-D convolution on the tcgen05 kernels (DEFORM = false instantiations); bf16 gate 2e-2 against torch
    fp32."""
    import deform_conv3d_pytorch_op_b200 as dcn
    g = torch.Generator().manual_seed(8)
    x = torch.randn(2, 32, 6, 11, 9, generator=g).cuda().requires_grad_(True)
    m = dcn.Conv3d(32, 40, 3, stride=(1, 2, 2), padding=1, dilation=1, groups=1, precision="bf16").cuda()
    y = m(x)
    with torch.backends.cudnn.flags(enabled=True, allow_tf32=False):
        ref = torch.nn.functional.conv3d(x, m.weight, m.bias, stride=(1, 2, 2), padding=1)
        dy = torch.randn_like(ref)
        gx, gw = torch.autograd.grad(ref, [x, m.weight], dy)
    _check_status()
    assert cases.rel_err(y.detach().cpu().numpy(), ref.detach().cpu().numpy()) <= TOL_BF16
    hx, hw = torch.autograd.grad(y, [x, m.weight], dy)
    _check_status()
    assert cases.rel_err(hx.cpu().numpy(), gx.cpu().numpy()) <= TOL_BF16
    assert cases.rel_err(hw.cpu().numpy(), gw.cpu().numpy()) <= TOL_BF16


@pytest.mark.parametrize("ndim,channels_last", [(2, False), (3, False), (3, True)])
def test_bf16_plain_conv_stride1_input_gradient_as_gather(ndim, channels_last):
    """Stride-1 plain convolution: the input gradient runs on the forward kernel as a convolution of dy with
    mirrored taps and transposed weights (conv2d/lib/conv2d_cuda.cpp:184-191 + col2im in the reference).  Dilation,
    groups, rectangular kernel and non-square padding; through the fused (overwriting) and the accumulating entry."""
    import deform_conv3d_pytorch_op_b200 as dcn
    g = torch.Generator().manual_seed(12)
    size = (13, 11) if ndim == 2 else (5, 9, 8)
    k = (3, 2) if ndim == 2 else (2, 3, 3)
    pad = (2, 1) if ndim == 2 else (1, 2, 0)
    dil = (2, 1) if ndim == 2 else (1, 2, 1)
    x = torch.randn((2, 32) + size, generator=g).cuda()
    if channels_last:
        x = x.contiguous(memory_format=torch.channels_last_3d)
    w = (torch.randn((48, 16) + k, generator=g) * 0.1).cuda()
    conv = torch.nn.functional.conv3d if ndim == 3 else torch.nn.functional.conv2d
    xr, wr = x.detach().clone().requires_grad_(True), w.clone().requires_grad_(True)
    with torch.backends.cudnn.flags(enabled=True, allow_tf32=False):
        ref = conv(xr, wr, None, stride=1, padding=pad, dilation=dil, groups=2)
        dy = torch.randn_like(ref)
        gx, gw = torch.autograd.grad(ref, [xr, wr], dy)
    op = dcn.Op(x, w, 1, pad, dil, 32, 2, deformable=False, std_size_rule=True, precision="bf16")
    assert op.channels_last == channels_last
    dx, _, dw, _ = op.backward(x, None, w, dy, True, False, True, False)
    _check_status()
    assert cases.rel_err(dx.cpu().numpy(), gx.cpu().numpy()) <= TOL_BF16
    assert cases.rel_err(dw.cpu().numpy(), gw.cpu().numpy()) <= TOL_BF16
    dx2, _ = op.backward_data(x, None, w, dy)              # accumulates into a zeroed buffer
    _check_status()
    assert cases.rel_err(dx2.cpu().numpy(), dx.cpu().numpy()) <= 1e-6


def test_bf16_is_deterministic_in_forward():
    case = cases.TC_CASES[0]
    tensors = cases.make_inputs(case)
    a = helpers.run_ours(case, tensors, "bf16")["y"]
    b = helpers.run_ours(case, tensors, "bf16")["y"]
    assert np.array_equal(a, b)


@pytest.mark.parametrize("name", ["tc2_c256", "tc3_groups"])
def test_bf16_weight_gradient_is_deterministic(name):
    """The position splits of the weight gradient are stored in slices and added in split order (the reference
    accumulates over the batch in a fixed order too: beta = 1 GEMMs in its sample loop,
    deform3d/lib/deform_conv3d_cuda.cpp:278-330): two runs give the same bits."""
    case = [c for c in cases.TC_CASES if c.name == name][0]
    tensors = cases.make_inputs(case)
    a = helpers.run_ours(case, tensors, "bf16")["dw"]
    b = helpers.run_ours(case, tensors, "bf16")["dw"]
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


@pytest.mark.parametrize("name", ["tc2_small", "tc2_dg_groups", "tc2_cpg16_tiles", "tc2_c128_tail", "tc3_small", "tc3_groups",
                                  "tc3_o512"])
def test_channels_last_io_matches_reference_layout(name):
    """Channels-last activations (torch.channels_last / channels_last_3d storage) in and out of the bf16 path:
    same arithmetic as the reference layout, no layout pass, results returned channels-last."""
    import deform_conv3d_pytorch_op_b200 as dcn
    case = {c.name: c for c in cases.TC_CASES}[name]
    mf = torch.channels_last if case.ndim == 2 else torch.channels_last_3d
    x, w, off, dy, b = [None if t is None else t.cuda() for t in cases.make_inputs(case)]
    ref = dcn.Op(x, w, case.stride, case.pad, case.dil, case.cpg, case.G, precision="bf16")
    assert not ref.channels_last
    y_r = ref.forward(x, off, w, b)
    dx_r, doff_r, dw_r, db_r = ref.backward(x, off, w, dy, True, True, True, True, None)
    x_cl, dy_cl = x.contiguous(memory_format=mf), dy.contiguous(memory_format=mf)
    op = dcn.Op(x_cl, w, case.stride, case.pad, case.dil, case.cpg, case.G, precision="bf16")
    assert op.channels_last == (not x_cl.is_contiguous())
    y_c, fws = op.forward(x_cl, off, w, b, keep_workspace=True)
    dx_c, doff_c, dw_c, db_c = op.backward(x_cl, off, w, dy_cl, True, True, True, True, fws)
    dx_s, doff_s = op.backward_data(x_cl, off, w, dy_cl)
    dw_s, db_s = op.backward_weight(x_cl, off, dy_cl, True, True)
    _check_status()
    if op.channels_last:
        assert y_c.is_contiguous(memory_format=mf) and dx_c.is_contiguous(memory_format=mf)
    assert y_c.shape == y_r.shape and dx_c.shape == dx_r.shape
    # the forward arithmetic is identical (same bf16 operands, same accumulation order inside a tile)
    assert cases.rel_err(y_c.cpu().numpy(), y_r.cpu().numpy()) <= 1e-5
    for a, r in ((dx_c, dx_r), (doff_c, doff_r), (dw_c, dw_r), (db_c, db_r), (dx_s, dx_r), (doff_s, doff_r),
                 (dw_s, dw_r), (db_s, db_r)):
        assert cases.rel_err(a.cpu().numpy(), r.cpu().numpy()) <= 1e-3


def test_channels_last_needs_the_bf16_path():
    import deform_conv3d_pytorch_op_b200 as dcn
    from deform_conv3d_pytorch_op_b200 import _lib
    import ctypes
    p = _lib.make_problem(2, torch.float32, 2, 16, 16, (8, 8), (3, 3), 1, 1, 1, 1, 16, precision=_lib.PREC_EXACT,
                          channels_last=True)
    assert _lib.lib().dcn_validate(ctypes.byref(p)) == -3
    # the tensor-level wrapper keeps the exact path on the reference layout and converts
    x = torch.randn(2, 16, 8, 8).cuda().contiguous(memory_format=torch.channels_last)
    w = torch.randn(16, 16, 3, 3).cuda()
    off = torch.zeros(2, 18, 8, 8).cuda()
    op = dcn.Op(x, w, 1, 1, 1, 16, 1, precision="exact")
    assert not op.channels_last
    y = op.forward(x, off, w, None)
    ref = torch.nn.functional.conv2d(x.cpu().double(), w.cpu().double(), None, padding=1)      # zero offsets
    assert cases.rel_err(y.cpu().numpy(), ref.numpy()) <= 1e-4


# ---- shared-memory-accumulating backward-data kernel of the 2-D deformable operator ---------------------------
_B2_CASES = ["tc2_small", "tc2_dg_groups", "tc2_c256", "tc2_stride_dil", "tc2_cpg16_tiles", "tc2_c128_tail"]


@pytest.mark.parametrize("name", _B2_CASES + ["cfg1", "cfg2_sample"])
def test_tensor_core_point_entries_bit_exact(name):
    """The sampling-point entries that the tensor-core backward-data kernel consumes (located by its own pre-pass:
    validity, low / high corner, fractions) against the fp32 oracle: corner indices and validity equal, and the
    coordinate rebuilt from the entry (low corner + fraction, exact) equal bit for bit."""
    import dataclasses
    import deform_conv3d_pytorch_op_b200 as dcn
    from oracle import oracle as orc
    if name == "cfg1":
        case = cases.BASELINE[1]
    elif name == "cfg2_sample":
        case = dataclasses.replace(cases.BASELINE[2], N=2)
    else:
        case = {c.name: c for c in cases.TC_CASES}[name]
    x, w, off, dy, b = cases.make_inputs(case)
    op = dcn.Op(x.cuda(), w.cuda(), case.stride, case.pad, case.dil, case.cpg, case.G, precision="bf16")
    p = case.problem()
    offd = off.cuda()
    for n in range(case.N):
        coords, valid, lo, hi = [t.cpu().numpy() for t in op.debug_tc_points(offd, n)]
        rc, rv, rlo, rhi = orc.dump_points(p, np.ascontiguousarray(off[n].numpy()))
        assert np.array_equal(valid, rv)                 # also: no entry with inconsistent encodings (-1)
        ok = rv != 0
        assert np.array_equal(lo[ok], rlo[ok]) and np.array_equal(hi[ok], rhi[ok])
        assert np.array_equal(coords[ok].view(np.uint32), rc[ok].view(np.uint32))
        assert (lo[~ok] == -1).all() and (hi[~ok] == -1).all()
    _check_status()


def test_fixed_point_plane_budget_and_early_spill():
    """Worst case for the fixed-point dX plane: constant dy and weight (every col value sits at the bound the scale
    is chosen from) and offsets that send EVERY sample of EVERY tap to the same input pixel.  The magnitude budget
    runs out, the kernel switches to additions that look at the element they found, and the element crosses 2^30
    and is flushed to dX early -- the result must still be the oracle's."""
    import deform_conv3d_pytorch_op_b200 as dcn
    from oracle import oracle as orc
    # one term is 2^18 fixed-point steps here (scale 2^13 x col 32 x weight 1): 24 * 24 * 9 = 5184 of them on one
    # element pass 2^30, and the budget (2^30 over all elements) is spent after an eighth of the sample
    N, C, O, H, W = 1, 8, 32, 24, 24
    case = cases.Case("b2_spill", 2, N, C, O, (H, W), (3, 3), (1, 1), (1, 1), (1, 1), 1, 8)
    p = case.problem()
    x = torch.rand(N, C, H, W) * 2 - 1
    w = torch.ones(O, C, 3, 3)
    dy = torch.ones(N, O, H, W)
    off = torch.zeros(N, 18, H, W)
    th, tw = 5.0, 9.0
    hh, ww = torch.meshgrid(torch.arange(H, dtype=torch.float32), torch.arange(W, dtype=torch.float32), indexing="ij")
    for tap in range(9):
        kh, kw = tap // 3, tap % 3
        off[0, tap * 2] = th - (hh - 1 + kh)
        off[0, tap * 2 + 1] = tw - (ww - 1 + kw)
    xd, wd, od, dyd = x.cuda(), w.cuda(), off.cuda(), dy.cuda()
    op = dcn.Op(xd, wd, case.stride, case.pad, case.dil, case.cpg, case.G, precision="bf16")
    dx, doff, dw, _ = op.backward(xd, od, wd, dyd, True, True, True, False, None)
    dx_s, _ = op.backward_data(xd, od, wd, dyd)
    _check_status()
    dx_ref, _ = orc.backward_data(p, x.numpy().astype(np.float64), off.numpy().astype(np.float64),
                                  w.numpy().astype(np.float64), dy.numpy().astype(np.float64))
    assert dx_ref[0, 0, 5, 9] == H * W * 9 * O          # all 5184 samples of a channel land on one pixel
    assert cases.rel_err(dx.cpu().numpy(), dx_ref) <= 1e-5
    assert cases.rel_err(dx_s.cpu().numpy(), dx_ref) <= 1e-5


def test_bounded_wait_gives_up_and_reports_timeout():
    """A device-side wait that cannot complete (a barrier nothing arrives on) runs into its limit: the kernel
    returns, the status word reports DCN_ERR_TIMEOUT once, and the library keeps working afterwards."""
    from deform_conv3d_pytorch_op_b200 import _lib
    L = _lib.lib()
    dev = torch.device("cuda")
    st = _lib.current_stream(dev)
    assert L.dcn_check_status(st) == 0
    flag = torch.zeros(1, dtype=torch.int32, device=dev)
    assert L.dcn_debug_expire_wait(_lib.ptr(flag), st) == 0
    assert L.dcn_check_status(st) == -6                  # DCN_ERR_TIMEOUT
    assert int(flag.item()) == 1
    assert L.dcn_check_status(st) == 0                   # reading clears the word
    with pytest.raises(_lib.DcnError):
        assert L.dcn_debug_expire_wait(None, st) == 0
        _lib.check(L.dcn_check_status(st), "device status")
    case = cases.TC_CASES[0]
    ours = helpers.run_ours(case, cases.make_inputs(case), "bf16")      # the context is still usable
    _check_status()
    assert np.isfinite(ours["y"]).all()
