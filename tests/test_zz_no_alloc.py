"""The allocation-free forward entry point (dcn_forward_static_scratch), called through the C ABI.

Some callers cannot give the library a workspace because they may not allocate device memory at the point
of the call (plugin enqueue hooks, real-time loops, processes whose pool already owns the device).  For them
the library carries a fixed 32 MiB scratch array.  This test checks that the entry point produces what the
ordinary workspace-based entry point produces, on two consecutive calls (the array is shared and keeps the
previous call's bytes), and that oversize problems are refused before any launch.  Collected last on purpose.
"""
import ctypes

import numpy as np
import pytest
import torch

from tests import cases

TOL_BF16 = 2e-2


def _problem(case, n=None):
    from deform_conv3d_pytorch_op_b200 import _lib
    return _lib.make_problem(case.ndim, torch.float32, case.N if n is None else n, case.C, case.O, case.in_size,
                             case.kernel, case.stride, case.pad, case.dil, case.G, case.cpg, True, False, True,
                             _lib.PREC_BF16)


def test_oversize_problem_is_refused_on_the_host():
    from deform_conv3d_pytorch_op_b200 import _lib
    L = _lib.lib()
    assert L.dcn_static_scratch_bytes() == 32 << 20
    big = _problem(cases.BASELINE[2])                       # forward workspace ~ 54 MB > 32 MiB
    assert L.dcn_workspace_bytes(ctypes.byref(big), 0) > L.dcn_static_scratch_bytes()
    one = ctypes.c_void_p(256)                              # never dereferenced: refusal comes first
    assert L.dcn_forward_static_scratch(ctypes.byref(big), one, one, one, None, one, None) == -8
    exact = _problem(cases.TC_CASES[0])
    exact.precision = _lib.PREC_EXACT
    assert L.dcn_forward_static_scratch(ctypes.byref(exact), one, one, one, None, one, None) == -3


@pytest.mark.gpu
@pytest.mark.parametrize("name", ["tc2_small", "tc3_groups"])
def test_static_scratch_forward_matches_workspace_forward(name):
    from deform_conv3d_pytorch_op_b200 import _lib
    L = _lib.lib()
    case = {c.name: c for c in cases.TC_CASES}[name]
    dev = torch.device("cuda")
    stream = _lib.current_stream(dev)
    prob = _problem(case)
    free_before_second_call = None
    for seed in (0, 1):                                    # two calls in a row on the shared array
        x, w, off, dy, b = [None if t is None else t.to(dev) for t in cases.make_inputs(case, seed=seed)]
        out_shape = (case.N, case.O) + _lib.output_size(prob)
        y_ws = torch.full(out_shape, float("nan"), device=dev)
        y_st = torch.full(out_shape, float("nan"), device=dev)
        nbytes = L.dcn_workspace_bytes(ctypes.byref(prob), 0)
        ws = torch.empty(nbytes, dtype=torch.uint8, device=dev)
        _lib.check(L.dcn_forward(ctypes.byref(prob), _lib.ptr(x), _lib.ptr(off), _lib.ptr(w), _lib.ptr(b),
                                 _lib.ptr(y_ws), _lib.ptr(ws), nbytes, stream), "dcn_forward")
        if seed == 1:
            torch.cuda.synchronize()
            free_before_second_call = torch.cuda.mem_get_info(dev)[0]
        _lib.check(L.dcn_forward_static_scratch(ctypes.byref(prob), _lib.ptr(x), _lib.ptr(off), _lib.ptr(w),
                                                _lib.ptr(b), _lib.ptr(y_st), stream), "dcn_forward_static_scratch")
        torch.cuda.synchronize()
        if seed == 1:
            # nothing was allocated on the device by the call (the first call may have loaded device code)
            assert torch.cuda.mem_get_info(dev)[0] == free_before_second_call
        _lib.check(L.dcn_check_status(stream), "device status")
        a, r = y_st.cpu().numpy(), y_ws.cpu().numpy()
        assert np.isfinite(a).all() and np.isfinite(r).all()
        assert cases.rel_err(a, r) <= TOL_BF16, cases.rel_err(a, r)
        assert np.array_equal(a, r)                        # same kernels, same inputs: identical bits


@pytest.mark.gpu
def test_static_scratch_forward_takes_channels_last_activations():
    """Same entry point with dcn_problem.channels_last = 1: x and y are [N, spatial, channels]."""
    from deform_conv3d_pytorch_op_b200 import _lib
    L = _lib.lib()
    case = {c.name: c for c in cases.TC_CASES}["tc2_small"]
    dev = torch.device("cuda")
    stream = _lib.current_stream(dev)
    prob = _problem(case)
    x, w, off, dy, b = [None if t is None else t.to(dev) for t in cases.make_inputs(case)]
    out_shape = (case.N, case.O) + _lib.output_size(prob)
    y_ref = torch.empty(out_shape, device=dev)
    _lib.check(L.dcn_forward_static_scratch(ctypes.byref(prob), _lib.ptr(x), _lib.ptr(off), _lib.ptr(w), _lib.ptr(b),
                                            _lib.ptr(y_ref), stream), "reference layout")
    prob.channels_last = 1
    x_cl = x.permute(0, 2, 3, 1).contiguous()                        # [N, H, W, C]
    y_cl = torch.full((case.N,) + _lib.output_size(prob) + (case.O,), float("nan"), device=dev)
    _lib.check(L.dcn_forward_static_scratch(ctypes.byref(prob), _lib.ptr(x_cl), _lib.ptr(off), _lib.ptr(w),
                                            _lib.ptr(b), _lib.ptr(y_cl), stream), "channels last")
    torch.cuda.synchronize()
    _lib.check(L.dcn_check_status(stream), "device status")
    a, r = y_cl.permute(0, 3, 1, 2).cpu().numpy(), y_ref.cpu().numpy()
    assert np.isfinite(a).all()
    assert cases.rel_err(a, r) <= 1e-5, cases.rel_err(a, r)


@pytest.mark.gpu
def test_static_scratch_address_is_resolved_per_device():
    """On a box with several GPUs the fixed array's address is resolved for each device separately."""
    if torch.cuda.device_count() < 2:
        pytest.skip("one GPU")
    from deform_conv3d_pytorch_op_b200 import _lib
    L = _lib.lib()
    case = {c.name: c for c in cases.TC_CASES}["tc2_small"]
    prob = _problem(case)
    outs = []
    for d in (0, 1):
        dev = torch.device("cuda", d)
        with torch.cuda.device(dev):
            x, w, off, dy, b = [None if t is None else t.to(dev) for t in cases.make_inputs(case)]
            y = torch.full((case.N, case.O) + _lib.output_size(prob), float("nan"), device=dev)
            _lib.check(L.dcn_forward_static_scratch(ctypes.byref(prob), _lib.ptr(x), _lib.ptr(off), _lib.ptr(w),
                                                    _lib.ptr(b), _lib.ptr(y), _lib.current_stream(dev)), "device %d" % d)
            torch.cuda.synchronize(dev)
            outs.append(y.cpu().numpy())
    assert np.isfinite(outs[0]).all() and np.array_equal(outs[0], outs[1])
