"""CPU checks of the C-ABI library: it loads, exports every symbol include/dcn.h declares, and its host-side
argument contract (the reference's shape_check) answers without touching a GPU."""
import ctypes
import os
import re

import pytest
import torch

from deform_conv3d_pytorch_op_b200 import _lib, build

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


@pytest.fixture(scope="module")
def L():
    build.build()
    return _lib.lib()


def test_header_symbols_are_exported(L):
    text = open(os.path.join(ROOT, "include", "dcn.h")).read()
    text = re.sub(r"/\*.*?\*/", "", text, flags=re.S)
    declared = set(re.findall(r"\b(dcn_[a-z0-9_]+)\s*\(", text))
    assert len(declared) >= 20
    # the header and the binding list the same entry points, and the library exports each of them
    assert declared == set(_lib.GENERIC_SYMBOLS + _lib.LEGACY_SYMBOLS)
    for sym in sorted(declared):
        assert hasattr(L, sym), sym


def test_channels_last_is_a_bf16_option(L):
    assert L.dcn_validate(ctypes.byref(_p(channels_last=True))) == -3            # exact precision: NCHW only
    ok = _p(C=16, O=16, G=1, cpg=16, precision=_lib.PREC_BF16, channels_last=True)
    assert L.dcn_validate(ctypes.byref(ok)) == 0
    assert L.dcn_launch_count(ctypes.byref(ok), _lib.PASS_BACKWARD) == 7        # no dx transpose pass
    ok.channels_last = 0
    assert L.dcn_launch_count(ctypes.byref(ok), _lib.PASS_BACKWARD) == 8
    ok.channels_last = 2
    assert L.dcn_validate(ctypes.byref(ok)) == -3


def _p(**kw):
    base = dict(ndim=2, dtype=torch.float32, N=2, C=4, O=6, in_size=(7, 7), kernel=(3, 3), stride=(1, 1), pad=(1, 1),
                dil=(1, 1), G=2, cpg=2)
    base.update(kw)
    return _lib.make_problem(**base)


def test_output_size_rules(L):
    # deformable rule ignores dilation (deform3d/lib/deform_conv3d_cuda.cpp:15-17)
    assert _lib.output_size(_p(dil=(2, 2), pad=(2, 2), stride=(2, 2))) == (5, 5)
    # plain conv rule is dilation-aware (conv2d/lib/conv2d_cuda.cpp:20-22)
    assert _lib.output_size(_p(dil=(2, 2), pad=(2, 2), stride=(2, 2), deformable=False, std_size_rule=True)) == (4, 4)
    # BASELINE config 4: 8x28x28, k3, stride (1,2,2), pad 2, dilation 2 -> 10x15x15
    p = _lib.make_problem(3, torch.float32, 16, 128, 256, (8, 28, 28), (3, 3, 3), (1, 2, 2), (2, 2, 2), (2, 2, 2), 4, 16)
    assert _lib.output_size(p) == (10, 15, 15)


def test_shape_contract(L):
    ok = _p()
    assert L.dcn_validate(ctypes.byref(ok)) == 0
    assert L.dcn_validate(ctypes.byref(_p(C=5))) == -2           # C % G
    assert L.dcn_validate(ctypes.byref(_p(O=5))) == -2           # O % G
    assert L.dcn_validate(ctypes.byref(_p(cpg=3))) == -2         # C % cpg
    assert L.dcn_validate(ctypes.byref(_p(in_size=(1, 1), pad=(0, 0)))) == -2   # empty output
    bad = _p()
    bad.ndim = 4
    assert L.dcn_validate(ctypes.byref(bad)) == -3
    assert L.dcn_validate(ctypes.byref(_p(precision=_lib.PREC_BF16, dtype=torch.float64))) == -3
    assert L.dcn_status_string(-2).decode().startswith("sizes")
    assert L.dcn_workspace_bytes(ctypes.byref(ok), 0) == 0       # EXACT precision needs no scratch


def test_sizes_beyond_the_32_bit_index_range_are_refused(L):
    """The kernels index positions, input elements of a sample and offset channels with 32-bit integers (the reference
    does too: `int` everywhere in deform3d/lib/deform_conv3d_cuda_kernel.cu:62-131); sizes past that are refused on
    the host with DCN_ERR_LIMIT instead of overflowing on the device."""
    big_batch = _p(N=70000, in_size=(256, 256), pad=(1, 1))                       # N * ov >= 2^31
    assert L.dcn_validate(ctypes.byref(big_batch)) == -8
    big_plane = _lib.make_problem(3, torch.float32, 1, 2048, 8, (64, 256, 256), (1, 1, 1), (1, 1, 1), (0, 0, 0),
                                  (1, 1, 1), 1, 2048)                               # C * iv >= 2^31
    assert L.dcn_validate(ctypes.byref(big_plane)) == -8
    many_offsets = _lib.make_problem(3, torch.float32, 1, 64, 8, (32, 128, 128), (3, 3, 3), (1, 1, 1), (1, 1, 1),
                                     (1, 1, 1), 1, 1)                               # dg * kv * 3 * ov >= 2^31
    assert L.dcn_validate(ctypes.byref(many_offsets)) == -8
    assert L.dcn_status_string(-8).decode().startswith("problem exceeds")
    assert L.dcn_workspace_bytes(ctypes.byref(big_batch), 0) == 0 and L.dcn_launch_count(ctypes.byref(big_batch), 0) == 0
    # the largest benchmark configuration is far inside the range
    cfg3 = _lib.make_problem(3, torch.float32, 8, 64, 64, (16, 56, 56), (3, 3, 3), (1, 1, 1), (1, 1, 1), (1, 1, 1), 1, 64)
    assert L.dcn_validate(ctypes.byref(cfg3)) == 0


def test_null_pointers_are_refused_before_any_launch(L):
    ok = _p()
    assert L.dcn_forward(ctypes.byref(ok), None, None, None, None, None, None, 0, None) == -1
    assert L.dcn_backward_data(ctypes.byref(ok), None, None, None, None, None, None, None, 0, None) == -1
    assert L.dcn_backward_weight(ctypes.byref(ok), None, None, None, None, None, None, 0, None) == -1


def test_offset_conv_problem_of_a_layer(L):
    """The convolution that produces a deformable problem's offsets (caller pattern deform3d/test_model.py:18-30):
    same taps, stride, padding, dilation 1, dg*kv*D output channels, and the deformable problem's output size."""
    p = _lib.make_problem(3, torch.float32, 2, 8, 6, (5, 9, 9), (3, 3, 3), (1, 2, 2), (1, 2, 2), (2, 2, 2), 2, 4)
    q = _lib.dcn_problem()
    assert L.dcn_offset_conv_problem(ctypes.byref(p), ctypes.byref(q)) == 0
    assert (q.O, q.G, q.deformable, q.C, q.N) == (2 * 27 * 3, 1, 0, 8, 2)
    assert tuple(q.dil) == (1, 1, 1) and tuple(q.k) == tuple(p.k) and tuple(q.stride) == tuple(p.stride)
    assert _lib.output_size(q) == _lib.output_size(p)
    plain = _p(deformable=False, std_size_rule=True)
    assert L.dcn_offset_conv_problem(ctypes.byref(plain), ctypes.byref(q)) == -3      # not a deformable problem
    # EXACT precision: the layer's backward workspace is the offset gradient, the forward needs none
    n_off = 2 * (2 * 27 * 3) * int(torch.Size(_lib.output_size(p)).numel()) * 4
    assert L.dcn_layer_workspace_bytes(ctypes.byref(p), _lib.PASS_FORWARD) == 0
    assert n_off <= L.dcn_layer_workspace_bytes(ctypes.byref(p), _lib.PASS_BACKWARD) < n_off + 256
    assert L.dcn_layer_forward(ctypes.byref(p), None, None, None, None, None, None, None, None, 0, None) == -1


def test_missing_library_fails_loudly(monkeypatch):
    monkeypatch.setattr(_lib, "_lib", None)
    monkeypatch.setattr(_lib, "LIB_PATH", "/nonexistent/libdcn.so")
    with pytest.raises(_lib.DcnError):
        _lib.lib()


def test_module_surface():
    import deform_conv3d_pytorch_op_b200 as dcn
    m = dcn.ConvOffset3d(8, 16, 3, stride=1, padding=1, dilation=1, channel_per_group=2, bias=True, groups=2)
    assert tuple(m.weight.shape) == (16, 4, 3, 3, 3) and tuple(m.bias.shape) == (16,)
    assert m.offset_channels == 4 * 27 * 3
    assert set(m.state_dict().keys()) == {"weight", "bias"}
    m2 = dcn.DeformConv2d(8, 8, 3, deformable_groups=4, bias=False)
    assert m2.channel_per_group == 2 and m2.bias is None and m2.offset_channels == 4 * 9 * 2
    with pytest.raises(ValueError):
        dcn.ConvOffset3d(6, 8, 3, groups=4)
    leg = dcn.LegacyConvOffset2d(4, 4, 3, 1, 1, 2)
    assert leg.bias is None and leg.dilation == (1, 1)
    c = dcn.Conv2d(4, 6, 3, groups=2)
    assert tuple(c.weight.shape) == (6, 2, 3, 3)
    c3 = dcn.Conv3d(4, 6, (1, 3, 3), groups=2)
    assert tuple(c3.weight.shape) == (6, 2, 1, 3, 3)
    layer = dcn.DeformLayer3d(8, 16, 3, padding=1, deformable_groups=2)
    assert tuple(layer.conv_offset.weight.shape) == (2 * 27 * 3, 8, 3, 3, 3)
    assert set(layer.state_dict().keys()) == {"conv.weight", "conv.bias", "conv_offset.weight", "conv_offset.bias"}
