"""The reference's FFI call surface on torch tensors, one namespace per reference package.

Each function has the reference symbol's name and argument order and forwards to the matching
reference-named C entry point of libdcn.so.  ``columns`` (the im2col scratch the reference makes its
caller allocate) is accepted and ignored.  As in the reference, the caller allocates and zero-fills the
output / gradient tensors; the functions return 1.

* deform_conv3d_op  -- deform3d/lib/deform_conv3d_cuda.h:12-34, loaded by deform3d/deform_conv3d_op/__init__.py:2-12
* deform_conv2d_op  -- deform2d/lib/deform_conv2d_cuda.h:12-31 (fp32, no dilation / group)
* deform_conv2d_double_op -- deform2d_double/lib/deform_conv2d_cuda.h:12-34 (fp64)
* conv2d_op         -- conv2d/lib/conv2d_cuda.h:17-39
"""
from __future__ import annotations

import ctypes
import types

import torch

from . import _lib
from ._lib import DcnError

_i = ctypes.c_int


def _chk(name, *tensors, dtype):
    dev = None
    for t in tensors:
        if t is None:
            continue
        if not t.is_cuda or not t.is_contiguous():
            raise DcnError(name + ": tensors must be contiguous CUDA tensors")
        if t.dtype != dtype:
            raise DcnError(name + ": expected dtype %s, got %s" % (dtype, t.dtype))
        if dev is not None and t.device != dev:
            raise DcnError(name + ": tensors on different GPUs")       # THCAssertSameGPU
        dev = t.device
    return dev


def _call(sym, dev, *args):
    fn = getattr(_lib.lib(), sym)
    with torch.cuda.device(dev):
        r = fn(*args, _lib.current_stream(dev))
    if r != 1:
        _lib.check(r, sym)
    return 1


def _expect(t, shape, msg):
    if tuple(t.shape) != tuple(shape):
        raise DcnError(msg)


def _out3(inp, w, pad, stride):
    return tuple((inp.size(i + 2) + 2 * pad[i] - w.size(i + 2)) // stride[i] + 1 for i in range(inp.dim() - 2))


# ---- deform3d -----------------------------------------------------------------------------------------
def _d3_sizes(inp, w):
    return [_i(inp.size(0)), _i(inp.size(1)), _i(inp.size(2)), _i(inp.size(3)), _i(inp.size(4)), _i(w.size(0)),
            _i(w.size(2)), _i(w.size(3)), _i(w.size(4))]


def _d3_forward(input, weight, offset, columns, output, pad_l, pad_h, pad_w, stride_l, stride_h, stride_w,
                dilation_l, dilation_h, dilation_w, channel_per_deformable_group, group):
    dev = _chk("deform_conv_forward_cuda", input, weight, offset, output, dtype=torch.float32)
    _expect(output, (input.size(0), weight.size(0)) + _out3(input, weight, (pad_l, pad_h, pad_w),
                                                            (stride_l, stride_h, stride_w)), "error output size")
    return _call("dcn_deform3d_deform_conv_forward_cuda", dev, _lib.ptr(input), _lib.ptr(weight), _lib.ptr(offset),
                 _lib.ptr(output), *_d3_sizes(input, weight), _i(pad_l), _i(pad_h), _i(pad_w), _i(stride_l),
                 _i(stride_h), _i(stride_w), _i(dilation_l), _i(dilation_h), _i(dilation_w),
                 _i(channel_per_deformable_group), _i(group))


def _d3_backward_input_offset(input, weight, offset, grad_output, columns, grad_input, grad_offset, pad_l, pad_h,
                              pad_w, stride_l, stride_h, stride_w, dilation_l, dilation_h, dilation_w,
                              channel_per_deformable_group, group):
    dev = _chk("deform_conv_backward_input_offset_cuda", input, weight, offset, grad_output, grad_input, grad_offset,
               dtype=torch.float32)
    _expect(grad_offset, offset.shape, "offset vs grad_offset")
    _expect(grad_input, input.shape, "input vs grad_input")
    return _call("dcn_deform3d_deform_conv_backward_input_offset_cuda", dev, _lib.ptr(input), _lib.ptr(weight),
                 _lib.ptr(offset), _lib.ptr(grad_output), _lib.ptr(grad_input), _lib.ptr(grad_offset),
                 *_d3_sizes(input, weight), _i(pad_l), _i(pad_h), _i(pad_w), _i(stride_l), _i(stride_h), _i(stride_w),
                 _i(dilation_l), _i(dilation_h), _i(dilation_w), _i(channel_per_deformable_group), _i(group))


def _d3_backward_weight(input, offset, grad_output, columns, grad_weight, pad_l, pad_h, pad_w, stride_l, stride_h,
                        stride_w, dilation_l, dilation_h, dilation_w, channel_per_deformable_group, group):
    dev = _chk("deform_conv_backward_weight_cuda", input, offset, grad_output, grad_weight, dtype=torch.float32)
    return _call("dcn_deform3d_deform_conv_backward_weight_cuda", dev, _lib.ptr(input), _lib.ptr(offset),
                 _lib.ptr(grad_output), _lib.ptr(grad_weight), *_d3_sizes(input, grad_weight), _i(pad_l), _i(pad_h),
                 _i(pad_w), _i(stride_l), _i(stride_h), _i(stride_w), _i(dilation_l), _i(dilation_h), _i(dilation_w),
                 _i(channel_per_deformable_group), _i(group))


# ---- 2-D (fp32 legacy and fp64) -----------------------------------------------------------------------
def _d2_sizes(inp, w):
    return [_i(inp.size(0)), _i(inp.size(1)), _i(inp.size(2)), _i(inp.size(3)), _i(w.size(0)), _i(w.size(2)),
            _i(w.size(3))]


def _d2_forward(input, weight, offset, columns, output, pad_h, pad_w, stride_h, stride_w,
                channel_per_deformable_group):
    dev = _chk("deform_conv_forward_cuda", input, weight, offset, output, dtype=torch.float32)
    _expect(output, (input.size(0), weight.size(0)) + _out3(input, weight, (pad_h, pad_w), (stride_h, stride_w)),
            "error output size")
    return _call("dcn_deform2d_deform_conv_forward_cuda", dev, _lib.ptr(input), _lib.ptr(weight), _lib.ptr(offset),
                 _lib.ptr(output), *_d2_sizes(input, weight), _i(pad_h), _i(pad_w), _i(stride_h), _i(stride_w),
                 _i(channel_per_deformable_group))


def _d2_backward_input_offset(input, weight, offset, grad_output, columns, grad_input, grad_offset, pad_h, pad_w,
                              stride_h, stride_w, channel_per_deformable_group):
    dev = _chk("deform_conv_backward_input_offset_cuda", input, weight, offset, grad_output, grad_input, grad_offset,
               dtype=torch.float32)
    _expect(grad_offset, offset.shape, "offset vs grad_offset")
    _expect(grad_input, input.shape, "input vs grad_input")
    return _call("dcn_deform2d_deform_conv_backward_input_offset_cuda", dev, _lib.ptr(input), _lib.ptr(weight),
                 _lib.ptr(offset), _lib.ptr(grad_output), _lib.ptr(grad_input), _lib.ptr(grad_offset),
                 *_d2_sizes(input, weight), _i(pad_h), _i(pad_w), _i(stride_h), _i(stride_w),
                 _i(channel_per_deformable_group))


def _d2_backward_weight(input, offset, grad_output, columns, grad_weight, pad_h, pad_w, stride_h, stride_w,
                        channel_per_deformable_group):
    dev = _chk("deform_conv_backward_weight_cuda", input, offset, grad_output, grad_weight, dtype=torch.float32)
    return _call("dcn_deform2d_deform_conv_backward_weight_cuda", dev, _lib.ptr(input), _lib.ptr(offset),
                 _lib.ptr(grad_output), _lib.ptr(grad_weight), *_d2_sizes(input, grad_weight), _i(pad_h), _i(pad_w),
                 _i(stride_h), _i(stride_w), _i(channel_per_deformable_group))


def _d2d_forward(input, weight, offset, columns, output, pad_h, pad_w, stride_h, stride_w, dilation_h, dilation_w,
                 channel_per_deformable_group, group):
    dev = _chk("deform_conv_forward_cuda", input, weight, offset, output, dtype=torch.float64)
    _expect(output, (input.size(0), weight.size(0)) + _out3(input, weight, (pad_h, pad_w), (stride_h, stride_w)),
            "error output size")
    return _call("dcn_deform2d_double_deform_conv_forward_cuda", dev, _lib.ptr(input), _lib.ptr(weight),
                 _lib.ptr(offset), _lib.ptr(output), *_d2_sizes(input, weight), _i(pad_h), _i(pad_w), _i(stride_h),
                 _i(stride_w), _i(dilation_h), _i(dilation_w), _i(channel_per_deformable_group), _i(group))


def _d2d_backward_input_offset(input, weight, offset, grad_output, columns, grad_input, grad_offset, pad_h, pad_w,
                               stride_h, stride_w, dilation_h, dilation_w, channel_per_deformable_group, group):
    dev = _chk("deform_conv_backward_input_offset_cuda", input, weight, offset, grad_output, grad_input, grad_offset,
               dtype=torch.float64)
    _expect(grad_offset, offset.shape, "offset vs grad_offset")
    _expect(grad_input, input.shape, "input vs grad_input")
    return _call("dcn_deform2d_double_deform_conv_backward_input_offset_cuda", dev, _lib.ptr(input),
                 _lib.ptr(weight), _lib.ptr(offset), _lib.ptr(grad_output), _lib.ptr(grad_input),
                 _lib.ptr(grad_offset), *_d2_sizes(input, weight), _i(pad_h), _i(pad_w), _i(stride_h), _i(stride_w),
                 _i(dilation_h), _i(dilation_w), _i(channel_per_deformable_group), _i(group))


def _d2d_backward_weight(input, offset, grad_output, columns, grad_weight, pad_h, pad_w, stride_h, stride_w,
                         dilation_h, dilation_w, channel_per_deformable_group, group):
    dev = _chk("deform_conv_backward_weight_cuda", input, offset, grad_output, grad_weight, dtype=torch.float64)
    return _call("dcn_deform2d_double_deform_conv_backward_weight_cuda", dev, _lib.ptr(input), _lib.ptr(offset),
                 _lib.ptr(grad_output), _lib.ptr(grad_weight), *_d2_sizes(input, grad_weight), _i(pad_h), _i(pad_w),
                 _i(stride_h), _i(stride_w), _i(dilation_h), _i(dilation_w), _i(channel_per_deformable_group),
                 _i(group))


# ---- plain conv2d -------------------------------------------------------------------------------------
def _c2_forward(input, weight, columns, output, pad_h, pad_w, stride_h, stride_w, dilation_h, dilation_w, group):
    dev = _chk("conv_forward_cuda", input, weight, output, dtype=torch.float32)
    return _call("dcn_conv2d_conv_forward_cuda", dev, _lib.ptr(input), _lib.ptr(weight), _lib.ptr(output),
                 *_d2_sizes(input, weight), _i(pad_h), _i(pad_w), _i(stride_h), _i(stride_w), _i(dilation_h),
                 _i(dilation_w), _i(group))


def _c2_backward_input(weight, grad_output, columns, grad_input, pad_h, pad_w, stride_h, stride_w, dilation_h,
                       dilation_w, group):
    dev = _chk("conv_backward_input_cuda", weight, grad_output, grad_input, dtype=torch.float32)
    return _call("dcn_conv2d_conv_backward_input_cuda", dev, _lib.ptr(weight), _lib.ptr(grad_output),
                 _lib.ptr(grad_input), *_d2_sizes(grad_input, weight), _i(pad_h), _i(pad_w), _i(stride_h),
                 _i(stride_w), _i(dilation_h), _i(dilation_w), _i(group))


def _c2_backward_weight(input, grad_output, columns, grad_weight, pad_h, pad_w, stride_h, stride_w, dilation_h,
                        dilation_w, group):
    dev = _chk("conv_backward_weight_cuda", input, grad_output, grad_weight, dtype=torch.float32)
    return _call("dcn_conv2d_conv_backward_weight_cuda", dev, _lib.ptr(input), _lib.ptr(grad_output),
                 _lib.ptr(grad_weight), *_d2_sizes(input, grad_weight), _i(pad_h), _i(pad_w), _i(stride_h),
                 _i(stride_w), _i(dilation_h), _i(dilation_w), _i(group))


deform_conv3d_op = types.SimpleNamespace(
    deform_conv_forward_cuda=_d3_forward,
    deform_conv_backward_input_offset_cuda=_d3_backward_input_offset,
    deform_conv_backward_weight_cuda=_d3_backward_weight)
deform_conv2d_op = types.SimpleNamespace(
    deform_conv_forward_cuda=_d2_forward,
    deform_conv_backward_input_offset_cuda=_d2_backward_input_offset,
    deform_conv_backward_weight_cuda=_d2_backward_weight)
deform_conv2d_double_op = types.SimpleNamespace(
    deform_conv_forward_cuda=_d2d_forward,
    deform_conv_backward_input_offset_cuda=_d2d_backward_input_offset,
    deform_conv_backward_weight_cuda=_d2d_backward_weight)
conv2d_op = types.SimpleNamespace(
    conv_forward_cuda=_c2_forward,
    conv_backward_input_cuda=_c2_backward_input,
    conv_backward_weight_cuda=_c2_backward_weight)
