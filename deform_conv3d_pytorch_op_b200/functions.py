"""autograd Functions with the reference's call signatures.

* :class:`ConvOffset3dFunction` -- deform3d/deform_conv3d_functions/deform_conv3d_function.py:7-77
* :class:`ConvOffset2dFunction` -- deform2d_double/deform_conv2d_functions/deform_conv2d_function.py:7-77
* :class:`Conv2dFunction`       -- conv2d/conv2d_functions/conv2d_function.py:8-67
* :class:`Conv3dFunction`       -- the same call form over three spatial axes (no counterpart in the reference)
* :class:`DeformLayerFunction`  -- offset-producing convolution + deformable convolution as one unit, the
  caller pattern of deform3d/test_model.py:18-30
* :class:`LegacyConvOffset2dFunction` -- the stateful fp32 2-D form,
  deform2d/deform_conv2d_functions/deform_conv2d_function.py:7-57

``.apply`` keeps the reference's positional order; ``backward`` returns the same slots.  Differences:
gradients are computed only for the inputs that need them (the reference always computes dX and dOffset
together), and two optional trailing arguments select the arithmetic (``precision``: exact | bf16 | auto)
and the 3-D out-of-bounds offset pseudo-gradient (``oob_offset_grad``).
"""
from __future__ import annotations

import torch
from torch.autograd import Function
from torch.autograd.function import once_differentiable

from .ops import Op, check_status, status_check_enabled


def _tup(v, n):
    return tuple(v) if isinstance(v, (tuple, list)) else (v,) * n


class _ConvOffsetNdFunction(Function):
    NDIM = 0

    @staticmethod
    def _fwd(ndim, ctx, inputs, offset, weight, bias, stride, padding, dilation, channel_per_group, group,
             precision, oob_offset_grad):
        if inputs.dim() != ndim + 2:
            raise RuntimeError("input dim")
        ctx.op = Op(inputs, weight, _tup(stride, ndim), _tup(padding, ndim), _tup(dilation, ndim), channel_per_group,
                    group, deformable=True, std_size_rule=False, oob_offset_grad=oob_offset_grad,
                    precision=precision)
        ctx.has_bias = bias is not None
        ctx.save_for_backward(inputs, offset, weight)
        ctx.fwd_ws = None
        need_bwd = any(t is not None and t.requires_grad for t in (inputs, offset, weight, bias))
        if need_bwd and torch.is_grad_enabled():
            y, ctx.fwd_ws = ctx.op.forward(inputs, offset, weight, bias, keep_workspace=True)
            ctx.x_version = inputs._version
            return y
        return ctx.op.forward(inputs, offset, weight, bias)

    @staticmethod
    def _bwd(ctx, grad_output):
        inputs, offset, weight = ctx.saved_tensors
        need = ctx.needs_input_grad
        want_db = ctx.has_bias and need[3]
        xcl = ctx.fwd_ws if (ctx.fwd_ws is not None and inputs._version == ctx.x_version) else None
        ctx.fwd_ws = None
        grads = ctx.op.backward(inputs, offset, weight, grad_output, need[0], need[1], need[2], want_db, xcl)
        if status_check_enabled() and not torch.cuda.is_current_stream_capturing():
            check_status(inputs.device)
        return grads


class ConvOffset3dFunction(_ConvOffsetNdFunction):
    @staticmethod
    def forward(ctx, inputs, offset, weight, bias=None, stride=(1, 1, 1), padding=(0, 0, 0), dilation=(1, 1, 1),
                channel_per_group=1, group=1, precision=None, oob_offset_grad=None):
        return _ConvOffsetNdFunction._fwd(3, ctx, inputs, offset, weight, bias, stride, padding, dilation,
                                          channel_per_group, group, precision, oob_offset_grad)

    @staticmethod
    @once_differentiable
    def backward(ctx, grad_output):
        return _ConvOffsetNdFunction._bwd(ctx, grad_output) + (None,) * 7


class ConvOffset2dFunction(_ConvOffsetNdFunction):
    @staticmethod
    def forward(ctx, inputs, offset, weight, bias=None, stride=(1, 1), padding=(0, 0), dilation=(1, 1),
                channel_per_group=1, group=1, precision=None, oob_offset_grad=None):
        return _ConvOffsetNdFunction._fwd(2, ctx, inputs, offset, weight, bias, stride, padding, dilation,
                                          channel_per_group, group, precision, oob_offset_grad)

    @staticmethod
    @once_differentiable
    def backward(ctx, grad_output):
        return _ConvOffsetNdFunction._bwd(ctx, grad_output) + (None,) * 7


class _ConvNdFunction(Function):
    """Plain (integer-tap) convolution on the same kernels with the deformable part switched off."""

    @staticmethod
    def _fwd(ndim, ctx, inputs, weight, bias, stride, padding, dilation, group, precision):
        if inputs.dim() != ndim + 2:
            raise RuntimeError("input dim")
        ctx.op = Op(inputs, weight, _tup(stride, ndim), _tup(padding, ndim), _tup(dilation, ndim), inputs.size(1),
                    group, deformable=False, std_size_rule=True, precision=precision)
        ctx.has_bias = bias is not None
        ctx.save_for_backward(inputs, weight)
        ctx.fwd_ws = None
        if torch.is_grad_enabled() and any(t is not None and t.requires_grad for t in (inputs, weight, bias)):
            y, ctx.fwd_ws = ctx.op.forward(inputs, None, weight, bias, keep_workspace=True)
            ctx.x_version = inputs._version
            return y
        return ctx.op.forward(inputs, None, weight, bias)

    @staticmethod
    def _bwd(ctx, grad_output):
        inputs, weight = ctx.saved_tensors
        need = ctx.needs_input_grad
        want_db = ctx.has_bias and need[2]
        xcl = ctx.fwd_ws if (ctx.fwd_ws is not None and inputs._version == ctx.x_version) else None
        ctx.fwd_ws = None
        grad_input, _, grad_weight, grad_bias = ctx.op.backward(inputs, None, weight, grad_output, need[0], False,
                                                                need[1], want_db, xcl)
        return grad_input, grad_weight, grad_bias, None, None, None, None, None


class Conv2dFunction(_ConvNdFunction):
    @staticmethod
    def forward(ctx, inputs, weight, bias=None, stride=(1, 1), padding=(0, 0), dilation=(1, 1), group=1,
                precision=None):
        return _ConvNdFunction._fwd(2, ctx, inputs, weight, bias, stride, padding, dilation, group, precision)

    @staticmethod
    @once_differentiable
    def backward(ctx, grad_output):
        return _ConvNdFunction._bwd(ctx, grad_output)


class Conv3dFunction(_ConvNdFunction):
    """The 3-D counterpart of :class:`Conv2dFunction` (the reference's plain-convolution package is 2-D only,
    conv2d/lib/conv2d_cuda.cpp:77-290; the same im2col + GEMM structure over (l, h, w))."""

    @staticmethod
    def forward(ctx, inputs, weight, bias=None, stride=(1, 1, 1), padding=(0, 0, 0), dilation=(1, 1, 1), group=1,
                precision=None):
        return _ConvNdFunction._fwd(3, ctx, inputs, weight, bias, stride, padding, dilation, group, precision)

    @staticmethod
    @once_differentiable
    def backward(ctx, grad_output):
        return _ConvNdFunction._bwd(ctx, grad_output)


class DeformLayerFunction(Function):
    """``apply(inputs, offset_weight, offset_bias, weight, bias, stride, padding, dilation, channel_per_group,
    group[, precision, oob_offset_grad])``: the offset-producing convolution and the deformable convolution of the
    reference's model scripts (deform3d/test_model.py:18-30, deform2d/test_model.py:19-31) as one differentiable
    unit; 2-D or 3-D by the input's rank.  The offsets never pass through the caller."""

    @staticmethod
    def forward(ctx, inputs, offset_weight, offset_bias, weight, bias, stride, padding, dilation,
                channel_per_group=1, group=1, precision=None, oob_offset_grad=None):
        ndim = inputs.dim() - 2
        ctx.op = Op(inputs, weight, _tup(stride, ndim), _tup(padding, ndim), _tup(dilation, ndim), channel_per_group,
                    group, oob_offset_grad=oob_offset_grad, precision=precision)
        ctx.has_bias = bias is not None
        ctx.has_offset_bias = offset_bias is not None
        ctx.fwd_ws = None
        train = torch.is_grad_enabled() and any(
            t is not None and t.requires_grad for t in (inputs, offset_weight, offset_bias, weight, bias))
        if train:
            y, offset, ctx.fwd_ws = ctx.op.layer_forward(inputs, offset_weight, offset_bias, weight, bias,
                                                         keep_workspace=True)
            ctx.x_version = inputs._version
        else:
            y, offset = ctx.op.layer_forward(inputs, offset_weight, offset_bias, weight, bias)
        ctx.save_for_backward(inputs, offset, offset_weight, weight)
        return y

    @staticmethod
    @once_differentiable
    def backward(ctx, grad_output):
        inputs, offset, offset_weight, weight = ctx.saved_tensors
        need = ctx.needs_input_grad
        xcl = ctx.fwd_ws if (ctx.fwd_ws is not None and inputs._version == ctx.x_version) else None
        ctx.fwd_ws = None
        dx, dow, dob, dw, db = ctx.op.layer_backward(
            inputs, offset, offset_weight, weight, grad_output, need[0], need[1], ctx.has_offset_bias and need[2],
            need[3], ctx.has_bias and need[4], xcl)
        if status_check_enabled() and not torch.cuda.is_current_stream_capturing():
            check_status(inputs.device)
        return (dx, dow, dob, dw, db) + (None,) * 7


class LegacyConvOffset2dFunction:
    """``ConvOffset2dFunction(stride, padding, channel_per_group)(input, offset, weight)`` -- the stateful call
    form of the fp32 2-D package (no dilation, no groups, no bias)."""

    def __init__(self, stride, padding, channel_per_group):
        self.stride = _tup(stride, 2)
        self.padding = _tup(padding, 2)
        self.channel_per_group = channel_per_group

    def __call__(self, inputs, offset, weight):
        return ConvOffset2dFunction.apply(inputs, offset, weight, None, self.stride, self.padding, (1, 1),
                                          self.channel_per_group, 1)
