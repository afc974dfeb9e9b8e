"""nn.Modules with the reference's constructor signatures.

* :class:`ConvOffset3d` -- deform3d/deform_conv3d_modules/deform_conv3d_model.py:11-50
* :class:`ConvOffset2d` -- deform2d_double/deform_conv2d_modules/deform_conv2d_model.py:11-52 (any float dtype)
* :class:`Conv2d`       -- conv2d/conv2d_modules/conv2d_model.py:11-46
* :class:`Conv3d`       -- the same module over three spatial axes (no counterpart in the reference)
* :class:`LegacyConvOffset2d` -- deform2d/deform_conv2d_modules/deform_conv2d_model.py:11-32
* :class:`DeformLayer3d` / :class:`DeformLayer2d` -- offset-producing convolution + deformable convolution, the
  pair of modules the reference's model scripts build by hand (deform3d/test_model.py:18-30)

Parameter names (``weight`` [O, C/G, k...], ``bias`` [O]) match, so state dicts are interchangeable.
Initialisation is Kaiming-normal (fan_out) for the weight and U(-0.1, 0.1) for the bias as in the reference;
the constant-1 overwrite of the weight that the 3-D and fp64 2-D reference modules perform afterwards
(deform_conv3d_model.py:39) is a debugging leftover and is not reproduced.
``deformable_groups=`` is accepted as an alternative to ``channel_per_group`` (cpg = in_channels / dg).
"""
from __future__ import annotations

import torch
import torch.nn as nn
from torch.nn.modules.utils import _pair, _triple

from .functions import (Conv2dFunction, Conv3dFunction, ConvOffset2dFunction, ConvOffset3dFunction,
                        DeformLayerFunction)


def _resolve_cpg(in_channels, channel_per_group, deformable_groups):
    if deformable_groups is not None:
        if in_channels % deformable_groups != 0:
            raise ValueError("in_channels must be divisible by deformable_groups")
        return in_channels // deformable_groups
    if in_channels % channel_per_group != 0:
        raise ValueError("in_channels must be divisible by channel_per_group")
    return channel_per_group


class _ConvOffsetNd(nn.Module):
    _ntuple = None
    _function = None

    def __init__(self, in_channels, out_channels, kernel_size, stride=1, padding=0, dilation=1, channel_per_group=1,
                 bias=True, groups=1, deformable_groups=None, precision=None, oob_offset_grad=None, device=None,
                 dtype=None):
        super().__init__()
        nt = type(self)._ntuple
        self.in_channels = in_channels
        self.out_channels = out_channels
        self.kernel_size = nt(kernel_size)
        self.stride = nt(stride)
        self.padding = nt(padding)
        self.dilation = nt(dilation)
        self.channel_per_group = _resolve_cpg(in_channels, channel_per_group, deformable_groups)
        self.group = groups
        self.precision = precision
        self.oob_offset_grad = oob_offset_grad
        if in_channels % groups != 0:
            raise ValueError('in_channels must be divisible by groups')
        if out_channels % groups != 0:
            raise ValueError('out_channels must be divisible by groups')
        kw = {"device": device, "dtype": dtype}
        self.weight = nn.Parameter(torch.empty(out_channels, in_channels // groups, *self.kernel_size, **kw))
        nn.init.kaiming_normal_(self.weight, mode='fan_out')
        if bias:
            self.bias = nn.Parameter(torch.empty(out_channels, **kw))
            nn.init.uniform_(self.bias, -0.1, 0.1)
        else:
            self.register_parameter('bias', None)

    @property
    def deformable_groups(self):
        return self.in_channels // self.channel_per_group

    @property
    def offset_channels(self):
        n = 1
        for k in self.kernel_size:
            n *= k
        return self.deformable_groups * n * len(self.kernel_size)

    def forward(self, input, offset):
        return type(self)._function.apply(input, offset, self.weight, self.bias, self.stride, self.padding,
                                          self.dilation, self.channel_per_group, self.group, self.precision,
                                          self.oob_offset_grad)

    def extra_repr(self):
        return ("{in_channels}, {out_channels}, kernel_size={kernel_size}, stride={stride}, padding={padding}, "
                "dilation={dilation}, channel_per_group={channel_per_group}, groups={group}").format(**self.__dict__)


class ConvOffset3d(_ConvOffsetNd):
    _ntuple = staticmethod(_triple)
    _function = ConvOffset3dFunction


class ConvOffset2d(_ConvOffsetNd):
    _ntuple = staticmethod(_pair)
    _function = ConvOffset2dFunction


class LegacyConvOffset2d(ConvOffset2d):
    """``ConvOffset2d(in_channels, out_channels, kernel_size, stride=1, padding=0, channel_per_group=1)``:
    fp32, no dilation, no groups, no bias."""

    def __init__(self, in_channels, out_channels, kernel_size, stride=1, padding=0, channel_per_group=1, **kw):
        super().__init__(in_channels, out_channels, kernel_size, stride, padding, 1, channel_per_group, False, 1, **kw)


class _ConvNd(nn.Module):
    _ntuple = None
    _function = None

    def __init__(self, in_channels, out_channels, kernel_size, stride=1, padding=0, dilation=1, bias=True, groups=1,
                 precision=None, device=None, dtype=None):
        super().__init__()
        nt = type(self)._ntuple
        self.in_channels = in_channels
        self.out_channels = out_channels
        self.kernel_size = nt(kernel_size)
        self.stride = nt(stride)
        self.padding = nt(padding)
        self.dilation = nt(dilation)
        self.group = groups
        self.precision = precision
        if in_channels % groups != 0:
            raise ValueError('in_channels must be divisible by groups')
        if out_channels % groups != 0:
            raise ValueError('out_channels must be divisible by groups')
        kw = {"device": device, "dtype": dtype}
        self.weight = nn.Parameter(torch.empty(out_channels, in_channels // groups, *self.kernel_size, **kw))
        nn.init.kaiming_normal_(self.weight, mode='fan_out')
        if bias:
            self.bias = nn.Parameter(torch.empty(out_channels, **kw))
            nn.init.uniform_(self.bias, -0.1, 0.1)
        else:
            self.register_parameter('bias', None)

    def forward(self, inputs):
        return type(self)._function.apply(inputs, self.weight, self.bias, self.stride, self.padding, self.dilation,
                                          self.group, self.precision)


class Conv2d(_ConvNd):
    _ntuple = staticmethod(_pair)
    _function = Conv2dFunction


class Conv3d(_ConvNd):
    """Plain 3-D convolution on the library's kernels (same constructor as :class:`Conv2d` with triples)."""
    _ntuple = staticmethod(_triple)
    _function = Conv3dFunction


class _DeformLayerNd(nn.Module):
    """The reference's model-script pattern as one module: ``conv_offset`` (a stock convolution module that only
    holds the parameters of the offset-producing convolution: same kernel, stride and padding as the deformable
    one, dilation 1, ``dg * kv * D`` output channels) and ``conv`` (a :class:`ConvOffset3d` / :class:`ConvOffset2d`).
    ``forward(input)`` runs both through one library call, so state dicts of a model that keeps the two modules
    side by side (deform3d/test_model.py:18-30) load unchanged under the names ``conv_offset.*`` / ``conv.*``.
    ``offset_std``: the offset weights start at N(0, offset_std^2) with zero bias (offsets near zero)."""
    _conv = None
    _deform = None

    def __init__(self, in_channels, out_channels, kernel_size, stride=1, padding=0, dilation=1, channel_per_group=1,
                 bias=True, groups=1, deformable_groups=None, offset_bias=True, offset_std=0.01, precision=None,
                 oob_offset_grad=None, device=None, dtype=None):
        super().__init__()
        cls = type(self)
        self.conv = cls._deform(in_channels, out_channels, kernel_size, stride, padding, dilation, channel_per_group,
                                bias, groups, deformable_groups, precision, oob_offset_grad, device, dtype)
        self.conv_offset = cls._conv(in_channels, self.conv.offset_channels, self.conv.kernel_size, self.conv.stride,
                                     self.conv.padding, bias=offset_bias, device=device, dtype=dtype)
        nn.init.normal_(self.conv_offset.weight, 0.0, offset_std)
        if offset_bias:
            nn.init.zeros_(self.conv_offset.bias)

    def forward(self, input):
        c = self.conv
        return DeformLayerFunction.apply(input, self.conv_offset.weight, self.conv_offset.bias, c.weight, c.bias,
                                         c.stride, c.padding, c.dilation, c.channel_per_group, c.group, c.precision,
                                         c.oob_offset_grad)


class DeformLayer3d(_DeformLayerNd):
    _conv = nn.Conv3d
    _deform = ConvOffset3d


class DeformLayer2d(_DeformLayerNd):
    _conv = nn.Conv2d
    _deform = ConvOffset2d


DeformConv2d = ConvOffset2d
DeformConv3d = ConvOffset3d
