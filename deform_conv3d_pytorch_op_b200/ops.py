"""Tensor-level entry points over the C ABI: the three passes of the operator on torch CUDA tensors.

These are the counterparts of the reference's FFI calls (``deform_conv3d_op.deform_conv_forward_cuda`` and
siblings, deform3d/lib/deform_conv3d_cuda.h:12-34) with the output allocation the reference does in Python
(deform3d/deform_conv3d_functions/deform_conv3d_function.py:26-32, 53-54, 64) folded in.  torch is used for
device memory and the current stream only; all arithmetic happens in libdcn.so.
"""
from __future__ import annotations

import ctypes
import os
from typing import Optional, Tuple

import torch

from . import _lib
from ._lib import DcnError

_PRECISIONS = {"exact": _lib.PREC_EXACT, "fp32": _lib.PREC_EXACT, "bf16": _lib.PREC_BF16}


def default_precision() -> str:
    """``DCN_PRECISION`` = exact | bf16 | auto (default exact: compute in the tensor dtype)."""
    return os.environ.get("DCN_PRECISION", "exact").lower()


def default_oob_offset_grad() -> bool:
    """``DCN_OOB_OFFSET_GRAD`` = reference | zero (default reference; only 3-D has the term)."""
    return os.environ.get("DCN_OOB_OFFSET_GRAD", "reference").lower() != "zero"


def check_status(device=None) -> None:
    """Reads and clears the library's device-side status word on ``device`` (default: the current CUDA device)
    and raises :class:`DcnError` if a bounded device-side wait of a tensor-core kernel gave up since the last
    check.  Synchronises the device's current stream.  The word is sticky and process-wide per device, so a check
    tells that *some* call since the previous check failed, not which one: check once per step (or per call while
    debugging; ``DCN_CHECK_STATUS=1`` makes every backward pass of the autograd Functions do so)."""
    dev = torch.device("cuda", torch.cuda.current_device()) if device is None else torch.device(device)
    with torch.cuda.device(dev):
        _lib.check(_lib.lib().dcn_check_status(_lib.current_stream(dev)), "device status")


def status_check_enabled() -> bool:
    """``DCN_CHECK_STATUS=1``: poll the status word after every backward pass (never inside a stream capture)."""
    return os.environ.get("DCN_CHECK_STATUS", "0") not in ("", "0")


def _nvtx_enabled() -> bool:
    """``DCN_NVTX=1``: wrap every library call of :class:`Op` in an NVTX range named after the entry point, so that
    the passes show up by name on a profiler's timeline (the reference has only wall-clock prints,
    deform2d/test_function.py:30-58)."""
    return os.environ.get("DCN_NVTX", "0") not in ("", "0")


class _Range:
    def __init__(self, name: str):
        self.on = _nvtx_enabled()
        self.name = name

    def __enter__(self):
        if self.on:
            torch.cuda.nvtx.range_push(self.name)

    def __exit__(self, *exc):
        if self.on:
            torch.cuda.nvtx.range_pop()
        return False


def _prep(t: Optional[torch.Tensor], name: str, ref: Optional[torch.Tensor] = None) -> Optional[torch.Tensor]:
    if t is None:
        return None
    if not t.is_cuda:
        raise DcnError("%s must be a CUDA tensor (there is no CPU implementation)" % name)
    if ref is not None:
        if t.device != ref.device:
            raise DcnError("%s is on %s but input is on %s" % (name, t.device, ref.device))
        if t.dtype != ref.dtype:
            raise DcnError("%s has dtype %s but input has %s" % (name, t.dtype, ref.dtype))
    return t.contiguous()


class Op:
    """One validated operator instance (geometry + precision) bound to a device."""

    def __init__(self, x: torch.Tensor, weight: torch.Tensor, stride, padding, dilation, channel_per_group: int,
                 group: int, deformable: bool = True, std_size_rule: bool = False,
                 oob_offset_grad: Optional[bool] = None, precision: Optional[str] = None,
                 channels_last: Optional[bool] = None):
        ndim = x.dim() - 2
        if ndim not in (2, 3):
            raise DcnError("input dim")                       # reference: check(input_dim == 5, "input dim")
        if weight.dim() != ndim + 2:
            raise DcnError("kernel dim")
        if x.size(1) != weight.size(1) * group:
            raise DcnError("input c != kernel c")
        self.ndim = ndim
        self.device = x.device
        self.dtype = x.dtype
        prec = (precision or default_precision()).lower()
        if oob_offset_grad is None:
            oob_offset_grad = default_oob_offset_grad()
        cpg = channel_per_group if deformable else x.size(1)
        # Channels-last activations (torch.channels_last / channels_last_3d storage) are taken and produced as they
        # are by the bf16 path: no layout pass around the kernels.  Default: follow the input's memory format.
        self.memory_format = torch.channels_last if ndim == 2 else torch.channels_last_3d
        if channels_last is None:
            channels_last = (not x.is_contiguous()) and x.is_contiguous(memory_format=self.memory_format)
        mk = lambda pr: _lib.make_problem(ndim, x.dtype, x.size(0), x.size(1), weight.size(0), tuple(x.shape[2:]),
                                          tuple(weight.shape[2:]), stride, padding, dilation, group, cpg,
                                          deformable, std_size_rule, oob_offset_grad, pr,
                                          channels_last and pr == _lib.PREC_BF16)
        if prec == "auto":
            # bf16 tensor-core path where the shape allows it and the problem is big enough to pay for its
            # layout pre-passes (ten launches per step against three of the exact path)
            kvol = int(torch.Size(weight.shape[2:]).numel())
            out_guess = 1
            for i, k_, s_, p_ in zip(x.shape[2:], weight.shape[2:], _lib._triple(stride, ndim, 1)[3 - ndim:],
                                     _lib._triple(padding, ndim, 0)[3 - ndim:]):
                out_guess *= max(1, (i + 2 * p_ - k_) // s_ + 1)
            flops_per_pass = 2.0 * x.size(0) * weight.size(0) * weight.size(1) * kvol * out_guess
            p = mk(_lib.PREC_BF16) if (x.dtype == torch.float32 and flops_per_pass >= 1e8) else None
            if p is None or not _lib.lib().dcn_precision_supported(ctypes.byref(p)):
                p = mk(_lib.PREC_EXACT)
        elif prec in _PRECISIONS:
            p = mk(_PRECISIONS[prec])
        else:
            raise DcnError("unknown precision %r (exact | bf16 | auto)" % prec)
        _lib.check(_lib.lib().dcn_validate(ctypes.byref(p)), "shape check")
        if not _lib.lib().dcn_precision_supported(ctypes.byref(p)):
            raise DcnError("precision %r is not available for this problem (needs float32 tensors and channel "
                           "counts per group that are multiples of 8); there is no silent fallback" % prec)
        self.p = p
        self.channels_last = bool(p.channels_last)
        self.deformable = deformable
        self.out_size = _lib.output_size(p)
        self.offset_channels = (x.size(1) // cpg) * int(torch.Size(weight.shape[2:]).numel()) * ndim
        self.N, self.C, self.O = x.size(0), x.size(1), weight.size(0)
        self.weight_shape = tuple(weight.shape)

    # -- helpers ---------------------------------------------------------------------------------
    def _act(self, t: Optional[torch.Tensor], name: str, ref: Optional[torch.Tensor] = None) -> Optional[torch.Tensor]:
        """An activation-like tensor (input, output gradient) in the storage order the problem was built for."""
        t = _prep(t, name, ref) if not self.channels_last else t
        if t is None or not self.channels_last:
            return t
        if not t.is_cuda:
            raise DcnError("%s must be a CUDA tensor (there is no CPU implementation)" % name)
        if ref is not None and (t.device != ref.device or t.dtype != ref.dtype):
            raise DcnError("%s does not match the input's device / dtype" % name)
        return t.contiguous(memory_format=self.memory_format)

    def _new_act(self, shape, like: torch.Tensor, zero: bool = False) -> torch.Tensor:
        mf = self.memory_format if self.channels_last else torch.contiguous_format
        t = torch.empty(tuple(shape), dtype=like.dtype, device=like.device, memory_format=mf)
        return t.zero_() if zero else t

    def _ws(self, which: int):
        nbytes = _lib.lib().dcn_workspace_bytes(ctypes.byref(self.p), which)
        if nbytes == 0:
            return None, 0
        ws = torch.empty(nbytes, dtype=torch.uint8, device=self.device)
        return ws, nbytes

    def _check_offset(self, offset: torch.Tensor):
        want = (self.N, self.offset_channels) + tuple(self.out_size)
        if tuple(offset.shape) != want:
            raise DcnError("offset shape %s, expected %s" % (tuple(offset.shape), want))

    # -- passes ----------------------------------------------------------------------------------
    def backward(self, x, offset, weight, dy, want_dx=True, want_doffset=True, want_dw=True, want_dbias=False,
                 x_channels_last: Optional[torch.Tensor] = None):
        """All gradients through the fused entry point (outputs overwritten; scratch shared between the data
        and weight kernels).  ``x_channels_last``: the forward workspace kept by :meth:`forward` (bf16 path)."""
        x = self._act(x, "input")
        weight = _prep(weight, "weight", x)
        dy = self._act(dy, "grad_output", x)
        offset = _prep(offset, "offset", x) if self.deformable else None
        if not self.deformable:
            want_doffset = False
        dx = self._new_act(x.shape, x) if want_dx else None
        doff = torch.empty_like(offset) if want_doffset else None
        dw = torch.empty(self.weight_shape, dtype=x.dtype, device=x.device) if want_dw else None
        db = torch.empty(self.O, dtype=x.dtype, device=x.device) if want_dbias else None
        ws, nb = self._ws(_lib.PASS_BACKWARD)
        with torch.cuda.device(x.device), _Range("dcn_backward"):
            st = _lib.lib().dcn_backward(ctypes.byref(self.p), _lib.ptr(x), _lib.ptr(offset), _lib.ptr(weight),
                                         _lib.ptr(dy), _lib.ptr(x_channels_last), _lib.ptr(dx), _lib.ptr(doff),
                                         _lib.ptr(dw), _lib.ptr(db), _lib.ptr(ws), nb, _lib.current_stream(x.device))
        _lib.check(st, "dcn_backward")
        return dx, doff, dw, db

    def forward(self, x, offset, weight, bias=None, keep_workspace: bool = False):
        x = self._act(x, "input")
        weight = _prep(weight, "weight", x)
        bias = _prep(bias, "bias", x)
        if self.deformable:
            offset = _prep(offset, "offset", x)
            self._check_offset(offset)
        else:
            offset = None
        y = self._new_act((self.N, self.O) + tuple(self.out_size), x)
        ws, nb = self._ws(_lib.PASS_FORWARD)
        with torch.cuda.device(x.device), _Range("dcn_forward"):
            st = _lib.lib().dcn_forward(ctypes.byref(self.p), _lib.ptr(x), _lib.ptr(offset), _lib.ptr(weight),
                                        _lib.ptr(bias), _lib.ptr(y), _lib.ptr(ws), nb, _lib.current_stream(x.device))
        _lib.check(st, "dcn_forward")
        if keep_workspace:
            # the channels-last bf16 copy of x sits at the start of the workspace; backward can take it over
            return y, ws
        return y

    def backward_data(self, x, offset, weight, dy, want_dx=True, want_doffset=True
                      ) -> Tuple[Optional[torch.Tensor], Optional[torch.Tensor]]:
        weight = _prep(weight, "weight")
        dy = self._act(dy, "grad_output", weight)
        dx = doff = None
        if self.deformable:
            x = self._act(x, "input", weight)
            offset = _prep(offset, "offset", weight)
            self._check_offset(offset)
        else:
            offset = None
            want_doffset = False
        if want_dx:
            dx = self._new_act((self.N, self.C) + tuple(self.p.in_)[3 - self.ndim:], dy, zero=True)
        if want_doffset:
            doff = torch.empty((self.N, self.offset_channels) + tuple(self.out_size), dtype=dy.dtype, device=dy.device)
        if dx is None and doff is None:
            return None, None
        ws, nb = self._ws(_lib.PASS_BACKWARD_DATA)
        with torch.cuda.device(dy.device), _Range("dcn_backward_data"):
            st = _lib.lib().dcn_backward_data(ctypes.byref(self.p), _lib.ptr(x) if self.deformable else None,
                                              _lib.ptr(offset), _lib.ptr(weight), _lib.ptr(dy), _lib.ptr(dx),
                                              _lib.ptr(doff), _lib.ptr(ws), nb, _lib.current_stream(dy.device))
        _lib.check(st, "dcn_backward_data")
        return dx, doff

    def backward_weight(self, x, offset, dy, want_dw=True, want_dbias=False
                        ) -> Tuple[Optional[torch.Tensor], Optional[torch.Tensor]]:
        x = self._act(x, "input")
        dy = self._act(dy, "grad_output", x)
        offset = _prep(offset, "offset", x) if self.deformable else None
        dw = torch.zeros(self.weight_shape, dtype=x.dtype, device=x.device) if want_dw else None
        db = torch.empty(self.O, dtype=x.dtype, device=x.device) if want_dbias else None
        if dw is None and db is None:
            return None, None
        ws, nb = self._ws(_lib.PASS_BACKWARD_WEIGHT) if want_dw else (None, 0)
        with torch.cuda.device(x.device), _Range("dcn_backward_weight"):
            st = _lib.lib().dcn_backward_weight(ctypes.byref(self.p), _lib.ptr(x), _lib.ptr(offset), _lib.ptr(dy),
                                                _lib.ptr(dw), _lib.ptr(db), _lib.ptr(ws), nb,
                                                _lib.current_stream(x.device))
        _lib.check(st, "dcn_backward_weight")
        return dw, db

    # -- deformable layer: offset-producing convolution + deformable convolution in one call -------------------
    def offset_weight_shape(self):
        """Weight shape of the convolution that produces this operator's offsets: [dg*kv*D, C, k...]."""
        return (self.offset_channels, self.C) + tuple(self.weight_shape[2:])

    def _layer_ws(self, which: int):
        nbytes = _lib.lib().dcn_layer_workspace_bytes(ctypes.byref(self.p), which)
        if nbytes == 0:
            return None, 0
        return torch.empty(nbytes, dtype=torch.uint8, device=self.device), nbytes

    def layer_forward(self, x, offset_weight, offset_bias, weight, bias=None, keep_workspace: bool = False):
        """offset = conv(x, offset_weight) + offset_bias; y = deform_conv(x, offset, weight) + bias.
        Returns (y, offset[, workspace])."""
        if not self.deformable:
            raise DcnError("the layer entry points need a deformable operator")
        x = self._act(x, "input")
        weight = _prep(weight, "weight", x)
        bias = _prep(bias, "bias", x)
        offset_weight = _prep(offset_weight, "offset_weight", x)
        offset_bias = _prep(offset_bias, "offset_bias", x)
        if tuple(offset_weight.shape) != self.offset_weight_shape():
            raise DcnError("offset_weight shape %s, expected %s" % (tuple(offset_weight.shape),
                                                                    self.offset_weight_shape()))
        y = self._new_act((self.N, self.O) + tuple(self.out_size), x)
        offset = torch.empty((self.N, self.offset_channels) + tuple(self.out_size), dtype=x.dtype, device=x.device)
        ws, nb = self._layer_ws(_lib.PASS_FORWARD)
        with torch.cuda.device(x.device), _Range("dcn_layer_forward"):
            st = _lib.lib().dcn_layer_forward(ctypes.byref(self.p), _lib.ptr(x), _lib.ptr(offset_weight),
                                              _lib.ptr(offset_bias), _lib.ptr(weight), _lib.ptr(bias), _lib.ptr(offset),
                                              _lib.ptr(y), _lib.ptr(ws), nb, _lib.current_stream(x.device))
        _lib.check(st, "dcn_layer_forward")
        return (y, offset, ws) if keep_workspace else (y, offset)

    def layer_backward(self, x, offset, offset_weight, weight, dy, want_dx=True, want_dow=True, want_dob=False,
                       want_dw=True, want_dbias=False, x_channels_last: Optional[torch.Tensor] = None):
        """Gradients of the layer: (dx, doffset_weight, doffset_bias, dweight, dbias); dx includes the path
        through the offsets."""
        x = self._act(x, "input")
        weight = _prep(weight, "weight", x)
        offset_weight = _prep(offset_weight, "offset_weight", x)
        offset = _prep(offset, "offset", x)
        self._check_offset(offset)
        dy = self._act(dy, "grad_output", x)
        dx = self._new_act(x.shape, x) if want_dx else None
        dow = torch.empty_like(offset_weight) if want_dow else None
        dob = torch.empty(self.offset_channels, dtype=x.dtype, device=x.device) if want_dob else None
        dw = torch.empty(self.weight_shape, dtype=x.dtype, device=x.device) if want_dw else None
        db = torch.empty(self.O, dtype=x.dtype, device=x.device) if want_dbias else None
        ws, nb = self._layer_ws(_lib.PASS_BACKWARD)
        with torch.cuda.device(x.device), _Range("dcn_layer_backward"):
            st = _lib.lib().dcn_layer_backward(ctypes.byref(self.p), _lib.ptr(x), _lib.ptr(offset),
                                               _lib.ptr(offset_weight), _lib.ptr(weight), _lib.ptr(dy),
                                               _lib.ptr(x_channels_last), _lib.ptr(dx), _lib.ptr(dow), _lib.ptr(dob),
                                               _lib.ptr(dw), _lib.ptr(db), _lib.ptr(ws), nb,
                                               _lib.current_stream(x.device))
        _lib.check(st, "dcn_layer_backward")
        return dx, dow, dob, dw, db

    def debug_tc_points(self, offset: torch.Tensor, n: int):
        """Coordinates / validity / corner indices of sample ``n`` decoded from the sampling-point entries that the
        tensor-core backward-data kernel of the 2-D deformable operator consumes (bf16 precision)."""
        offset = _prep(offset, "offset")
        dg, kv, ov = self.C // self.p.cpg, self.offset_channels // (self.C // self.p.cpg) // self.ndim, 1
        for s in self.out_size:
            ov *= s
        coords = torch.empty((dg, kv, ov, self.ndim), dtype=offset.dtype, device=offset.device)
        valid = torch.empty((dg, kv, ov), dtype=torch.int32, device=offset.device)
        lo = torch.empty((dg, kv, ov, self.ndim), dtype=torch.int32, device=offset.device)
        hi = torch.empty_like(lo)
        ws, nb = self._ws(_lib.PASS_BACKWARD)
        with torch.cuda.device(offset.device), _Range("dcn_debug_tc_points"):
            st = _lib.lib().dcn_debug_tc_points(ctypes.byref(self.p), _lib.ptr(offset), n, _lib.ptr(coords),
                                                _lib.ptr(valid), _lib.ptr(lo), _lib.ptr(hi), _lib.ptr(ws), nb,
                                                _lib.current_stream(offset.device))
        _lib.check(st, "dcn_debug_tc_points")
        return coords, valid, lo, hi

    def debug_points(self, offset: torch.Tensor, n: int):
        """Coordinates / validity / corner indices of sample ``n`` as the device routine computes them."""
        offset = _prep(offset, "offset")
        dg, kv, ov = self.C // self.p.cpg, self.offset_channels // (self.C // self.p.cpg) // self.ndim, 1
        for s in self.out_size:
            ov *= s
        coords = torch.empty((dg, kv, ov, self.ndim), dtype=offset.dtype, device=offset.device)
        valid = torch.empty((dg, kv, ov), dtype=torch.int32, device=offset.device)
        lo = torch.empty((dg, kv, ov, self.ndim), dtype=torch.int32, device=offset.device)
        hi = torch.empty_like(lo)
        with torch.cuda.device(offset.device), _Range("dcn_debug_points"):
            st = _lib.lib().dcn_debug_points(ctypes.byref(self.p), _lib.ptr(offset), n, _lib.ptr(coords),
                                             _lib.ptr(valid), _lib.ptr(lo), _lib.ptr(hi),
                                             _lib.current_stream(offset.device))
        _lib.check(st, "dcn_debug_points")
        return coords, valid, lo, hi
