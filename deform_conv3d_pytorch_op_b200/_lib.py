"""ctypes binding of ``csrc/libdcn.so`` (the C ABI declared in ``include/dcn.h``).

There is no CPU implementation and no fallback: if the library is missing or a call fails, an
exception is raised.
"""
from __future__ import annotations

import ctypes
import os
from typing import Optional, Sequence

import torch

_HERE = os.path.dirname(os.path.abspath(__file__))
LIB_PATH = os.path.join(_HERE, "csrc", "libdcn.so")

DCN_F32, DCN_F64 = 0, 1
PREC_EXACT, PREC_BF16 = 0, 1
PASS_FORWARD, PASS_BACKWARD_DATA, PASS_BACKWARD_WEIGHT, PASS_BACKWARD = 0, 1, 2, 3


class DcnError(RuntimeError):
    """Raised where the reference would have raised through THError (shape_check) or on a CUDA failure."""


class dcn_problem(ctypes.Structure):
    _fields_ = [
        ("ndim", ctypes.c_int32), ("dtype", ctypes.c_int32), ("precision", ctypes.c_int32),
        ("deformable", ctypes.c_int32), ("std_size_rule", ctypes.c_int32), ("oob_offset_grad", ctypes.c_int32),
        ("N", ctypes.c_int32), ("C", ctypes.c_int32), ("O", ctypes.c_int32), ("G", ctypes.c_int32),
        ("cpg", ctypes.c_int32),
        ("in_", ctypes.c_int32 * 3), ("k", ctypes.c_int32 * 3), ("stride", ctypes.c_int32 * 3),
        ("pad", ctypes.c_int32 * 3), ("dil", ctypes.c_int32 * 3),
        ("channels_last", ctypes.c_int32),
    ]


_lib: Optional[ctypes.CDLL] = None

# every symbol include/dcn.h declares (checked by the CPU test-suite)
GENERIC_SYMBOLS = [
    "dcn_version", "dcn_status_string", "dcn_output_size", "dcn_validate", "dcn_precision_supported",
    "dcn_workspace_bytes", "dcn_launch_count", "dcn_forward", "dcn_backward_data", "dcn_backward_weight", "dcn_backward", "dcn_debug_points",
    "dcn_debug_tc_points", "dcn_debug_expire_wait",
    "dcn_check_status", "dcn_static_scratch_bytes", "dcn_forward_static_scratch",
    "dcn_offset_conv_problem", "dcn_layer_workspace_bytes", "dcn_layer_forward", "dcn_layer_backward", "dcn_layer_launch_count",
]
LEGACY_SYMBOLS = [
    "dcn_deform3d_deform_conv_forward_cuda", "dcn_deform3d_deform_conv_backward_input_offset_cuda",
    "dcn_deform3d_deform_conv_backward_weight_cuda",
    "dcn_deform2d_deform_conv_forward_cuda", "dcn_deform2d_deform_conv_backward_input_offset_cuda",
    "dcn_deform2d_deform_conv_backward_weight_cuda",
    "dcn_deform2d_double_deform_conv_forward_cuda", "dcn_deform2d_double_deform_conv_backward_input_offset_cuda",
    "dcn_deform2d_double_deform_conv_backward_weight_cuda",
    "dcn_conv2d_conv_forward_cuda", "dcn_conv2d_conv_backward_input_cuda", "dcn_conv2d_conv_backward_weight_cuda",
]


def lib() -> ctypes.CDLL:
    """Load libdcn.so (once).  Fails loudly when it has not been built."""
    global _lib
    if _lib is None:
        if not os.path.exists(LIB_PATH):
            raise DcnError(
                "libdcn.so is missing (%s): build it with `python -m deform_conv3d_pytorch_op_b200.build`; "
                "there is no fallback implementation" % LIB_PATH)
        L = ctypes.CDLL(LIB_PATH)
        vp, pp = ctypes.c_void_p, ctypes.POINTER(dcn_problem)
        L.dcn_version.restype = ctypes.c_int
        L.dcn_status_string.restype = ctypes.c_char_p
        L.dcn_status_string.argtypes = [ctypes.c_int]
        L.dcn_output_size.argtypes = [pp, ctypes.POINTER(ctypes.c_int32)]
        L.dcn_validate.argtypes = [pp]
        L.dcn_precision_supported.argtypes = [pp]
        L.dcn_workspace_bytes.restype = ctypes.c_size_t
        L.dcn_workspace_bytes.argtypes = [pp, ctypes.c_int]
        L.dcn_launch_count.argtypes = [pp, ctypes.c_int]
        L.dcn_forward.argtypes = [pp, vp, vp, vp, vp, vp, vp, ctypes.c_size_t, vp]
        L.dcn_backward_data.argtypes = [pp, vp, vp, vp, vp, vp, vp, vp, ctypes.c_size_t, vp]
        L.dcn_backward_weight.argtypes = [pp, vp, vp, vp, vp, vp, vp, ctypes.c_size_t, vp]
        L.dcn_backward.argtypes = [pp, vp, vp, vp, vp, vp, vp, vp, vp, vp, vp, ctypes.c_size_t, vp]
        L.dcn_debug_points.argtypes = [pp, vp, ctypes.c_int32, vp, vp, vp, vp, vp]
        L.dcn_debug_tc_points.argtypes = [pp, vp, ctypes.c_int32, vp, vp, vp, vp, vp, ctypes.c_size_t, vp]
        L.dcn_debug_expire_wait.argtypes = [vp, vp]
        L.dcn_check_status.argtypes = [vp]
        L.dcn_static_scratch_bytes.restype = ctypes.c_size_t
        L.dcn_forward_static_scratch.argtypes = [pp, vp, vp, vp, vp, vp, vp]
        L.dcn_offset_conv_problem.argtypes = [pp, pp]
        L.dcn_layer_workspace_bytes.restype = ctypes.c_size_t
        L.dcn_layer_workspace_bytes.argtypes = [pp, ctypes.c_int]
        L.dcn_layer_launch_count.argtypes = [pp, ctypes.c_int]
        L.dcn_layer_forward.argtypes = [pp, vp, vp, vp, vp, vp, vp, vp, vp, ctypes.c_size_t, vp]
        L.dcn_layer_backward.argtypes = [pp, vp, vp, vp, vp, vp, vp, vp, vp, vp, vp, vp, vp, ctypes.c_size_t, vp]
        _lib = L
    return _lib


def check(status: int, what: str = "") -> None:
    if status != 0:
        raise DcnError("%s failed: %s (status %d)" % (what or "libdcn call", lib().dcn_status_string(status).decode(),
                                                       status))


def _triple(v, ndim: int, fill: int):
    if isinstance(v, int):
        v = (v,) * ndim
    v = tuple(int(a) for a in v)
    if len(v) != ndim:
        raise DcnError("expected %d values, got %r" % (ndim, v))
    return (fill,) * (3 - ndim) + v


def make_problem(ndim: int, dtype: torch.dtype, N: int, C: int, O: int, in_size: Sequence[int],
                 kernel: Sequence[int], stride, pad, dil, G: int, cpg: int, deformable: bool = True,
                 std_size_rule: bool = False, oob_offset_grad: bool = True,
                 precision: int = PREC_EXACT, channels_last: bool = False) -> dcn_problem:
    p = dcn_problem()
    p.ndim = ndim
    if dtype == torch.float32:
        p.dtype = DCN_F32
    elif dtype == torch.float64:
        p.dtype = DCN_F64
    else:
        raise DcnError("tensors must be float32 or float64, got %s" % dtype)
    p.precision = precision
    p.deformable = 1 if deformable else 0
    p.std_size_rule = 1 if std_size_rule else 0
    p.oob_offset_grad = 1 if oob_offset_grad else 0
    p.N, p.C, p.O, p.G, p.cpg = int(N), int(C), int(O), int(G), int(cpg)
    p.in_[:] = _triple(in_size, ndim, 1)
    p.k[:] = _triple(kernel, ndim, 1)
    p.stride[:] = _triple(stride, ndim, 1)
    p.pad[:] = _triple(pad, ndim, 0)
    p.dil[:] = _triple(dil, ndim, 1)
    p.channels_last = 1 if channels_last else 0
    return p


def output_size(p: dcn_problem):
    out = (ctypes.c_int32 * 3)()
    check(lib().dcn_output_size(ctypes.byref(p), out), "dcn_output_size")
    return tuple(out)[3 - p.ndim:]


def ptr(t: Optional[torch.Tensor]):
    return None if t is None else ctypes.c_void_p(t.data_ptr())


def current_stream(device) -> ctypes.c_void_p:
    return ctypes.c_void_p(torch.cuda.current_stream(device).cuda_stream)
