"""TEST INFRASTRUCTURE ONLY -- the checker, never the product.

CPU restatement of the reference operator, used by the tests, by the smoke check and by the
CPU-baseline leg of the benchmark.  The shipped operator never imports this module.

The per-sample device kernels are restated in ``dcn_oracle.cpp`` (loaded here through ctypes);
this file restates the reference's host launchers, i.e. the serial loop over the batch, the
per-group split and the three GEMMs (paths relative to the reference project root):

* forward            deform3d/lib/deform_conv3d_cuda.cpp:90-165   (im2col, then y_j = W_j . col_j)
* backward to input  deform3d/lib/deform_conv3d_cuda.cpp:168-262  (col_j = W_j^T . dy_j, then the
  and offset                                                       offset kernel, then the input kernel)
* backward to weight deform3d/lib/deform_conv3d_cuda.cpp:265-336  (im2col again, dW_j += dy_j . col_j^T)
* 2-D fp64 twin      deform2d_double/lib/deform_conv2d_cuda.cpp:82-325
* 2-D fp32 (legacy)  deform2d/lib/deform_conv2d_cuda.cpp:82-235   (no groups, no dilation)
* plain 2-D conv     conv2d/lib/conv2d_cuda.cpp:77-290
* output size rule   deform3d/lib/deform_conv3d_cuda.cpp:15-17 (dilation ignored) versus
                     conv2d/lib/conv2d_cuda.cpp:20-22 (dilation-aware)
* bias add / grad    deform3d/deform_conv3d_functions/deform_conv3d_function.py:41-42, 73-74

The GEMMs are numpy matmuls in the tensor dtype (fp32 -> SGEMM, fp64 -> DGEMM), which is what
the reference asks of cuBLAS.  Parity pins: the committed vectors under ``tests/golden`` were
produced by the reference's own device kernels (built from the reference checkout into
``oracle/_ref`` and run on a B200, see ``tests/golden/make_golden.py``); the oracle is checked
against them and against independent properties (zero offsets == ordinary convolution, interior
offsets == torchvision's deform_conv2d, finite differences in fp64).
"""
from __future__ import annotations

import ctypes
import os
import subprocess
from dataclasses import dataclass, field
from typing import Optional, Sequence, Tuple

import numpy as np

_HERE = os.path.dirname(os.path.abspath(__file__))
_LIB_PATH = os.path.join(_HERE, "liboracle.so")
_lib = None


def build(force: bool = False) -> str:
    """Compile ``liboracle.so`` (and ``oracle/_ref`` when the reference checkout is present)."""
    if force or not os.path.exists(_LIB_PATH) or (
            os.path.getmtime(_LIB_PATH) < os.path.getmtime(os.path.join(_HERE, "dcn_oracle.cpp"))):
        subprocess.check_call(["make", "-s", "-f", os.path.join(_HERE, "Makefile"), "all"], cwd=_HERE)
    return _LIB_PATH


def lib() -> ctypes.CDLL:
    global _lib
    if _lib is None:
        if not os.path.exists(_LIB_PATH):
            build()
        _lib = ctypes.CDLL(_LIB_PATH)
    return _lib


@dataclass
class Problem:
    """Geometry of one call.  2-D problems give 2-tuples; they are padded with a unit axis."""
    ndim: int
    N: int
    C: int
    O: int
    in_size: Sequence[int]
    kernel: Sequence[int]
    stride: Sequence[int] = (1, 1, 1)
    pad: Sequence[int] = (0, 0, 0)
    dil: Sequence[int] = (1, 1, 1)
    G: int = 1
    cpg: int = 1                 # channels per deformable group (the reference's channel_per_group)
    deformable: bool = True
    std_size_rule: bool = False  # True: dilation-aware output size (plain conv2d package)
    oob_offset_grad: bool = True  # 3-D only: the reference's pull-back term for invalid samples
    out_size: Tuple[int, ...] = field(init=False)

    def __post_init__(self):
        nd = self.ndim
        assert nd in (2, 3)

        def tup(v):
            v = tuple(int(a) for a in (v if isinstance(v, (tuple, list)) else (v,) * nd))
            return v[-nd:] if len(v) >= nd else v

        self.in_size, self.kernel = tup(self.in_size), tup(self.kernel)
        self.stride, self.pad, self.dil = tup(self.stride), tup(self.pad), tup(self.dil)
        out = []
        for i in range(nd):
            if self.std_size_rule:
                out.append((self.in_size[i] + 2 * self.pad[i] - self.dil[i] * (self.kernel[i] - 1) - 1)
                           // self.stride[i] + 1)
            else:
                out.append((self.in_size[i] + 2 * self.pad[i] - self.kernel[i]) // self.stride[i] + 1)
        self.out_size = tuple(out)

    # 3-slot views (leading unit axis for 2-D)
    def _p3(self, v, fill):
        return (fill,) * (3 - self.ndim) + tuple(v)

    @property
    def kv(self):
        return int(np.prod(self.kernel))

    @property
    def ov(self):
        return int(np.prod(self.out_size))

    @property
    def iv(self):
        return int(np.prod(self.in_size))

    @property
    def offset_channels(self):
        return (self.C // self.cpg) * self.kv * self.ndim

    def geo_args(self):
        i3 = lambda v, f: (ctypes.c_int * 3)(*self._p3(v, f))
        return (ctypes.c_int(self.ndim), ctypes.c_int(self.C), i3(self.in_size, 1), i3(self.out_size, 1),
                i3(self.kernel, 1), i3(self.pad, 0), i3(self.stride, 1), i3(self.dil, 1),
                ctypes.c_int(self.cpg))


def _sfx(dtype):
    dtype = np.dtype(dtype)
    if dtype == np.float32:
        return "f32"
    if dtype == np.float64:
        return "f64"
    raise TypeError("oracle supports float32 / float64, got %s" % dtype)


def _ptr(a: np.ndarray):
    assert a.flags["C_CONTIGUOUS"]
    return ctypes.c_void_p(a.ctypes.data)


def im2col(p: Problem, x_n: np.ndarray, off_n: Optional[np.ndarray]) -> np.ndarray:
    col = np.empty((p.C * p.kv, p.ov), dtype=x_n.dtype)
    s = _sfx(x_n.dtype)
    if p.deformable:
        getattr(lib(), "orc_deform_im2col_" + s)(*p.geo_args(), _ptr(x_n), _ptr(off_n), _ptr(col))
    else:
        getattr(lib(), "orc_im2col_" + s)(*p.geo_args(), _ptr(x_n), _ptr(col))
    return col


def col2im_input(p: Problem, col: np.ndarray, off_n: Optional[np.ndarray], dx_n: np.ndarray) -> None:
    s = _sfx(col.dtype)
    if p.deformable:
        getattr(lib(), "orc_deform_col2im_input_" + s)(*p.geo_args(), _ptr(col), _ptr(off_n), _ptr(dx_n))
    else:
        getattr(lib(), "orc_col2im_" + s)(*p.geo_args(), _ptr(col), _ptr(dx_n))


def col2im_offset(p: Problem, col: np.ndarray, x_n: np.ndarray, off_n: np.ndarray, doff_n: np.ndarray) -> None:
    s = _sfx(col.dtype)
    oob = 1 if (p.oob_offset_grad and p.ndim == 3) else 0
    getattr(lib(), "orc_deform_col2im_offset_" + s)(*p.geo_args(), _ptr(col), _ptr(x_n), _ptr(off_n),
                                                   ctypes.c_int(oob), _ptr(doff_n))


def dump_points(p: Problem, off_n: np.ndarray):
    """(coords [dg,kv,ov,nd], valid [dg,kv,ov], lo [dg,kv,ov,nd], hi [...]) for one sample."""
    dg = p.C // p.cpg
    shp = (dg, p.kv, p.ov)
    pts = np.empty(shp + (p.ndim,), dtype=off_n.dtype)
    valid = np.empty(shp, dtype=np.int32)
    lo = np.empty(shp + (p.ndim,), dtype=np.int32)
    hi = np.empty(shp + (p.ndim,), dtype=np.int32)
    getattr(lib(), "orc_dump_points_" + _sfx(off_n.dtype))(*p.geo_args(), _ptr(off_n), _ptr(pts), _ptr(valid),
                                                           _ptr(lo), _ptr(hi))
    return pts, valid, lo, hi


def _c(a, dtype=None):
    return np.ascontiguousarray(a, dtype=dtype)


def forward(p: Problem, x, offset, weight, bias=None) -> np.ndarray:
    """y[n] = W . im2col(x[n], offset[n]) per group, plus bias (broadcast)."""
    x, weight = _c(x), _c(weight)
    dt = x.dtype
    y = np.zeros((p.N, p.O) + p.out_size, dtype=dt)
    Kg, Og = (p.C // p.G) * p.kv, p.O // p.G
    Wg = weight.reshape(p.G, Og, Kg)
    for n in range(p.N):
        col = im2col(p, _c(x[n]), _c(offset[n]) if p.deformable else None).reshape(p.G, Kg, p.ov)
        yn = y[n].reshape(p.G, Og, p.ov)
        for j in range(p.G):
            yn[j] = Wg[j] @ col[j]
    if bias is not None:
        y += np.asarray(bias, dtype=dt).reshape((1, -1) + (1,) * p.ndim)
    return y


def backward_data(p: Problem, x, offset, weight, dy):
    """(dx, doffset).  dx accumulates into zeros, doffset is overwritten, as in the reference."""
    x, weight, dy = _c(x), _c(weight), _c(dy)
    dt = x.dtype
    dx = np.zeros_like(x)
    doff = np.zeros((p.N, p.offset_channels) + p.out_size, dtype=dt) if p.deformable else None
    Kg, Og = (p.C // p.G) * p.kv, p.O // p.G
    Wg = weight.reshape(p.G, Og, Kg)
    for n in range(p.N):
        dyn = dy[n].reshape(p.G, Og, p.ov)
        col = np.empty((p.G, Kg, p.ov), dtype=dt)
        for j in range(p.G):
            col[j] = Wg[j].T @ dyn[j]
        col = col.reshape(p.C * p.kv, p.ov)
        if p.deformable:
            off_n = _c(offset[n])
            col2im_offset(p, col, _c(x[n]), off_n, doff[n])
            col2im_input(p, col, off_n, dx[n])
        else:
            col2im_input(p, col, None, dx[n])
    return dx, doff


def backward_weight(p: Problem, x, offset, dy) -> np.ndarray:
    x, dy = _c(x), _c(dy)
    dt = x.dtype
    Kg, Og = (p.C // p.G) * p.kv, p.O // p.G
    dW = np.zeros((p.G, Og, Kg), dtype=dt)
    for n in range(p.N):
        col = im2col(p, _c(x[n]), _c(offset[n]) if p.deformable else None).reshape(p.G, Kg, p.ov)
        dyn = dy[n].reshape(p.G, Og, p.ov)
        for j in range(p.G):
            dW[j] += dyn[j] @ col[j].T
    return dW.reshape((p.O, p.C // p.G) + tuple(p.kernel))


def backward_bias(p: Problem, dy) -> np.ndarray:
    return np.asarray(dy).sum(axis=(0,) + tuple(range(2, 2 + p.ndim)))


def fwd_bwd(p: Problem, x, offset, weight, dy, bias=None):
    """One full pass (all gradients), the unit the benchmark times."""
    y = forward(p, x, offset, weight, bias)
    dx, doff = backward_data(p, x, offset, weight, dy)
    dw = backward_weight(p, x, offset, dy)
    return y, dx, doff, dw
