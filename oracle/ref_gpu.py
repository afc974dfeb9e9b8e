"""TEST INFRASTRUCTURE ONLY.  Drives the reference's own device kernels (compiled unmodified from the
reference checkout into ``oracle/_ref/libref_*.so`` by ``oracle/Makefile``) on a CUDA device, with the
reference's host loops restated around them: serial over the batch, per group, GEMMs by ``torch.mm`` in the
tensor dtype where the reference calls cuBLAS (deform3d/lib/deform_conv3d_cuda.cpp:105-158, 186-253,
278-330 and the 2-D / plain-conv twins).  Used to produce the committed golden vectors and, on a GPU box,
to pin the CPU oracle against the real reference kernels.  The reference launches on the legacy default
stream, so every call here is bracketed by device synchronisation.
"""
from __future__ import annotations

import ctypes
import os

import torch

_HERE = os.path.dirname(os.path.abspath(__file__))
_REF = os.path.join(_HERE, "_ref")
_libs = {}


def available() -> bool:
    return all(os.path.exists(os.path.join(_REF, "libref_%s.so" % n))
               for n in ("deform3d", "deform2d", "deform2d_double", "conv2d"))


def _lib(name):
    if name not in _libs:
        _libs[name] = ctypes.CDLL(os.path.join(_REF, "libref_%s.so" % name))
    return _libs[name]


def _i3(v):
    return (ctypes.c_int * len(v))(*[int(a) for a in v])


def _p(t):
    return ctypes.c_void_p(t.data_ptr())


class RefOp:
    """variant: 'deform3d' (fp32), 'deform2d' (fp32, dilation must be 1, G must be 1), 'deform2d_double'
    (fp64), 'conv2d' (fp32 plain)."""

    def __init__(self, variant, prob):
        self.v = variant
        self.p = prob          # oracle.Problem
        self.lib = _lib(variant)
        if variant == "deform2d":
            assert tuple(prob.dil) == (1, 1) and prob.G == 1
        self.dtype = torch.float64 if variant == "deform2d_double" else torch.float32

    # --- kernel calls on one sample -------------------------------------------------------------------
    def _geo(self):
        p = self.p
        return _i3(p.in_size), _i3(p.out_size), _i3(p.kernel), _i3(p.pad), _i3(p.stride), _i3(p.dil)

    def _sync(self, rc):
        assert rc == 0, "reference kernel launch failed: %d" % rc
        torch.cuda.synchronize()

    def im2col(self, x_n, off_n):
        p = self.p
        col = torch.empty(p.C * p.kv, p.ov, dtype=self.dtype, device=x_n.device)
        i, o, k, pad, s, d = self._geo()
        torch.cuda.synchronize()
        if self.v == "deform3d":
            rc = self.lib.ref3d_im2col(_p(x_n), _p(off_n), p.C, i, o, k, pad, s, d, p.cpg, _p(col))
        elif self.v == "deform2d":
            rc = self.lib.ref2d_im2col(_p(x_n), _p(off_n), p.C, i, o, k, pad, s, p.cpg, _p(col))
        elif self.v == "deform2d_double":
            rc = self.lib.ref2dd_im2col(_p(x_n), _p(off_n), p.C, i, o, k, pad, s, d, p.cpg, _p(col))
        else:
            rc = self.lib.refc2d_im2col(_p(x_n), p.C, i, o, k, pad, s, d, _p(col))
        self._sync(rc)
        return col

    def col2im_input(self, col, off_n, dx_n):
        p = self.p
        i, o, k, pad, s, d = self._geo()
        torch.cuda.synchronize()
        if self.v == "deform3d":
            rc = self.lib.ref3d_col2im_input(_p(col), _p(off_n), p.C, i, o, k, pad, s, d, p.cpg, _p(dx_n))
        elif self.v == "deform2d":
            rc = self.lib.ref2d_col2im_input(_p(col), _p(off_n), p.C, i, o, k, pad, s, p.cpg, _p(dx_n))
        elif self.v == "deform2d_double":
            rc = self.lib.ref2dd_col2im_input(_p(col), _p(off_n), p.C, i, o, k, pad, s, d, p.cpg, _p(dx_n))
        else:
            rc = self.lib.refc2d_col2im(_p(col), p.C, i, o, k, pad, s, d, _p(dx_n))
        self._sync(rc)

    def col2im_offset(self, col, x_n, off_n, doff_n):
        p = self.p
        i, o, k, pad, s, d = self._geo()
        torch.cuda.synchronize()
        if self.v == "deform3d":
            rc = self.lib.ref3d_col2im_offset(_p(col), _p(x_n), _p(off_n), p.C, i, o, k, pad, s, d, p.cpg, _p(doff_n))
        elif self.v == "deform2d":
            rc = self.lib.ref2d_col2im_offset(_p(col), _p(x_n), _p(off_n), p.C, i, o, k, pad, s, p.cpg, _p(doff_n))
        else:
            rc = self.lib.ref2dd_col2im_offset(_p(col), _p(x_n), _p(off_n), p.C, i, o, k, pad, s, d, p.cpg,
                                               _p(doff_n))
        self._sync(rc)

    # --- the reference's host launchers ---------------------------------------------------------------
    def forward(self, x, off, w, bias=None):
        p = self.p
        Kg, Og = (p.C // p.G) * p.kv, p.O // p.G
        y = torch.zeros((p.N, p.O) + tuple(p.out_size), dtype=self.dtype, device=x.device)
        Wg = w.reshape(p.G, Og, Kg)
        for n in range(p.N):
            col = self.im2col(x[n].contiguous(), off[n].contiguous() if off is not None else None)
            col = col.view(p.G, Kg, p.ov)
            yn = y[n].view(p.G, Og, p.ov)
            for j in range(p.G):
                yn[j] = torch.mm(Wg[j], col[j])
        if bias is not None:
            y += bias.view((1, -1) + (1,) * p.ndim)
        return y

    def backward_data(self, x, off, w, dy):
        p = self.p
        Kg, Og = (p.C // p.G) * p.kv, p.O // p.G
        dx = torch.zeros_like(x)
        doff = torch.zeros_like(off) if off is not None else None
        Wg = w.reshape(p.G, Og, Kg)
        for n in range(p.N):
            dyn = dy[n].reshape(p.G, Og, p.ov)
            col = torch.empty(p.G, Kg, p.ov, dtype=self.dtype, device=x.device)
            for j in range(p.G):
                col[j] = torch.mm(Wg[j].t(), dyn[j])
            col = col.view(p.C * p.kv, p.ov)
            if off is not None:
                off_n = off[n].contiguous()
                self.col2im_offset(col, x[n].contiguous(), off_n, doff[n])
                self.col2im_input(col, off_n, dx[n])
            else:
                self.col2im_input(col, None, dx[n])
        return dx, doff

    def backward_weight(self, x, off, dy):
        p = self.p
        Kg, Og = (p.C // p.G) * p.kv, p.O // p.G
        dW = torch.zeros(p.G, Og, Kg, dtype=self.dtype, device=x.device)
        for n in range(p.N):
            col = self.im2col(x[n].contiguous(), off[n].contiguous() if off is not None else None).view(p.G, Kg, p.ov)
            dyn = dy[n].reshape(p.G, Og, p.ov)
            for j in range(p.G):
                dW[j] += torch.mm(dyn[j], col[j].t())
        return dW.view((p.O, p.C // p.G) + tuple(p.kernel))


def variant_for(case) -> str:
    """Which reference package serves a test case."""
    if not case.deformable:
        return "conv2d"
    if case.ndim == 3:
        return "deform3d"
    return "deform2d_double" if case.dtype == "float64" else "deform2d"
