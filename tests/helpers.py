"""Shared helpers of the GPU parity tests."""
from __future__ import annotations

import numpy as np
import torch

from oracle import oracle as orc
from tests import cases


def run_ours(case, tensors, precision="exact", oob=True, device="cuda"):
    """fwd + bwd through the public Functions (autograd) on the CUDA path; numpy results."""
    import deform_conv3d_pytorch_op_b200 as dcn
    x, w, off, dy, b = [None if t is None else t.to(device) for t in tensors]
    x = x.clone().requires_grad_(True)
    w = w.clone().requires_grad_(True)
    if b is not None:
        b = b.clone().requires_grad_(True)
    if case.deformable:
        off = off.clone().requires_grad_(True)
        fn = dcn.ConvOffset3dFunction if case.ndim == 3 else dcn.ConvOffset2dFunction
        y = fn.apply(x, off, w, b, case.stride, case.pad, case.dil, case.cpg, case.G, precision, oob)
    else:
        y = dcn.Conv2dFunction.apply(x, w, b, case.stride, case.pad, case.dil, case.G, precision)
    y.backward(dy)
    torch.cuda.synchronize()
    out = {"y": y.detach().cpu().numpy(), "dx": x.grad.cpu().numpy(), "dw": w.grad.cpu().numpy()}
    if case.deformable:
        out["doff"] = off.grad.cpu().numpy()
    if b is not None:
        out["db"] = b.grad.cpu().numpy()
    return out


def run_oracle(case, tensors, dtype=None, oob=True):
    """Same pass on the CPU oracle, optionally in another dtype (float64 = the tolerance oracle)."""
    x, w, off, dy, b = [None if t is None else t.numpy() for t in tensors]
    if dtype is not None:
        x, w, dy = x.astype(dtype), w.astype(dtype), dy.astype(dtype)
        off = None if off is None else off.astype(dtype)
        b = None if b is None else b.astype(dtype)
    p = case.problem(oob=oob)
    p.N = x.shape[0]
    out = {"y": orc.forward(p, x, off, w, b)}
    out["dx"], doff = orc.backward_data(p, x, off, w, dy)
    if doff is not None:
        out["doff"] = doff
    out["dw"] = orc.backward_weight(p, x, off, dy)
    if b is not None:
        out["db"] = orc.backward_bias(p, dy)
    return out


def lattice_mask(case, off_np, tol=1e-6):
    """True where the offset derivative is one-sided and the fp32 and float64 evaluations may legitimately pick
    different sides: some coordinate of the sampling point lies within tol of the integer lattice, or the
    fp32 coordinate (one rounding of base + offset) selects other corners than the float64 one.  Shape of doff."""
    p = case.problem()
    N = off_np.shape[0]
    p.N = N
    mask = np.zeros(off_np.shape, dtype=bool)
    nd = case.ndim
    for n in range(N):
        o32 = np.ascontiguousarray(off_np[n].astype(np.float32))
        pts, valid, lo, hi = orc.dump_points(p, o32)
        pts64, valid64, lo64, hi64 = orc.dump_points(p, o32.astype(np.float64))
        frac = np.abs(pts64 - np.round(pts64))
        near = (frac < tol).any(axis=-1)            # [dg, kv, ov]
        near |= (valid != valid64)
        both = (valid != 0) & (valid64 != 0)
        near |= both & ((lo != lo64).any(axis=-1) | (hi != hi64).any(axis=-1))
        near = np.repeat(near[:, :, None, :], nd, axis=2).reshape((-1,) + tuple(p.out_size))
        mask[n] = near
    return mask


def offsets_at_fp32_coordinates(case, off_np):
    """float64 offsets that make a float64 evaluation sample at exactly the coordinates the reference's fp32
    arithmetic produces: p32 = fp32(base) + off32 (one fp32 rounding, deform3d/lib/deform_conv3d_cuda_kernel.cu:
    117-119), returned as p32 - base in float64 (exact).  Validity (p > -1, p < size) and the truncation to corner
    indices are discontinuous in p, so a float64 oracle fed the raw offsets disagrees with ANY fp32 implementation,
    the reference included, at the few points whose fp32 coordinate rounds onto -1, size or an integer; with these
    offsets the oracle takes the reference's decisions and does everything else in float64."""
    p = case.problem()
    nd = case.ndim
    out_sz, k = tuple(p.out_size), tuple(p.kernel)
    kv = int(np.prod(k))
    N = off_np.shape[0]
    dg = off_np.shape[1] // (kv * nd)
    off32 = off_np.astype(np.float32).reshape((N, dg, kv, nd) + out_sz)
    res = np.empty(off32.shape, dtype=np.float64)
    taps = np.stack(np.unravel_index(np.arange(kv), k), axis=-1)             # [kv, nd]
    for a in range(nd):
        o = np.arange(out_sz[a], dtype=np.int64) * p.stride[a] - p.pad[a]     # [out_a]
        shape_o = [1] * nd
        shape_o[a] = out_sz[a]
        base = o.reshape(shape_o)[None, None, None] + (taps[:, a] * p.dil[a]).reshape((1, 1, kv) + (1,) * nd)
        p32 = base.astype(np.float32) + off32[:, :, :, a]
        res[:, :, :, a] = p32.astype(np.float64) - base
    return res.reshape(off_np.shape)
