"""Test cases: the input recipes of the reference's own test scripts, parameter corners, and the
benchmark configurations, with one seeded generator shared by the oracle and the CUDA path."""
from __future__ import annotations

from dataclasses import dataclass
from typing import Optional, Tuple

import numpy as np
import torch

from oracle import oracle as orc


@dataclass
class Case:
    name: str
    ndim: int
    N: int
    C: int
    O: int
    in_size: Tuple[int, ...]
    kernel: Tuple[int, ...]
    stride: Tuple[int, ...]
    pad: Tuple[int, ...]
    dil: Tuple[int, ...]
    G: int = 1
    cpg: int = 1
    dtype: str = "float32"
    deformable: bool = True
    bias: bool = False
    offset_std: float = 1.0        # offsets ~ N(0, std^2); "rand" recipe -> U(0,1) when offset_uniform
    offset_uniform: bool = False
    fixed: Optional[str] = None     # name of a hand-written recipe (see make_inputs)
    x_uniform01: bool = False       # inputs ~ U(0,1) like the reference's torch.rand recipes

    def problem(self, oob=True) -> orc.Problem:
        return orc.Problem(self.ndim, self.N, self.C, self.O, self.in_size, self.kernel, self.stride, self.pad,
                           self.dil, self.G, self.cpg, deformable=self.deformable,
                           std_size_rule=not self.deformable, oob_offset_grad=oob)


def _t(v, n):
    return (v,) * n


# --- recipes taken from the reference's test scripts (inputs only; the reference stores no outputs) -----
REFERENCE_RECIPES = [
    # deform3d/test_function.py:6-35: rows [1,1,1],[2,2,2],[1,1,1], zero offsets, ones weight, pad 1, dil 2
    Case("d3_test_function", 3, 1, 1, 1, _t(3, 3), _t(3, 3), _t(1, 3), _t(1, 3), _t(2, 3), 1, 1, fixed="d3_rows"),
    # deform3d/test_gradient.py:9-30
    Case("d3_test_gradient", 3, 2, 2, 4, _t(7, 3), _t(3, 3), _t(2, 3), _t(2, 3), _t(2, 3), 2, 2, bias=True,
         offset_uniform=True, x_uniform01=True),
    # deform3d/test_model.py:7-33 (k=1, no padding)
    Case("d3_test_model", 3, 2, 1, 1, _t(3, 3), _t(1, 3), _t(1, 3), _t(0, 3), _t(1, 3), 1, 1, offset_std=0.5),
    # deform2d_double/test_function.py:7-46: ones 3x3 input, 1x1 kernel, zero offsets, fp64
    Case("d2d_test_function", 2, 1, 1, 1, _t(3, 2), _t(1, 2), _t(1, 2), _t(0, 2), _t(1, 2), 1, 1, dtype="float64",
         fixed="ones"),
    # deform2d_double/test_gradient.py:7-53
    Case("d2d_test_gradient", 2, 2, 2, 4, _t(7, 2), _t(1, 2), _t(2, 2), _t(2, 2), _t(2, 2), 2, 2, dtype="float64",
         bias=True, offset_uniform=True, x_uniform01=True),
    # deform2d/test_gradient.py:11-51 (fp32 legacy API: no dilation, no groups)
    Case("d2_test_gradient", 2, 2, 2, 3, _t(7, 2), _t(1, 2), _t(2, 2), _t(1, 2), _t(1, 2), 1, 2,
         offset_uniform=True, x_uniform01=True),
    # deform2d/test_function.py:7-62: rand 5x5 input, zero offsets
    Case("d2_test_function", 2, 1, 1, 1, _t(5, 2), _t(3, 2), _t(1, 2), _t(1, 2), _t(1, 2), 1, 1, fixed="zero_off",
         x_uniform01=True),
    # conv2d/test_gradient.py:8-27
    Case("c2_test_gradient", 2, 2, 2, 4, _t(7, 2), _t(1, 2), _t(2, 2), _t(2, 2), _t(2, 2), 2, 2, deformable=False,
         bias=True, x_uniform01=True),
]

# --- parameter corners -------------------------------------------------------------------------------
CORNERS = [
    Case("d2_oob_heavy", 2, 2, 4, 6, (9, 11), (3, 3), (1, 1), (1, 1), (1, 1), 2, 2, offset_std=4.0, bias=True),
    Case("d2_k3_s2_d2_dg", 2, 3, 8, 8, (10, 9), (3, 3), (2, 1), (2, 1), (2, 2), 2, 2, offset_std=1.5),
    Case("d2_rect_kernel", 2, 2, 6, 4, (8, 12), (1, 3), (1, 2), (0, 1), (1, 1), 1, 3, offset_std=2.0),
    Case("d2_double_corner", 2, 2, 4, 4, (6, 7), (3, 2), (1, 1), (1, 1), (1, 2), 2, 1, dtype="float64",
         offset_std=2.0, bias=True),
    Case("d3_oob_heavy", 3, 2, 4, 4, (4, 9, 7), (3, 3, 3), (1, 1, 1), (1, 1, 1), (1, 1, 1), 1, 2, offset_std=3.0),
    Case("d3_groups_stride", 3, 2, 8, 12, (5, 8, 8), (3, 3, 3), (1, 2, 2), (2, 2, 2), (2, 2, 2), 4, 2, offset_std=2.0,
         bias=True),
    Case("d3_k133", 3, 1, 4, 4, (3, 6, 6), (1, 3, 3), (1, 1, 1), (0, 1, 1), (1, 1, 1), 1, 4, offset_std=1.0),
    Case("d3_single_voxel", 3, 1, 1, 1, (1, 1, 1), (1, 1, 1), (1, 1, 1), (0, 0, 0), (1, 1, 1), 1, 1, offset_std=0.6),
    Case("d3_double", 3, 1, 2, 2, (3, 5, 4), (2, 3, 3), (1, 1, 1), (1, 1, 1), (1, 1, 1), 1, 1, dtype="float64",
         offset_std=1.5),
    Case("c2_k3_groups", 2, 3, 8, 12, (11, 9), (3, 3), (2, 1), (1, 2), (1, 2), 4, 8, deformable=False, bias=True),
    Case("c2_ragged_tiles", 2, 1, 3, 5, (13, 17), (5, 3), (1, 1), (2, 1), (1, 1), 1, 3, deformable=False),
]

# --- tensor-core eligible shapes (channels per group multiples of 8) -----------------------------------
TC_CASES = [
    Case("tc2_small", 2, 2, 16, 32, (12, 12), (3, 3), (1, 1), (1, 1), (1, 1), 1, 16, offset_std=2.0, bias=True),
    Case("tc2_dg_groups", 2, 2, 64, 48, (14, 10), (3, 3), (1, 1), (1, 1), (1, 1), 2, 8, offset_std=2.0),
    Case("tc2_c256", 2, 1, 256, 256, (14, 14), (3, 3), (1, 1), (1, 1), (1, 1), 1, 64, offset_std=3.0),
    Case("tc2_stride_dil", 2, 2, 32, 40, (15, 13), (3, 3), (2, 1), (2, 2), (2, 2), 1, 8, offset_std=2.0),
    Case("tc3_small", 3, 2, 16, 16, (4, 8, 8), (3, 3, 3), (1, 1, 1), (1, 1, 1), (1, 1, 1), 1, 16, offset_std=1.5),
    Case("tc3_groups", 3, 1, 64, 64, (4, 7, 7), (3, 3, 3), (1, 2, 2), (2, 2, 2), (2, 2, 2), 4, 8, offset_std=2.0,
         bias=True),
    Case("tc3_o512", 3, 2, 128, 512, (2, 4, 4), (3, 3, 3), (1, 1, 1), (1, 1, 1), (1, 1, 1), 1, 32, offset_std=1.0),
    # four (deformable group, tap) keys per 64-channel chunk and more position tiles than SMs: the large corner
    # tables leave two operand stages, and CTAs with a second tile drain an accumulator between tables
    Case("tc2_cpg16_tiles", 2, 8, 64, 64, (50, 50), (3, 3), (1, 1), (1, 1), (1, 1), 1, 16, offset_std=2.5),
    # 157 position tiles on 148 SMs with 18 K chunks: the nine tiles of the partial last wave are split along K
    # and add into the zero-filled tail of y (which starts inside a sample)
    Case("tc2_c128_tail", 2, 8, 128, 64, (50, 50), (3, 3), (1, 1), (1, 1), (1, 1), 1, 32, offset_std=2.0, bias=True),
]

# --- BASELINE configurations 1-4 ------------------------------------------------------------------------
BASELINE = {
    1: Case("cfg1", 2, 2, 16, 32, (32, 32), (3, 3), (1, 1), (1, 1), (1, 1), 1, 16, offset_std=2.0),
    2: Case("cfg2", 2, 32, 256, 256, (56, 56), (3, 3), (1, 1), (1, 1), (1, 1), 1, 64, offset_std=3.0),
    3: Case("cfg3", 3, 8, 64, 64, (16, 56, 56), (3, 3, 3), (1, 1, 1), (1, 1, 1), (1, 1, 1), 1, 64, offset_std=1.5),
    4: Case("cfg4", 3, 16, 128, 256, (8, 28, 28), (3, 3, 3), (1, 2, 2), (2, 2, 2), (2, 2, 2), 4, 16, offset_std=2.0),
}


def make_inputs(case: Case, seed: int = 0, N: Optional[int] = None):
    """Tensors drawn on the CPU in the fixed order x, weight, offset, grad_out, bias (seeded)."""
    g = torch.Generator(device="cpu").manual_seed(seed)
    dt = torch.float32 if case.dtype == "float32" else torch.float64
    n = case.N if N is None else N
    p = case.problem()
    x = torch.rand((n, case.C) + tuple(case.in_size), generator=g, dtype=dt)
    if not case.x_uniform01:
        x = x * 2 - 1
    w = torch.empty((case.O, case.C // case.G) + tuple(case.kernel), dtype=dt)
    if case.x_uniform01:
        w.copy_(torch.rand(w.shape, generator=g, dtype=dt))
    else:
        torch.nn.init.kaiming_normal_(w, mode="fan_out", generator=g)
    off = None
    if case.deformable:
        shape = (n, p.offset_channels) + tuple(p.out_size)
        if case.offset_uniform:
            off = torch.rand(shape, generator=g, dtype=dt)
        else:
            off = torch.randn(shape, generator=g, dtype=dt) * case.offset_std
    dy = torch.randn((n, case.O) + tuple(p.out_size), generator=g, dtype=dt)
    b = (torch.rand(case.O, generator=g, dtype=dt) * 0.2 - 0.1) if case.bias else None
    if case.fixed == "d3_rows":
        x = torch.tensor([[1.0, 1, 1], [2.0, 2, 2], [1.0, 1, 1]], dtype=dt).expand(n, case.C, 3, 3, 3).contiguous()
        off.zero_(); w.fill_(1.0); dy.fill_(1.0)
    elif case.fixed == "ones":
        x.fill_(1.0); off.zero_(); w.fill_(1.0); dy.fill_(1.0)
    elif case.fixed == "zero_off":
        off.zero_()
    return x, w, off, dy, b


def np_inputs(case: Case, seed: int = 0, N: Optional[int] = None):
    return tuple(None if t is None else t.numpy() for t in make_inputs(case, seed, N))


def rel_err(a, b) -> float:
    """max|a-b| / max(max|b|, 1e-3) per tensor (the tolerance gates are stated on this quantity; the floor
    keeps tensors that are pure rounding residue, e.g. the offset gradient of a 1x1x1 input, from dividing
    noise by noise)."""
    a = np.asarray(a, dtype=np.float64)
    b = np.asarray(b, dtype=np.float64)
    den = max(float(np.abs(b).max()), 1e-3) if b.size else 1.0
    return float(np.abs(a - b).max() / den) if b.size else 0.0
