"""The benchmark configurations (2-D / 3-D deformable convolution, forward + backward) and the seeded
synthetic generator shared by the benchmark and the tests.  Tensors are drawn on the CPU in fp32 in the
fixed order x, weight, offset, grad_out so that every consumer sees identical bits."""
from __future__ import annotations

from dataclasses import dataclass
from typing import Optional, Tuple

import torch


@dataclass(frozen=True)
class Workload:
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
    G: int
    cpg: int
    offset_std: float

    @property
    def out_size(self):
        # the deformable operators ignore dilation in the size rule (reference behaviour)
        return tuple((i + 2 * p - k) // s + 1 for i, p, k, s in zip(self.in_size, self.pad, self.kernel, self.stride))

    @property
    def kv(self):
        n = 1
        for k in self.kernel:
            n *= k
        return n

    @property
    def ov(self):
        n = 1
        for o in self.out_size:
            n *= o
        return n

    @property
    def iv(self):
        n = 1
        for o in self.in_size:
            n *= o
        return n

    @property
    def offset_channels(self):
        return (self.C // self.cpg) * self.kv * self.ndim

    def flops(self, n: Optional[int] = None) -> float:
        """Algorithmic FLOPs of forward + both backward passes: 3 contractions of 2*N*O*(C/G)*kv*ov."""
        n = self.N if n is None else n
        return 3.0 * 2.0 * n * self.O * (self.C // self.G) * self.kv * self.ov

    def bytes_alg(self, n: Optional[int] = None):
        """Compulsory fp32 traffic, each tensor once per pass: (forward, backward)."""
        n = self.N if n is None else n
        x = n * self.C * self.iv
        off = n * self.offset_channels * self.ov
        w = self.O * (self.C // self.G) * self.kv
        y = n * self.O * self.ov
        fwd = 4.0 * (x + off + w + y)
        bwd = 4.0 * ((x + off + w + y) + (x + off + w))
        return fwd, bwd

    def bytes_gather_scatter(self, n: Optional[int] = None) -> float:
        """Bytes one gathering or scattering pass moves if every sample touches its 2^D corners in fp32:
        N * C * kv * ov samples x 2^D x 4 B.  Implementation-dependent and mostly cache-resident; informative."""
        n = self.N if n is None else n
        return 4.0 * (2 ** self.ndim) * n * self.C * self.kv * self.ov

    def bytes_per_pass(self, n: Optional[int] = None):
        """Compulsory fp32 traffic of each pass taken alone (every tensor it reads or writes, once)."""
        n = self.N if n is None else n
        x = n * self.C * self.iv
        off = n * self.offset_channels * self.ov
        w = self.O * (self.C // self.G) * self.kv
        y = n * self.O * self.ov
        return {"forward": 4.0 * (x + off + w + y), "backward_data": 4.0 * (x + off + w + y + x + off),
                "backward_weight": 4.0 * (x + off + y + w)}


CONFIGS = {
    1: Workload("cfg1_deform2d_16x32_32x32", 2, 2, 16, 32, (32, 32), (3, 3), (1, 1), (1, 1), (1, 1), 1, 16, 2.0),
    2: Workload("cfg2_deform2d_256x256_56x56_dg4", 2, 32, 256, 256, (56, 56), (3, 3), (1, 1), (1, 1), (1, 1), 1, 64, 3.0),
    3: Workload("cfg3_deform3d_64x64_16x56x56", 3, 8, 64, 64, (16, 56, 56), (3, 3, 3), (1, 1, 1), (1, 1, 1), (1, 1, 1),
                1, 64, 1.5),
    4: Workload("cfg4_deform3d_128x256_g4_dg8_d2", 3, 16, 128, 256, (8, 28, 28), (3, 3, 3), (1, 2, 2), (2, 2, 2),
                (2, 2, 2), 4, 16, 2.0),
}


def make_inputs(w: Workload, seed: int = 0, n: Optional[int] = None, pin: bool = False):
    """(x ~ U(-1,1), weight ~ Kaiming-normal fan_out, offset ~ N(0, std^2), grad_out ~ N(0,1)) on the CPU."""
    g = torch.Generator(device="cpu").manual_seed(seed)
    n = w.N if n is None else n
    x = torch.rand((n, w.C) + w.in_size, generator=g) * 2 - 1
    wt = torch.empty((w.O, w.C // w.G) + w.kernel)
    torch.nn.init.kaiming_normal_(wt, mode="fan_out", generator=g)
    off = torch.randn((n, w.offset_channels) + w.out_size, generator=g) * w.offset_std
    dy = torch.randn((n, w.O) + w.out_size, generator=g)
    ts = (x, wt, off, dy)
    if pin:
        ts = tuple(t.pin_memory() for t in ts)
    return ts
