"""Model-level workload: a 3-D ResNet-18-style video network whose 3x3x3 convolutions in stages 3-4 are
deformable (``ConvOffset3d``, 4 deformable groups) with offsets produced by a plain ``nn.Conv3d``.

The reference ships no model; its only model-level pattern is "offsets from a plain conv, then the deformable
conv, then backward" (deform3d/test_model.py:18-32), which this network scales up.  Everything except the
deformable operator is stock PyTorch.  ``deform=False`` swaps the deformable layers for plain convolutions of
the same shape, which lets the data-parallel control logic be exercised on CPU ranks (the deformable operator
itself has no CPU implementation).
"""
from __future__ import annotations

from typing import Optional

import torch
import torch.nn as nn
import torch.nn.functional as F

from .modules import ConvOffset3d


class DeformUnit(nn.Module):
    """offset = conv3d(x) (same kernel / stride / padding, 3*27*dg channels, tiny init); y = deform_conv(x, offset).
    The reference's out-of-bounds pull-back term of the offset gradient is not a derivative of the loss; the model
    trains with the true (zero) gradient for invalid samples unless ``oob_offset_grad=True``."""

    def __init__(self, cin, cout, stride, dg=4, precision="auto", deform=True, oob_offset_grad=False):
        super().__init__()
        self.deform = deform
        if deform:
            self.offset = nn.Conv3d(cin, dg * 27 * 3, 3, stride=stride, padding=1, bias=True)
            nn.init.normal_(self.offset.weight, std=0.01)
            nn.init.zeros_(self.offset.bias)
            self.conv = ConvOffset3d(cin, cout, 3, stride=stride, padding=1, dilation=1, deformable_groups=dg,
                                     bias=False, groups=1, precision=precision, oob_offset_grad=oob_offset_grad)
        else:
            self.conv = nn.Conv3d(cin, cout, 3, stride=stride, padding=1, bias=False)

    def forward(self, x):
        if self.deform:
            return self.conv(x, self.offset(x))
        return self.conv(x)


def _conv3(cin, cout, stride, deformable, precision, deform):
    if deformable:
        return DeformUnit(cin, cout, stride, 4, precision, deform)
    return nn.Conv3d(cin, cout, 3, stride=stride, padding=1, bias=False)


class BasicBlock(nn.Module):
    def __init__(self, cin, cout, stride, deformable, precision, deform):
        super().__init__()
        self.conv1 = _conv3(cin, cout, stride, deformable, precision, deform)
        self.bn1 = nn.BatchNorm3d(cout)
        self.conv2 = _conv3(cout, cout, 1, deformable, precision, deform)
        self.bn2 = nn.BatchNorm3d(cout)
        self.down = None
        if stride != 1 or cin != cout:
            self.down = nn.Sequential(nn.Conv3d(cin, cout, 1, stride=stride, bias=False), nn.BatchNorm3d(cout))

    def forward(self, x):
        idt = x if self.down is None else self.down(x)
        y = F.relu(self.bn1(self.conv1(x)), inplace=True)
        y = self.bn2(self.conv2(y))
        return F.relu(y + idt, inplace=True)


class R3D18Deform(nn.Module):
    """Stem 3->64 (3,7,7)/(1,2,2) + BN + ReLU + maxpool 3/2; stages 64/128/256/512 x 2 blocks, strides 1/2/2/2;
    stages 3-4 deformable; global average pool; linear 512 -> num_classes."""

    def __init__(self, num_classes=400, width=64, precision="auto", deform=True):
        super().__init__()
        w = width
        self.stem = nn.Sequential(nn.Conv3d(3, w, (3, 7, 7), stride=(1, 2, 2), padding=(1, 3, 3), bias=False),
                                  nn.BatchNorm3d(w), nn.ReLU(inplace=True),
                                  nn.MaxPool3d(3, stride=2, padding=1))
        cfg = [(w, w, 1, False), (w, 2 * w, 2, False), (2 * w, 4 * w, 2, True), (4 * w, 8 * w, 2, True)]
        stages = []
        for cin, cout, stride, deformable in cfg:
            stages.append(nn.Sequential(BasicBlock(cin, cout, stride, deformable, precision, deform),
                                        BasicBlock(cout, cout, 1, deformable, precision, deform)))
        self.stages = nn.Sequential(*stages)
        self.fc = nn.Linear(8 * w, num_classes)

    def forward(self, x):
        x = self.stages(self.stem(x))
        return self.fc(torch.flatten(F.adaptive_avg_pool3d(x, 1), 1))


def shard(t: torch.Tensor, rank: int, world: int) -> torch.Tensor:
    """Contiguous batch shard of rank `rank` (the batch must divide evenly)."""
    n = t.size(0)
    if n % world != 0:
        raise ValueError("batch %d does not divide over %d ranks" % (n, world))
    per = n // world
    return t[rank * per:(rank + 1) * per]


def all_reduce_grads(model: nn.Module, world: int, bucket_bytes: int = 25 << 20) -> int:
    """Sum-all-reduce every parameter gradient in flat buckets and divide by the world size (mean over the
    global batch).  Only parameter gradients cross the network: no activation is exchanged.  Returns the number
    of collectives issued."""
    import torch.distributed as dist
    grads = [p.grad for p in model.parameters() if p.grad is not None]
    n_coll, i = 0, 0
    while i < len(grads):
        bucket, size = [], 0
        while i < len(grads) and (not bucket or size + grads[i].numel() * grads[i].element_size() <= bucket_bytes):
            if bucket and grads[i].dtype != bucket[0].dtype:
                break
            bucket.append(grads[i])
            size += grads[i].numel() * grads[i].element_size()
            i += 1
        flat = torch.cat([g.reshape(-1) for g in bucket])
        dist.all_reduce(flat)
        flat.div_(world)
        off = 0
        for g in bucket:
            g.copy_(flat[off:off + g.numel()].view_as(g))
            off += g.numel()
        n_coll += 1
    return n_coll


def train_step(model: nn.Module, opt: torch.optim.Optimizer, clips: torch.Tensor, labels: torch.Tensor,
               world: int = 1, ddp: bool = False, check_status: bool = False) -> torch.Tensor:
    """forward + cross-entropy + backward + gradient all-reduce + SGD step on this rank's shard.
    ``check_status``: read the library's device status word after the step (synchronises the stream; raises if a
    bounded device-side wait gave up) -- meant for every N-th step of a training loop."""
    opt.zero_grad(set_to_none=True)
    loss = F.cross_entropy(model(clips), labels)
    loss.backward()
    if world > 1 and not ddp:
        all_reduce_grads(model.module if hasattr(model, "module") else model, world)
    opt.step()
    if check_status:
        from .ops import check_status as _check
        _check(clips.device)
    return loss.detach()


class GraphedTrainStep:
    """Forward + backward of one training step captured in a CUDA graph and replayed: the network's few hundred
    small launches per step (late stages work on a handful of positions per clip) stop costing host time, which
    is what bounds the step once the batch is split over several GPUs.  The gradient all-reduce (a few flat
    buckets) and the optimizer step run eagerly after the replay, outside the capture.
    Inputs are copied into static buffers before each replay."""

    def __init__(self, model: nn.Module, opt: torch.optim.Optimizer, clips: torch.Tensor, labels: torch.Tensor,
                 world: int = 1, warmup: int = 3):
        self.model, self.opt, self.world = model, opt, world
        self.clips = clips.clone()
        self.labels = labels.clone()
        side = torch.cuda.Stream()
        side.wait_stream(torch.cuda.current_stream())
        with torch.cuda.stream(side):
            for _ in range(warmup):                       # cuDNN algorithm selection, allocator warm-up
                self._fwd_bwd()
        torch.cuda.current_stream().wait_stream(side)
        torch.cuda.synchronize()
        self.graph = torch.cuda.CUDAGraph()
        with torch.cuda.graph(self.graph):
            self.loss = self._fwd_bwd()

    def _fwd_bwd(self):
        self.opt.zero_grad(set_to_none=False)
        loss = F.cross_entropy(self.model(self.clips), self.labels)
        loss.backward()
        return loss.detach()

    def __call__(self, clips: Optional[torch.Tensor] = None, labels: Optional[torch.Tensor] = None,
                 check_status: bool = False) -> torch.Tensor:
        if clips is not None:
            self.clips.copy_(clips, non_blocking=True)      # keeps the static buffer's memory format
        if labels is not None:
            self.labels.copy_(labels, non_blocking=True)
        self.graph.replay()
        if self.world > 1:
            all_reduce_grads(self.model, self.world)
        self.opt.step()
        if check_status:                                    # after the replay, outside any capture
            from .ops import check_status as _check
            _check(self.clips.device)
        return self.loss
