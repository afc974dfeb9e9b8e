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

import os

from .functions import DeformLayerFunction
from .modules import ConvOffset3d


class DeformUnit(nn.Module):
    """offset = conv3d(x) (same kernel / stride / padding, 3*27*dg channels, tiny init); y = deform_conv(x, offset).
    The reference's out-of-bounds pull-back term of the offset gradient is not a derivative of the loss; the model
    trains with the true (zero) gradient for invalid samples unless ``oob_offset_grad=True``.
    ``one_call`` (default: ``DCN_MODEL_ONE_CALL``, off): both convolutions through the library's layer entry point
    instead of a stock convolution followed by the deformable operator; the parameters are the same either way."""

    def __init__(self, cin, cout, stride, dg=4, precision="auto", deform=True, oob_offset_grad=False, one_call=None):
        super().__init__()
        self.deform = deform
        self.one_call = (os.environ.get("DCN_MODEL_ONE_CALL", "0") not in ("", "0")) if one_call is None else one_call
        if deform:
            self.offset = nn.Conv3d(cin, dg * 27 * 3, 3, stride=stride, padding=1, bias=True)
            nn.init.normal_(self.offset.weight, std=0.01)
            nn.init.zeros_(self.offset.bias)
            self.conv = ConvOffset3d(cin, cout, 3, stride=stride, padding=1, dilation=1, deformable_groups=dg,
                                     bias=False, groups=1, precision=precision, oob_offset_grad=oob_offset_grad)
        else:
            self.conv = nn.Conv3d(cin, cout, 3, stride=stride, padding=1, bias=False)

    def forward(self, x):
        if self.deform and self.one_call:
            c = self.conv
            return DeformLayerFunction.apply(x, self.offset.weight, self.offset.bias, c.weight, c.bias, c.stride,
                                             c.padding, c.dilation, c.channel_per_group, c.group, c.precision,
                                             c.oob_offset_grad)
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


class GradBuckets:
    """Parameter gradients as views into a few preallocated flat buffers.  The exchange step is then one in-place
    all-reduce (mean) per buffer: nothing is concatenated, divided or copied back.  Buckets are filled in reverse
    parameter order, the order in which backward produces the gradients.  Only parameter gradients cross the
    network: no activation is exchanged."""

    def __init__(self, model: nn.Module, bucket_bytes: int = 25 << 20):
        self.flats = []
        params = [p for p in reversed(list(model.parameters())) if p.requires_grad]
        i = 0
        while i < len(params):
            group, size = [], 0
            while i < len(params) and (not group or size + params[i].numel() * params[i].element_size() <= bucket_bytes):
                if group and (params[i].dtype != group[0].dtype or params[i].device != group[0].device):
                    break
                group.append(params[i])
                size += params[i].numel() * params[i].element_size()
                i += 1
            flat = torch.zeros(sum(p.numel() for p in group), dtype=group[0].dtype, device=group[0].device)
            off = 0
            for p in group:
                # the view has the parameter's own strides (channels-last weights keep their layout)
                p.grad = torch.as_strided(flat, p.size(), p.stride(), off) if _dense(p) else flat[off:off + p.numel()].view_as(p)
                off += p.numel()
            self.flats.append(flat)

    def zero(self):
        for f in self.flats:
            f.zero_()

    def all_reduce(self, world: int) -> int:
        """Mean over the ranks, in place; returns the number of collectives issued."""
        import torch.distributed as dist
        if world <= 1:
            return 0
        for f in self.flats:
            if dist.get_backend() == "nccl":
                dist.all_reduce(f, op=dist.ReduceOp.AVG)
            else:                                     # gloo has no AVG
                dist.all_reduce(f)
                f.div_(world)
        return len(self.flats)


def _dense(p: torch.Tensor) -> bool:
    """True if the parameter's elements occupy numel() consecutive storage slots in some dimension order."""
    return p.is_contiguous() or p.is_contiguous(memory_format=torch.channels_last_3d if p.dim() == 5 else
                                                torch.channels_last if p.dim() == 4 else torch.contiguous_format)


def all_reduce_grads(model: nn.Module, world: int, bucket_bytes: int = 25 << 20) -> int:
    """Mean-all-reduce of whatever gradients the parameters hold right now: they are moved into fresh flat buckets
    (a training loop keeps one :class:`GradBuckets` instead and lets backward write into it, see
    :func:`train_step`).  Returns the number of collectives issued."""
    grads = {id(p): p.grad for p in model.parameters() if p.grad is not None}
    gb = GradBuckets(model, bucket_bytes)
    for p in model.parameters():
        if id(p) in grads:
            p.grad.copy_(grads[id(p)])
        elif p.requires_grad:
            p.grad.zero_()
    return gb.all_reduce(world)


def train_step(model: nn.Module, opt: torch.optim.Optimizer, clips: torch.Tensor, labels: torch.Tensor,
               world: int = 1, ddp: bool = False, check_status: bool = False) -> torch.Tensor:
    """forward + cross-entropy + backward + gradient all-reduce + SGD step on this rank's shard.
    ``check_status``: read the library's device status word after the step (synchronises the stream; raises if a
    bounded device-side wait gave up) -- meant for every N-th step of a training loop."""
    inner = model.module if hasattr(model, "module") else model
    gb = None
    if world > 1 and not ddp:
        gb = getattr(inner, "_grad_buckets", None)
        if gb is None:
            gb = inner._grad_buckets = GradBuckets(inner)
        gb.zero()                                          # backward accumulates into the bucket views
    else:
        opt.zero_grad(set_to_none=True)
    loss = F.cross_entropy(model(clips), labels)
    loss.backward()
    if gb is not None:
        gb.all_reduce(world)
    opt.step()
    if check_status:
        from .ops import check_status as _check
        _check(clips.device)
    return loss.detach()


class GraphedTrainStep:
    """Forward + backward of one training step captured in a CUDA graph and replayed: the network's few hundred
    small launches per step (late stages work on a handful of positions per clip) stop costing host time, which
    is what bounds the step once the batch is split over several GPUs.  Gradients live in flat buckets
    (:class:`GradBuckets`); the all-reduce of the buckets and the optimizer step run eagerly after the replay,
    outside the capture.  Inputs are copied into static buffers before each replay."""

    def __init__(self, model: nn.Module, opt: torch.optim.Optimizer, clips: torch.Tensor, labels: torch.Tensor,
                 world: int = 1, warmup: int = 3):
        self.model, self.opt, self.world = model, opt, world
        self.clips = clips.clone()
        self.labels = labels.clone()
        self.buckets = GradBuckets(model)
        model._grad_buckets = self.buckets
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
        self.phase_events = None

    def _fwd_bwd(self):
        self.buckets.zero()                               # gradients accumulate into the bucket views
        loss = F.cross_entropy(self.model(self.clips), self.labels)
        loss.backward()
        return loss.detach()

    def __call__(self, clips: Optional[torch.Tensor] = None, labels: Optional[torch.Tensor] = None,
                 check_status: bool = False, timed: bool = False) -> torch.Tensor:
        """``timed``: record CUDA events around the three phases (compute = graph replay, exchange = all-reduce,
        optimizer) into ``self.phase_events`` (four events)."""
        ev = [torch.cuda.Event(enable_timing=True) for _ in range(4)] if timed else None
        if clips is not None:
            self.clips.copy_(clips, non_blocking=True)      # keeps the static buffer's memory format
        if labels is not None:
            self.labels.copy_(labels, non_blocking=True)
        if ev:
            ev[0].record()
        self.graph.replay()
        if ev:
            ev[1].record()
        self.buckets.all_reduce(self.world)
        if ev:
            ev[2].record()
        self.opt.step()
        if ev:
            ev[3].record()
            self.phase_events = ev
        if check_status:                                    # after the replay, outside any capture
            from .ops import check_status as _check
            _check(self.clips.device)
        return self.loss
