"""Model-level workload and its data-parallel control logic.

CPU part: two gloo ranks, each on half of the batch, must end up with the gradients of one process on the whole
batch (mean reduction), using the plain-convolution stand-in for the deformable layers (the operator itself is
CUDA-only).  GPU part: the real network (deformable stages) runs a training step on cuda:0 and its loss decreases
over a few steps of SGD on a fixed batch."""
import os
import socket

import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

from deform_conv3d_pytorch_op_b200 import r3d


def _free_port():
    s = socket.socket()
    s.bind(("127.0.0.1", 0))
    p = s.getsockname()[1]
    s.close()
    return p


def _make(width=8, classes=10):
    torch.manual_seed(0)
    m = r3d.R3D18Deform(num_classes=classes, width=width, deform=False)
    # BatchNorm statistics are per shard; use eval-mode BN so both runs compute the same function
    for mod in m.modules():
        if isinstance(mod, torch.nn.BatchNorm3d):
            mod.eval()
    return m


def _batch(n=4):
    g = torch.Generator().manual_seed(1)
    return torch.randn(n, 3, 4, 32, 32, generator=g), torch.randint(0, 10, (n,), generator=g)


def _worker(rank, world, port, out):
    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    dist.init_process_group("gloo", rank=rank, world_size=world)
    torch.set_num_threads(2)
    m = _make()
    x, y = _batch()
    xs, ys = r3d.shard(x, rank, world), r3d.shard(y, rank, world)
    loss = torch.nn.functional.cross_entropy(m(xs), ys)
    loss.backward()
    n_coll = r3d.all_reduce_grads(m, world, bucket_bytes=1 << 16)
    if rank == 0:
        torch.save({"grads": [p.grad.clone() for p in m.parameters()], "n_coll": n_coll}, out)
    dist.barrier()
    dist.destroy_process_group()


def test_two_gloo_ranks_match_single_process(tmp_path):
    out = str(tmp_path / "g.pt")
    mp.spawn(_worker, args=(2, _free_port(), out), nprocs=2, join=True)
    got = torch.load(out)
    m = _make()
    x, y = _batch()
    torch.nn.functional.cross_entropy(m(x), y).backward()
    assert got["n_coll"] >= 2                     # several buckets at this bucket size
    for a, p in zip(got["grads"], m.parameters()):
        assert torch.allclose(a, p.grad, rtol=1e-4, atol=1e-6)


def test_shard_checks_divisibility():
    with pytest.raises(ValueError):
        r3d.shard(torch.zeros(5, 1), 0, 2)
    assert r3d.shard(torch.arange(8).view(8, 1), 1, 4).flatten().tolist() == [2, 3]


def test_model_shapes_on_cpu_stand_in():
    m = r3d.R3D18Deform(num_classes=7, width=8, deform=False)
    assert m(torch.zeros(2, 3, 8, 32, 32)).shape == (2, 7)
    full = r3d.R3D18Deform(num_classes=400, width=64, deform=True)
    units = [mod for mod in full.modules() if isinstance(mod, r3d.DeformUnit)]
    assert len(units) == 8 and all(u.offset.out_channels == 324 for u in units)
    assert units[0].conv.in_channels == 128 and units[-1].conv.out_channels == 512


@pytest.mark.gpu
def test_deformable_network_trains_on_gpu():
    torch.manual_seed(0)
    m = r3d.R3D18Deform(num_classes=10, width=32, precision="auto").cuda()
    opt = torch.optim.SGD(m.parameters(), lr=0.05, momentum=0.9)
    g = torch.Generator().manual_seed(2)
    x = torch.randn(4, 3, 8, 64, 64, generator=g).cuda()
    y = torch.randint(0, 10, (4,), generator=g).cuda()
    opt = torch.optim.SGD(m.parameters(), lr=0.01, momentum=0.9)
    losses = [float(r3d.train_step(m, opt, x, y)) for _ in range(12)]
    assert all(torch.isfinite(torch.tensor(losses))), losses
    assert min(losses[-3:]) < losses[0], losses         # a fixed batch of 4 clips is memorised quickly
    # every deformable layer and every offset-producing conv received a gradient
    for mod in m.modules():
        if isinstance(mod, r3d.DeformUnit):
            assert mod.conv.weight.grad is not None and float(mod.conv.weight.grad.abs().sum()) > 0
            assert mod.offset.weight.grad is not None and float(mod.offset.weight.grad.abs().sum()) > 0
    from deform_conv3d_pytorch_op_b200 import _lib
    _lib.check(_lib.lib().dcn_check_status(_lib.current_stream(torch.device("cuda"))), "device status")


def _make_deform(width=16, classes=10):
    # the stock layers in plain fp32 (cuDNN otherwise picks TF32 algorithms, which differ with the batch size)
    torch.backends.cudnn.allow_tf32 = False
    torch.backends.cuda.matmul.allow_tf32 = False
    torch.manual_seed(0)
    m = r3d.R3D18Deform(num_classes=classes, width=width, precision="exact", deform=True)
    for mod in m.modules():
        if isinstance(mod, torch.nn.BatchNorm3d):
            mod.eval()
        if isinstance(mod, r3d.DeformUnit):
            torch.nn.init.normal_(mod.offset.weight, std=0.05)      # offsets that actually move the samples
    return m


def _gpu_worker(rank, world, port, out):
    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    os.environ["NCCL_NVLS_ENABLE"] = "0"
    torch.cuda.set_device(rank)
    dev = torch.device("cuda", rank)
    dist.init_process_group("nccl", rank=rank, world_size=world, device_id=dev)
    m = _make_deform().to(dev)
    x, y = _batch()
    xs, ys = r3d.shard(x, rank, world).to(dev), r3d.shard(y, rank, world).to(dev)
    gb = r3d.GradBuckets(m, bucket_bytes=1 << 18)          # backward writes straight into the flat buckets
    torch.nn.functional.cross_entropy(m(xs), ys).backward()
    n_coll = gb.all_reduce(world)
    torch.cuda.synchronize()
    if rank == 0:
        torch.save({"grads": [p.grad.detach().cpu().clone() for p in m.parameters()], "n_coll": n_coll}, out)
    dist.barrier()
    dist.destroy_process_group()


@pytest.mark.gpu
def test_two_gpu_ranks_with_deformable_layers_match_single_process(tmp_path):
    """The real network (deformable stages 3-4, exact precision) on two GPUs, half a batch each, gradients averaged
    through the flat buckets over NCCL, against one process on the whole batch."""
    if torch.cuda.device_count() < 2:
        pytest.skip("needs two GPUs")
    out = str(tmp_path / "g2.pt")
    mp.spawn(_gpu_worker, args=(2, _free_port(), out), nprocs=2, join=True)
    got = torch.load(out)
    m = _make_deform().cuda()
    x, y = _batch()
    torch.nn.functional.cross_entropy(m(x.cuda()), y.cuda()).backward()
    assert got["n_coll"] >= 2
    for a, p in zip(got["grads"], m.parameters()):
        ref = p.grad.cpu()
        scale = max(float(ref.abs().max()), 1e-6)
        assert float((a - ref).abs().max()) <= 1e-3 * scale + 1e-7, float((a - ref).abs().max()) / scale
