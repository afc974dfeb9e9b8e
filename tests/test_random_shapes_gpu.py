"""Seeded random geometries through both CUDA paths against the CPU oracle.

The reference tests a handful of hand-picked recipes (deform3d/test_gradient.py:9-30, deform2d_double/
test_gradient.py:7-53); the fixed cases of tests/cases.py restate them and add corners.  This sweep draws
geometries at random (dimensionality, groups, deformable groups, rectangular kernels, stride, padding, dilation,
ragged sizes, offsets large enough to leave the input) so that index arithmetic nobody thought to write a case for
gets exercised too.  Gates: exact path 1e-4 against the fp32 oracle (same arithmetic), bf16 path 2e-2 against the
float64 oracle evaluated at the reference's fp32 coordinates."""
import numpy as np
import pytest

from tests import cases, helpers

pytestmark = pytest.mark.gpu


def _draw(rng, ndim, tensor_core):
    for _ in range(200):
        G = int(rng.choice([1, 1, 2, 4])) if not tensor_core else int(rng.choice([1, 1, 2]))
        if tensor_core:
            cpg = int(rng.choice([8, 16]))
            cg = cpg * int(rng.choice([1, 2]))              # channels per convolution group: whole deformable groups
            og = int(rng.choice([8, 16, 24, 40]))
        else:
            cpg = int(rng.choice([1, 2, 3, 4]))
            cg = cpg * int(rng.choice([1, 2, 3]))
            og = int(rng.integers(1, 6))
        C, O = G * cg, G * og
        if C % cpg != 0:
            continue
        k = tuple(int(v) for v in rng.integers(1, 4, ndim))
        stride = tuple(int(v) for v in rng.integers(1, 3, ndim))
        pad = tuple(int(v) for v in rng.integers(0, 3, ndim))
        dil = tuple(int(v) for v in rng.integers(1, 3, ndim))
        lo, hi = (3, 8) if ndim == 3 else (4, 14)
        size = tuple(int(v) for v in rng.integers(lo, hi, ndim))
        if any((s + 2 * p - kk) // st + 1 < 1 or s + 2 * p < kk for s, p, kk, st in zip(size, pad, k, stride)):
            continue
        return dict(ndim=ndim, N=int(rng.integers(1, 4)), C=C, O=O, in_size=size, kernel=k, stride=stride, pad=pad,
                    dil=dil, G=G, cpg=cpg, bias=bool(rng.integers(0, 2)), offset_std=float(rng.choice([0.5, 1.5, 3.0])))
    raise RuntimeError("no valid geometry drawn")


def _cases(seed, count, tensor_core, dtype="float32"):
    rng = np.random.default_rng(seed)
    out = []
    for i in range(count):
        kw = _draw(rng, 2 + (i % 2), tensor_core)
        tag = "_tc" if tensor_core else ("_f64" if dtype == "float64" else "")
        out.append(cases.Case("rnd%s_%d" % (tag, i), dtype=dtype, **kw))
    return out


# fp32: these sizes take the latency-shaped small-problem kernels; fp64: the tiled kernels
@pytest.mark.parametrize("case", _cases(20240607, 24, False) + _cases(31337, 12, False, "float64"), ids=lambda c: c.name)
def test_exact_path_on_random_geometries(case):
    tensors = cases.make_inputs(case)
    ours = helpers.run_ours(case, tensors, "exact")
    same = helpers.run_oracle(case, tensors)
    tol = 1e-4 if case.dtype == "float32" else 1e-10
    for k in same:
        assert ours[k].shape == same[k].shape, (k, case)
        assert cases.rel_err(ours[k], same[k]) <= tol, (k, cases.rel_err(ours[k], same[k]), case)


@pytest.mark.parametrize("case", _cases(977, 16, True), ids=lambda c: c.name)
def test_bf16_path_on_random_geometries(case):
    import deform_conv3d_pytorch_op_b200 as dcn
    tensors = list(cases.make_inputs(case))
    off32 = helpers.offsets_at_fp32_coordinates(case, tensors[2].numpy())
    ours = helpers.run_ours(case, tensors, "bf16")
    dcn.check_status()
    t64 = [None if t is None else t.numpy().astype(np.float64) for t in tensors]
    x, w, _, dy, b = t64
    p = case.problem()
    p.N = x.shape[0]
    from oracle import oracle as orc
    ref = {"y": orc.forward(p, x, off32, w, b)}
    ref["dx"], ref["doff"] = orc.backward_data(p, x, off32, w, dy)
    ref["dw"] = orc.backward_weight(p, x, off32, dy)
    mask = helpers.lattice_mask(case, tensors[2].numpy())
    for k in ("y", "dx", "dw", "doff"):
        a, r = ours[k].astype(np.float64), ref[k]
        if k == "doff":
            a, r = np.where(mask, 0, a), np.where(mask, 0, r)
        assert cases.rel_err(a, r) <= 2e-2, (k, cases.rel_err(a, r), case)


@pytest.mark.parametrize("case", _cases(4242, 16, False), ids=lambda c: c.name)
def test_layer_forward_on_random_geometries(case):
    """The single-kernel layer forward (offsets formed in the kernel) against torch's fp32 convolution for the
    offsets and the library's own deformable Function, itself oracle-checked above, for y (fp32 gate 1e-4)."""
    import torch
    import deform_conv3d_pytorch_op_b200 as dcn
    x, w, off, dy, b = [None if t is None else t.cuda() for t in cases.make_inputs(case)]
    op = dcn.Op(x, w, case.stride, case.pad, case.dil, case.cpg, case.G)
    g = torch.Generator().manual_seed(3)
    w_off = (torch.randn(op.offset_weight_shape(), generator=g) * 0.2).cuda()
    b_off = (torch.randn(op.offset_channels, generator=g) * 0.5).cuda()
    y, offsets = op.layer_forward(x, w_off, b_off, w, b)
    conv = torch.nn.functional.conv3d if case.ndim == 3 else torch.nn.functional.conv2d
    with torch.backends.cudnn.flags(enabled=True, allow_tf32=False):
        off_ref = conv(x, w_off, b_off, stride=case.stride, padding=case.pad)
    assert offsets.shape == off_ref.shape
    assert cases.rel_err(offsets.cpu().numpy(), off_ref.cpu().numpy()) <= 1e-5
    fn = dcn.ConvOffset3dFunction if case.ndim == 3 else dcn.ConvOffset2dFunction
    y_ref = fn.apply(x, offsets, w, b, case.stride, case.pad, case.dil, case.cpg, case.G)
    assert cases.rel_err(y.cpu().numpy(), y_ref.cpu().numpy()) <= 1e-4


@pytest.mark.parametrize("case", _cases(5150, 12, False), ids=lambda c: c.name)
def test_layer_backward_on_random_geometries(case):
    """All five gradients of the single-kernel layer backward (offset gradient kept in shared memory) against
    autograd through torch's fp32 convolution followed by the library's deformable Function."""
    import torch
    import deform_conv3d_pytorch_op_b200 as dcn
    x, w, off, dy, b = [None if t is None else t.cuda() for t in cases.make_inputs(case)]
    op = dcn.Op(x, w, case.stride, case.pad, case.dil, case.cpg, case.G)
    g = torch.Generator().manual_seed(4)
    w_off = (torch.randn(op.offset_weight_shape(), generator=g) * 0.2).cuda()
    b_off = (torch.randn(op.offset_channels, generator=g) * 0.5).cuda()
    if b is None:
        b = torch.zeros(case.O, device="cuda")
    params = [t.clone().requires_grad_(True) for t in (x, w_off, b_off, w, b)]
    y = dcn.DeformLayerFunction.apply(params[0], params[1], params[2], params[3], params[4], case.stride, case.pad,
                                      case.dil, case.cpg, case.G, "exact", False)
    got = torch.autograd.grad(y, params, dy)
    conv = torch.nn.functional.conv3d if case.ndim == 3 else torch.nn.functional.conv2d
    fn = dcn.ConvOffset3dFunction if case.ndim == 3 else dcn.ConvOffset2dFunction
    ref_p = [t.clone().requires_grad_(True) for t in (x, w_off, b_off, w, b)]
    with torch.backends.cudnn.flags(enabled=True, allow_tf32=False):
        o = conv(ref_p[0], ref_p[1], ref_p[2], stride=case.stride, padding=case.pad)
        y_ref = fn.apply(ref_p[0], o, ref_p[3], ref_p[4], case.stride, case.pad, case.dil, case.cpg, case.G, "exact", False)
        want = torch.autograd.grad(y_ref, ref_p, dy)
    assert cases.rel_err(y.detach().cpu().numpy(), y_ref.detach().cpu().numpy()) <= 1e-4
    for name, a, r in zip(("dx", "doffset_weight", "doffset_bias", "dweight", "dbias"), got, want):
        assert cases.rel_err(a.cpu().numpy(), r.cpu().numpy()) <= 2e-4, (name, case)
