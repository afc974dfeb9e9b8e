"""Generates tests/golden/reference_vectors.npz: outputs of the REFERENCE's own device kernels
(oracle/_ref, built from the reference checkout by oracle/Makefile) on the reference's test recipes and on
a few parameter corners.  Needs a CUDA device; run from the repository root on a GPU box:

    python tests/golden/make_golden.py <output.npz>

The committed .npz was produced this way on a B200 and is what the CPU test-suite pins the oracle to.
fp32 2-D cases with dilation > 1 or groups > 1 have no fp32 reference package (deform2d has neither), so
they are not listed here.
"""
import os
import sys

import numpy as np
import torch

ROOT = os.path.dirname(os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
sys.path.insert(0, ROOT)

from oracle import ref_gpu  # noqa: E402
from tests import cases  # noqa: E402

GOLDEN_CASES = ["d3_test_function", "d3_test_gradient", "d3_test_model", "d2d_test_function", "d2d_test_gradient",
                "d2_test_gradient", "d2_test_function", "c2_test_gradient", "d2_oob_heavy_ref", "d2_double_corner",
                "d3_oob_heavy", "d3_groups_stride", "d3_k133", "c2_k3_groups"]


def all_cases():
    d = {c.name: c for c in cases.REFERENCE_RECIPES + cases.CORNERS}
    # the fp32 2-D reference package has no groups: a G=1 twin of the out-of-bounds-heavy corner
    import dataclasses
    d["d2_oob_heavy_ref"] = dataclasses.replace(d["d2_oob_heavy"], name="d2_oob_heavy_ref", G=1)
    return d


def main(out_path):
    assert torch.cuda.is_available() and ref_gpu.available()
    table = all_cases()
    blob = {}
    for name in GOLDEN_CASES:
        c = table[name]
        x, w, off, dy, b = cases.make_inputs(c)
        dev = "cuda"
        p = c.problem()
        op = ref_gpu.RefOp(ref_gpu.variant_for(c), p)
        xd, wd, dyd = x.to(dev), w.to(dev), dy.to(dev)
        offd = off.to(dev) if off is not None else None
        bd = b.to(dev) if b is not None else None
        y = op.forward(xd, offd, wd, bd)
        dx, doff = op.backward_data(xd, offd, wd, dyd)
        dw = op.backward_weight(xd, offd, dyd)
        blob[name + ".y"] = y.cpu().numpy()
        blob[name + ".dx"] = dx.cpu().numpy()
        blob[name + ".dw"] = dw.cpu().numpy()
        if doff is not None:
            blob[name + ".doff"] = doff.cpu().numpy()
        print(name, "y", tuple(y.shape), float(y.abs().max()))
    np.savez_compressed(out_path, **blob)
    print("wrote", out_path, os.path.getsize(out_path), "bytes")


if __name__ == "__main__":
    if len(sys.argv) != 2:
        sys.exit("usage: python tests/golden/make_golden.py <output .npz path>")
    main(sys.argv[1])
