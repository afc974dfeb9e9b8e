"""GPU box only: the CPU oracle against the reference's own device kernels (oracle/_ref, compiled unmodified
from the reference checkout), on the seeded test cases.  This is the pin that makes the oracle trustworthy;
the same comparison on the committed golden vectors runs in the CPU suite."""
import dataclasses

import pytest
import torch

from oracle import ref_gpu
from tests import cases, helpers

pytestmark = pytest.mark.gpu


def _cases():
    out = []
    for c in cases.REFERENCE_RECIPES + cases.CORNERS + cases.TC_CASES + [cases.BASELINE[1]]:
        if c.deformable and c.ndim == 2 and c.dtype == "float32" and (c.G != 1 or tuple(c.dil) != (1, 1)):
            continue        # the fp32 2-D reference package has neither groups nor dilation
        if c.ndim == 3 and c.dtype == "float64":
            continue        # no fp64 3-D reference package
        if not c.deformable and c.ndim != 2:
            continue
        out.append(c)
    return out


@pytest.mark.parametrize("case", _cases(), ids=lambda c: c.name)
def test_oracle_matches_reference_kernels(case):
    if not ref_gpu.available():
        pytest.skip("oracle/_ref not built (reference checkout absent when the repository was built)")
    tensors = cases.make_inputs(case)
    x, w, off, dy, b = [None if t is None else t.cuda() for t in tensors]
    op = ref_gpu.RefOp(ref_gpu.variant_for(case), case.problem())
    ref = {"y": op.forward(x, off, w, b)}
    ref["dx"], doff = op.backward_data(x, off, w, dy)
    if doff is not None:
        ref["doff"] = doff
    ref["dw"] = op.backward_weight(x, off, dy)
    mine = helpers.run_oracle(case, tensors)
    tol = 2e-5 if case.dtype == "float32" else 1e-12
    for k, v in ref.items():
        e = cases.rel_err(mine[k], v.cpu().numpy())
        assert e <= tol, (k, e)
