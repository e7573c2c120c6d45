"""The two restatements of the point-cloud depthwise convolution (torch and plain C) against each
other, the explicit backward against autograd of the forward, and - when present - against the
fixtures recorded from the reference's own CUDA kernels (tests/golden/pcloud_*.npz)."""
import os

import numpy as np
import pytest
import torch

from cases import PCLOUD_GOLDEN_CASES, pcloud_inputs
from conftest import rel_err
from oracle import c_oracle as co
from oracle import mesh_oracle as mo

GOLDEN_DIR = os.path.join(os.path.dirname(__file__), "golden")


def _n(t):
    return None if t is None else t.numpy()


@pytest.mark.parametrize("args", [(200, 60, 12, 9, 6, 2, 0, 5), (150, 80, 10, 17, 8, 1, 3, 6), (50, 50, 4, 3, 5, 3, 2, 7)])
def test_restatements_agree(args):
    d = pcloud_inputs(*args, shuffle=True)
    out = mo.pcloud_conv3d_forward(d["x"], d["filt"], d["nn_count"], d["nn_index"], d["bin_index"], d["bin_coeff"])
    gin, gf = mo.pcloud_conv3d_backward(d["g_out"], d["x"], d["filt"], d["nn_count"], d["nn_index"], d["bin_index"],
                                        d["bin_coeff"])
    c_out = co.pcloud_forward(_n(d["x"]), _n(d["filt"]), _n(d["nn_count"]), _n(d["nn_index"]), _n(d["bin_index"]),
                              _n(d["bin_coeff"]))
    c_gin, c_gf = co.pcloud_backward(_n(d["g_out"]), _n(d["x"]), _n(d["filt"]), _n(d["nn_count"]), _n(d["nn_index"]),
                                     _n(d["bin_index"]), _n(d["bin_coeff"]))
    assert rel_err(out, c_out) <= 1e-5 and rel_err(gin, c_gin) <= 1e-5 and rel_err(gf, c_gf) <= 1e-5


def test_backward_is_the_gradient_of_forward():
    d = pcloud_inputs(40, 30, 5, 4, 3, 2, 2, seed=9)
    x, w = d["x"].double().requires_grad_(), d["filt"].double().requires_grad_()
    out = mo.pcloud_conv3d_forward(x, w, d["nn_count"], d["nn_index"], d["bin_index"], d["bin_coeff"].double())
    (out * d["g_out"].double()).sum().backward()
    gin, gf = mo.pcloud_conv3d_backward(d["g_out"].double(), x.detach(), w.detach(), d["nn_count"], d["nn_index"],
                                        d["bin_index"], d["bin_coeff"].double())
    assert rel_err(gin, x.grad) <= 1e-12 and rel_err(gf, w.grad) <= 1e-12


@pytest.mark.parametrize("name", sorted(PCLOUD_GOLDEN_CASES))
def test_oracle_matches_reference_kernels(name):
    path = os.path.join(GOLDEN_DIR, name + ".npz")
    assert os.path.exists(path), "fixture missing: run tests/golden/make_golden.py on a GPU"
    z = np.load(path)
    d = pcloud_inputs(*PCLOUD_GOLDEN_CASES[name])
    for k, v in d.items():
        if isinstance(v, torch.Tensor):
            assert torch.equal(v, torch.from_numpy(z["in_" + k])), k
    out = mo.pcloud_conv3d_forward(d["x"], d["filt"], d["nn_count"], d["nn_index"], d["bin_index"], d["bin_coeff"])
    gin, gf = mo.pcloud_conv3d_backward(d["g_out"], d["x"], d["filt"], d["nn_count"], d["nn_index"], d["bin_index"],
                                        d["bin_coeff"])
    assert rel_err(out, z["ref_out"]) <= 1e-5 and rel_err(gin, z["ref_gin"]) <= 1e-5 and rel_err(gf, z["ref_gf"]) <= 1e-5
    c_out = co.pcloud_forward(_n(d["x"]), _n(d["filt"]), _n(d["nn_count"]), _n(d["nn_index"]), _n(d["bin_index"]),
                              _n(d["bin_coeff"]))
    assert rel_err(c_out, z["ref_out"]) <= 1e-5
