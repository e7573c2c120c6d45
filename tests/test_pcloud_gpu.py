"""Point-cloud depthwise convolution (hard and fuzzy bins), called through the C ABI (via the
operator API that mirrors picasso/point/pi_modules/conv3d.py), against the fp64 oracle and the
reference's own CUDA kernels on identical seeded inputs; gate 1e-4 relative per tensor."""
import os

import numpy as np
import pytest
import torch

from cases import PCLOUD_GOLDEN_CASES, pcloud_inputs
from conftest import rel_err

pytestmark = pytest.mark.gpu
TOL = 1e-4

CASES = [
    # Np, Mp, knn, F, C, r, T (0 = hard bins), shuffle
    (200, 60, 12, 9, 6, 2, 0, False),
    (150, 80, 10, 17, 8, 1, 3, False),
    (3000, 1000, 24, 33, 64, 1, 3, True),
    (4000, 4000, 16, 17, 128, 1, 0, False),
    (64, 16, 40, 5, 3, 3, 2, True),
    (2500, 700, 20, 51, 32, 1, 3, True),       # eight lanes per point: four points to a warp
    (900, 300, 37, 25, 12, 1, 0, True),        # four channels per lane without the warp-cooperative walk
    (700, 200, 70, 140, 128, 1, 3, False),     # runs longer than a warp; a filter table the cooperative kernels decline
]


def _dev(d):
    return {k: (v.cuda() if isinstance(v, torch.Tensor) else v) for k, v in d.items()}


@pytest.mark.parametrize("Np,Mp,knn,F,C,r,T,shuffle", CASES)
def test_matches_oracle_and_reference(Np, Mp, knn, F, C, r, T, shuffle):
    from oracle import mesh_oracle as mo, ref_cuda as ref
    from picassoplus_b200.point.pi_modules import conv3d
    d = pcloud_inputs(Np, Mp, knn, F, C, r, T, seed=19, shuffle=shuffle)
    c = _dev(d)
    dbl = lambda t: None if t is None else t.double()                               # noqa: E731
    want = mo.pcloud_conv3d_forward(d["x"].double(), d["filt"].double(), d["nn_count"], d["nn_index"], d["bin_index"],
                                    dbl(d["bin_coeff"]))
    wgin, wgf = mo.pcloud_conv3d_backward(d["g_out"].double(), d["x"].double(), d["filt"].double(), d["nn_count"],
                                          d["nn_index"], d["bin_index"], dbl(d["bin_coeff"]))
    if T == 0:
        out = conv3d.SPH3D_forward(c["x"], c["filt"], c["nn_count"], c["nn_index"], c["bin_index"])
        gin, gf = conv3d.SPH3D_backward(c["g_out"], c["x"], c["filt"], c["nn_count"], c["nn_index"], c["bin_index"])
    else:
        out = conv3d.fuzzySPH3D_forward(c["x"], c["filt"], c["nn_count"], c["nn_index"], c["bin_index"], c["bin_coeff"])
        gin, gf = conv3d.fuzzySPH3D_backward(c["g_out"], c["x"], c["filt"], c["nn_count"], c["nn_index"], c["bin_index"],
                                             c["bin_coeff"])
    assert rel_err(out, want) <= TOL and rel_err(gin, wgin) <= TOL and rel_err(gf, wgf) <= TOL
    no_pairs = torch.bincount(d["nn_index"][:, 0].long(), minlength=Mp) == 0
    assert torch.all(out[no_pairs.cuda()] == 0)                  # output points without a neighbour stay exactly 0
    again = conv3d._backward(c["g_out"], c["x"], c["filt"], c["nn_count"], c["nn_index"], c["bin_index"], c["bin_coeff"])
    assert torch.equal(again[0], gin) and torch.equal(again[1], gf)                  # run to run identical
    if ref.available():
        r_out = ref.pcloud_forward(c["x"], c["filt"], c["nn_count"], c["nn_index"], c["bin_index"], c["bin_coeff"])
        r_gin, r_gf = ref.pcloud_backward(c["g_out"], c["x"], c["filt"], c["nn_count"], c["nn_index"], c["bin_index"],
                                          c["bin_coeff"])
        assert rel_err(out, r_out) <= TOL and rel_err(gin, r_gin) <= TOL and rel_err(gf, r_gf) <= TOL


@pytest.mark.parametrize("name", sorted(PCLOUD_GOLDEN_CASES))
def test_against_committed_reference_fixtures(name):
    from picassoplus_b200.point.pi_modules import conv3d
    z = np.load(os.path.join(os.path.dirname(__file__), "golden", name + ".npz"))
    c = _dev(pcloud_inputs(*PCLOUD_GOLDEN_CASES[name]))
    out = conv3d._forward(c["x"], c["filt"], c["nn_count"], c["nn_index"], c["bin_index"], c["bin_coeff"])
    gin, gf = conv3d._backward(c["g_out"], c["x"], c["filt"], c["nn_count"], c["nn_index"], c["bin_index"], c["bin_coeff"])
    assert rel_err(out, z["ref_out"]) <= TOL and rel_err(gin, z["ref_gin"]) <= TOL and rel_err(gf, z["ref_gf"]) <= TOL


def test_module_and_autograd():
    """PCloudConv3d (fuzzy bins) through torch autograd against the oracle composition in fp64."""
    from oracle import mesh_oracle as mo
    from picassoplus_b200.point.layers import PCloudConv3d
    d = pcloud_inputs(500, 300, 12, 17, 16, 2, 3, seed=23)
    c = _dev(d)
    torch.manual_seed(0)
    mod = PCloudConv3d(16, 24, 17, depth_multiplier=2, with_bn=False).cuda()
    x = c["x"].clone().requires_grad_()
    y = mod(x, c["nn_count"], c["nn_index"], c["bin_index"], c["bin_coeff"])
    G = torch.randn_like(y)
    (y * G).sum().backward()
    P = lambda t: t.detach().cpu().double()                                          # noqa: E731
    xo, sw = P(d["x"]).requires_grad_(), P(mod.spatial_weights).requires_grad_()
    f = mo.pcloud_conv3d_forward(xo, sw, d["nn_count"], d["nn_index"], d["bin_index"], d["bin_coeff"].double())
    yo = torch.relu(f @ P(mod.depth_weights) + P(mod.biases))
    (yo * P(G)).sum().backward()
    assert rel_err(y, yo) <= TOL and rel_err(x.grad, xo.grad) <= TOL and rel_err(mod.spatial_weights.grad, sw.grad) <= TOL
