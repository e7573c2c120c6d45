"""The two restatements of mesh pooling / unpooling (torch and plain C) against each other, against
hand-made known answers, and - when present - against the fixtures recorded from the reference's own
CUDA kernels (tests/golden/pool_*.npz, made by tests/golden/make_golden.py on a GPU)."""
import os

import numpy as np
import pytest
import torch

from cases import POOL_GOLDEN_CASES, cluster_inputs
from conftest import max_abs, rel_err
from oracle import c_oracle as co
from oracle import mesh_oracle as mo

GOLDEN_DIR = os.path.join(os.path.dirname(__file__), "golden")


def _both(d):
    vr, vm, x = d["vt_replace"], d["vt_map"], d["x"]
    py = dict(maxp=mo.mesh_max_pool_forward(x, vr, vm, d["nv_out"]),
              avg=mo.mesh_avg_pool_forward(x, vr, vm, d["nv_out"]),
              avg_b=mo.mesh_avg_pool_backward(d["g_coarse"], vr, vm),
              unp=mo.mesh_unpool_forward(d["x_coarse"], vr, vm),
              unp_b=mo.mesh_unpool_backward(d["g_fine"], d["nv_out"], vr, vm))
    py["max_b"] = mo.mesh_max_pool_backward(d["g_coarse"], d["nv_in"], py["maxp"][1])
    n = lambda t: t.numpy()                                                           # noqa: E731
    c = dict(maxp=co.max_pool_forward(n(x), n(vr), n(vm), d["nv_out"]),
             avg=co.avg_pool_forward(n(x), n(vr), n(vm), d["nv_out"]),
             avg_b=co.avg_pool_backward(n(d["g_coarse"]), n(vr), n(vm)),
             unp=co.unpool_forward(n(d["x_coarse"]), n(vr), n(vm)),
             unp_b=co.unpool_backward(n(d["g_fine"]), d["nv_out"], n(vr), n(vm)))
    c["max_b"] = co.max_pool_backward(n(d["g_coarse"]), d["nv_in"], c["maxp"][1])
    return py, c


@pytest.mark.parametrize("nv_in,nv_out,C,ties", [(300, 90, 8, False), (257, 64, 5, False), (64, 64, 4, False),
                                                (500, 40, 3, True)])
def test_restatements_agree(nv_in, nv_out, C, ties):
    d = cluster_inputs(nv_in, nv_out, C, seed=7, ties=ties)
    py, c = _both(d)
    assert torch.equal(py["maxp"][0], torch.from_numpy(c["maxp"][0]))
    assert torch.equal(py["maxp"][1], torch.from_numpy(c["maxp"][1]))            # smallest id among ties in both
    for k in ("max_b", "avg_b", "unp"):
        assert torch.equal(py[k], torch.from_numpy(c[k])), k
    for k in ("avg", "unp_b"):
        assert rel_err(py[k], c[k]) <= 1e-6, k


def test_known_answers():
    # vertices 1..4: cluster {1,3,4} with representative 3 -> coarse 1; vertex 0 alone -> coarse 0; vertex 2 dropped
    vr = torch.tensor([0, -3, 0, 2, -3], dtype=torch.int32)
    vm = torch.tensor([0, -1, -1, 1, -1], dtype=torch.int32)
    x = torch.tensor([[1.0, -1.0], [5.0, 0.0], [9.0, 9.0], [2.0, 7.0], [3.0, 7.0]])
    out, idx = mo.mesh_max_pool_forward(x, vr, vm, 2)
    assert torch.equal(out, torch.tensor([[1.0, -1.0], [5.0, 7.0]]))
    assert torch.equal(idx, torch.tensor([[0, 0], [1, 3]], dtype=torch.int32))     # tie at 7.0 -> smaller id 3
    avg = mo.mesh_avg_pool_forward(x, vr, vm, 2)
    assert torch.allclose(avg, torch.tensor([[1.0, -1.0], [10.0 / 3, 14.0 / 3]]))
    up = mo.mesh_unpool_forward(torch.tensor([[1.0], [2.0]]), vr, vm)
    assert torch.equal(up, torch.tensor([[1.0], [2.0], [0.0], [2.0], [2.0]]))
    g = torch.arange(5, dtype=torch.float32).reshape(5, 1)
    assert torch.equal(mo.mesh_unpool_backward(g, 2, vr, vm), torch.tensor([[0.0], [8.0]]))
    assert torch.equal(mo.mesh_avg_pool_backward(torch.tensor([[3.0], [6.0]]), vr, vm),
                       torch.tensor([[3.0], [2.0], [0.0], [2.0], [2.0]]))


def test_backward_formulas_are_the_adjoints():
    d = cluster_inputs(120, 30, 4, seed=3)
    vr, vm = d["vt_replace"], d["vt_map"]
    x, gc, xc, gf = d["x"].double(), d["g_coarse"].double(), d["x_coarse"].double(), d["g_fine"].double()
    # <avg(x), g> == <x, avg_b(g)>,  <unpool(xc), gf> == <xc, unpool_b(gf)>
    assert abs(float((mo.mesh_avg_pool_forward(x, vr, vm, 30) * gc).sum() - (x * mo.mesh_avg_pool_backward(gc, vr, vm)).sum())) < 1e-9
    assert abs(float((mo.mesh_unpool_forward(xc, vr, vm) * gf).sum() - (xc * mo.mesh_unpool_backward(gf, 30, vr, vm)).sum())) < 1e-9


@pytest.mark.parametrize("name", sorted(POOL_GOLDEN_CASES))
def test_oracle_matches_reference_kernels(name):
    path = os.path.join(GOLDEN_DIR, name + ".npz")
    assert os.path.exists(path), "fixture missing: run tests/golden/make_golden.py on a GPU"
    z = np.load(path)
    nv_in, nv_out, C, seed = POOL_GOLDEN_CASES[name]
    d = cluster_inputs(nv_in, nv_out, C, seed)
    for k in ("vt_replace", "vt_map", "x", "g_coarse", "x_coarse", "g_fine"):
        assert torch.equal(d[k], torch.from_numpy(z["in_" + k])), k            # inputs reproducible from the seed
    py, c = _both(d)
    for impl in (py, c):
        assert max_abs(impl["maxp"][0], z["ref_max_out"]) == 0.0
        assert np.array_equal(np.asarray(impl["maxp"][1]), z["ref_max_index"])  # no ties in these inputs: bit-exact
        assert max_abs(impl["max_b"], z["ref_max_gin"]) == 0.0
        assert rel_err(impl["avg"], z["ref_avg_out"]) <= 1e-6
        assert max_abs(impl["avg_b"], z["ref_avg_gin"]) == 0.0
        assert max_abs(impl["unp"], z["ref_unpool_out"]) == 0.0
        assert rel_err(impl["unp_b"], z["ref_unpool_gin"]) <= 1e-6
