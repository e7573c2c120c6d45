"""Mesh pooling / unpooling kernels, called through the C ABI (via the operator API that mirrors
picasso/mesh/pi_modules/pool3d.py and unpool3d.py), against the oracle and the reference's own
CUDA kernels on identical seeded inputs.  Gates: values selected or copied (max pool, its backward,
average-pool backward, unpool forward) bit-exact, max indices bit-exact, sums (average pool
forward, unpool backward) <= 1e-6 relative (the reference adds with float atomics)."""
import numpy as np
import pytest
import torch

from cases import POOL_GOLDEN_CASES, cluster_inputs
from conftest import max_abs, rel_err

pytestmark = pytest.mark.gpu

CASES = [
    # NvIn, NvOut, C, ties
    (300, 90, 8, False),
    (257, 64, 5, False),          # scalar path (C not a multiple of 4)
    (64, 64, 4, False),           # every vertex its own cluster
    (5000, 700, 128, False),
    (20000, 5000, 64, True),      # equal maxima inside clusters
    (40, 1, 12, False),           # one cluster
]


def _dev(d):
    return {k: (v.cuda() if isinstance(v, torch.Tensor) else v) for k, v in d.items()}


@pytest.fixture(scope="module")
def mods():
    from picassoplus_b200.mesh.pi_modules import pool3d, unpool3d
    from oracle import mesh_oracle, ref_cuda
    return pool3d, unpool3d, mesh_oracle, ref_cuda


@pytest.mark.parametrize("nv_in,nv_out,C,ties", CASES)
def test_pool_and_unpool_match_oracle_and_reference(mods, nv_in, nv_out, C, ties):
    pool3d, unpool3d, mo, ref = mods
    d = cluster_inputs(nv_in, nv_out, C, seed=17, ties=ties)
    c = _dev(d)
    vt_out = torch.zeros(nv_out, 3, device="cuda")
    out, idx = pool3d.max_forward(c["x"], c["vt_replace"], c["vt_map"], vt_out)
    w_out, w_idx = mo.mesh_max_pool_forward(d["x"], d["vt_replace"], d["vt_map"], nv_out)
    assert torch.equal(out.cpu(), w_out) and torch.equal(idx.cpu(), w_idx)
    gin = pool3d.max_backward(c["g_coarse"], c["x"], idx)
    assert torch.equal(gin.cpu(), mo.mesh_max_pool_backward(d["g_coarse"], nv_in, w_idx))
    _, _, clusters = pool3d.max_forward(c["x"], c["vt_replace"], c["vt_map"], vt_out, return_clusters=True)
    assert torch.equal(pool3d.max_backward(c["g_coarse"], c["x"], idx, clusters), gin)     # the gather form
    avg = pool3d.avg_forward(c["x"], c["vt_replace"], c["vt_map"], vt_out)
    assert rel_err(avg, mo.mesh_avg_pool_forward(d["x"].double(), d["vt_replace"], d["vt_map"], nv_out)) <= 1e-6
    avg_b = pool3d.avg_backward(c["g_coarse"], c["x"], c["vt_replace"], c["vt_map"])
    assert torch.equal(avg_b.cpu(), mo.mesh_avg_pool_backward(d["g_coarse"], d["vt_replace"], d["vt_map"]))
    up = unpool3d.forward(c["x_coarse"], c["vt_replace"], c["vt_map"])
    assert torch.equal(up.cpu(), mo.mesh_unpool_forward(d["x_coarse"], d["vt_replace"], d["vt_map"]))
    up_b = unpool3d.backward(c["g_fine"], c["x_coarse"], c["vt_replace"], c["vt_map"])
    assert rel_err(up_b, mo.mesh_unpool_backward(d["g_fine"].double(), nv_out, d["vt_replace"], d["vt_map"])) <= 1e-6
    # run to run identical
    assert torch.equal(avg, pool3d.avg_forward(c["x"], c["vt_replace"], c["vt_map"], vt_out))
    assert torch.equal(up_b, unpool3d.backward(c["g_fine"], c["x_coarse"], c["vt_replace"], c["vt_map"]))
    if ref.available():
        r_out, r_idx = ref.max_pool_forward(c["x"], c["vt_replace"], c["vt_map"], nv_out)
        assert torch.equal(out, r_out)
        if not ties:
            assert torch.equal(idx, r_idx)
            assert torch.equal(gin, ref.max_pool_backward(c["g_coarse"], nv_in, r_idx))
        else:       # the reference's index among equal maxima depends on its thread order: any attaining member is right
            picked = torch.gather(c["x"], 0, r_idx.long())
            assert torch.equal(picked, r_out)
        assert rel_err(avg, ref.avg_pool_forward(c["x"], c["vt_replace"], c["vt_map"], nv_out)) <= 1e-6
        assert torch.equal(avg_b, ref.avg_pool_backward(c["g_coarse"], c["vt_replace"], c["vt_map"]))
        assert torch.equal(up, ref.unpool_forward(c["x_coarse"], c["vt_replace"], c["vt_map"]))
        assert rel_err(up_b, ref.unpool_backward(c["g_fine"], nv_out, c["vt_replace"], c["vt_map"])) <= 1e-6


@pytest.mark.parametrize("name", sorted(POOL_GOLDEN_CASES))
def test_against_committed_reference_fixtures(mods, name):
    import os
    pool3d, unpool3d, _, _ = mods
    path = os.path.join(os.path.dirname(__file__), "golden", name + ".npz")
    z = np.load(path)
    nv_in, nv_out, C, seed = POOL_GOLDEN_CASES[name]
    c = _dev(cluster_inputs(nv_in, nv_out, C, seed))
    vt_out = torch.zeros(nv_out, 3, device="cuda")
    out, idx = pool3d.max_forward(c["x"], c["vt_replace"], c["vt_map"], vt_out)
    assert max_abs(out, z["ref_max_out"]) == 0.0 and np.array_equal(idx.cpu().numpy(), z["ref_max_index"])
    assert max_abs(pool3d.max_backward(c["g_coarse"], c["x"], idx), z["ref_max_gin"]) == 0.0
    assert rel_err(pool3d.avg_forward(c["x"], c["vt_replace"], c["vt_map"], vt_out), z["ref_avg_out"]) <= 1e-6
    assert max_abs(pool3d.avg_backward(c["g_coarse"], c["x"], c["vt_replace"], c["vt_map"]), z["ref_avg_gin"]) == 0.0
    assert max_abs(unpool3d.forward(c["x_coarse"], c["vt_replace"], c["vt_map"]), z["ref_unpool_out"]) == 0.0
    assert rel_err(unpool3d.backward(c["g_fine"], c["x_coarse"], c["vt_replace"], c["vt_map"]), z["ref_unpool_gin"]) <= 1e-6


def test_autograd_through_pool_layers(mods):
    """Pool3d / Unpool3d modules: gradients of max, avg and unpool through torch autograd against the
    oracle's explicit backward formulas."""
    from picassoplus_b200.mesh.layers import Pool3d, Unpool3d
    _, _, mo, _ = mods
    d = cluster_inputs(900, 250, 16, seed=23)
    c = _dev(d)
    vt_out = torch.zeros(250, 3, device="cuda")
    for method in ("max", "avg"):
        x = c["x"].clone().requires_grad_()
        y = Pool3d(method)(x, c["vt_replace"], c["vt_map"], vt_out)
        y.backward(c["g_coarse"])
        if method == "max":
            _, idx = mo.mesh_max_pool_forward(d["x"], d["vt_replace"], d["vt_map"], 250)
            want = mo.mesh_max_pool_backward(d["g_coarse"], 900, idx)
        else:
            want = mo.mesh_avg_pool_backward(d["g_coarse"], d["vt_replace"], d["vt_map"])
        assert torch.equal(x.grad.cpu(), want)
    xc = c["x_coarse"].clone().requires_grad_()
    Unpool3d()(xc, c["vt_replace"], c["vt_map"]).backward(c["g_fine"])
    assert rel_err(xc.grad, mo.mesh_unpool_backward(d["g_fine"].double(), 250, d["vt_replace"], d["vt_map"])) <= 1e-6


def test_max_pool_gradient_with_memberless_coarse_vertices(mods):
    """More output rows than clusters: the extra coarse vertices have no members, record index 0 and hand their
    gradient to vertex 0 (picasso/mesh/pi_modules/source/mesh_pool3d_gpu.cu:93-105); the gather form does the same.
    Vertex 0 belongs to no cluster here, so no two writers meet there."""
    pool3d, _, mo, _ = mods
    d = cluster_inputs(400, 120, 8, seed=7)
    assert int(d["vt_map"][0]) < 0 and int(d["vt_replace"][0]) == 0       # this seed leaves vertex 0 outside every cluster
    c = _dev(d)
    nv_out = 121
    vt_out = torch.zeros(nv_out, 3, device="cuda")
    g = torch.randn(nv_out, 8, device="cuda")
    out, idx, clusters = pool3d.max_forward(c["x"], c["vt_replace"], c["vt_map"], vt_out, return_clusters=True)
    assert torch.all(out[120] == 0) and torch.all(idx[120] == 0)
    scatter = pool3d.max_backward(g, c["x"], idx)
    gather = pool3d.max_backward(g, c["x"], idx, clusters)
    assert torch.equal(scatter, gather) and torch.equal(gather[0], g[120])
    assert torch.equal(gather.cpu(), mo.mesh_max_pool_backward(g.cpu(), 400, idx.cpu()))


def test_bad_cluster_indices_are_reported(mods):
    pool3d, _, _, _ = mods
    c = _dev(cluster_inputs(100, 30, 4, seed=1))
    bad = c["vt_replace"].clone()
    bad[5] = -10 ** 6
    with pytest.raises(RuntimeError):
        pool3d.avg_forward(c["x"], bad, c["vt_map"], torch.zeros(30, 3, device="cuda"))
    assert torch.isfinite(pool3d.avg_forward(c["x"], c["vt_replace"], c["vt_map"], torch.zeros(30, 3, device="cuda"))).all()


@pytest.mark.parametrize("kind,L,orient", [("grid17x2", 4, False), ("grid17x2+drop", 3, True), ("ico2x3", 2, True),
                                           ("tet+iso", 5, True)])
def test_level_prepare_matches_the_separate_calls(kind, L, orient):
    """pb200_level_prepare (one fused pass per mesh level) against the separate entry points, the
    oracle, and the CSR built by pb200_build_vertex_csr: geometry and basis bit-identical to the
    separate kernels, nfCount and CSR bit-exact."""
    from cases import conv_inputs
    from oracle import mesh_oracle as mo
    from picassoplus_b200 import topology
    from picassoplus_b200.math_utils import sph_harm_coeff
    from picassoplus_b200.mesh.pi_modules import decimate
    d = conv_inputs(kind, 4, 1, 4, 2, seed=33)
    vertex = (d["vertex"] - 0.5).cuda()             # centre the meshes on the origin so both orientations occur
    face, vt_map = d["face"].cuda(), d["vt_map"].cuda()
    topology.clear_cache()
    got = topology.prepare_level(vertex, face, vt_map, d["nv_out"], L, orient=orient, want_normals=True)
    geo = decimate.compute_triangle_geometry_(vertex, face)
    assert torch.equal(got["geometry"], geo)
    want_n = mo.oriented_normals(geo.cpu(), vertex.cpu(), d["face"]) if orient else geo[:, :3].cpu()
    assert torch.equal(got["normals"].cpu(), want_n)
    if orient:
        assert (want_n != geo[:, :3].cpu()).any()            # the case does flip some normals
    assert torch.equal(got["coeff"], sph_harm_coeff(L, got["normals"]))
    assert max_abs(got["coeff"], mo.sph_harm_coeff(L, want_n)) <= 2e-6
    assert torch.equal(got["nf_count"].cpu(), mo.count_vertex_adjface(d["face"], d["vt_map"], d["nv_out"]))
    ref_csr = topology.build_vertex_csr(face, vt_map, d["vt_map"].shape[0], d["nv_out"])
    assert torch.equal(got["csr"].rowptr, ref_csr.rowptr)
    n = int(ref_csr.rowptr[-1])
    assert torch.equal(got["csr"].entries[:n], ref_csr.entries[:n])
    assert topology.vertex_csr(face, vt_map, d["vt_map"].shape[0], d["nv_out"]) is got["csr"]     # served from the cache
