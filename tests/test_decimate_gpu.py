"""Mesh decimation through the C ABI (pb200_mesh_simplify, pb200_combine_clusters) against the sequential
restatement -- bit for bit, floats included --, against the fixtures recorded from the reference's kernels,
and against the reference's kernels themselves where they are present."""
import os

import numpy as np
import pytest
import torch

from cases import DECIMATE_CASES, DECIMATE_GOLDEN_CASES, decimate_inputs
from oracle import c_oracle, ref_cuda

pytestmark = pytest.mark.gpu

GOLDEN_DIR = os.path.join(os.path.dirname(os.path.abspath(__file__)), "golden")
NAMES = ("vertexOut", "faceOut", "isDegenerate", "vtReplace", "vtMap", "nvOut", "mfOut")
INT_OUTPUTS = NAMES[1:]


@pytest.fixture
def device():
    return torch.device("cuda:0")


def dm():
    from picassoplus_b200.mesh.pi_modules import decimate
    return decimate


def on(dev, a):
    return torch.from_numpy(np.ascontiguousarray(a)).to(dev)


def run_lib(dev, vertex, face, geometry, nv_cum, mf_cum, remove, use_area, wgt_bnd):
    outs, info, cost = dm().simplify(on(dev, vertex), on(dev, face), on(dev, geometry), on(dev, nv_cum), on(dev, mf_cum),
                                     on(dev, remove), use_area, wgt_bnd, return_info=True)
    torch.cuda.synchronize()
    res = {k: v.cpu().numpy() for k, v in zip(NAMES, outs)}
    res["edgeCost"] = cost.cpu().numpy()
    return res, info


def same_bits(a, b):
    return np.array_equal(np.ascontiguousarray(a).view(np.uint32), np.ascontiguousarray(b).view(np.uint32))


def check_against_oracle(dev, arrs, use_area, wgt_bnd):
    o = c_oracle.mesh_simplify(*arrs, use_area, wgt_bnd)
    g, info = run_lib(dev, *arrs, use_area, wgt_bnd)
    assert info[0] == o["edgeCost"].shape[0]
    assert same_bits(g["edgeCost"], o["edgeCost"])                       # every candidate's cost, to the bit
    for k in INT_OUTPUTS:
        assert np.array_equal(g[k], o[k]), k
    assert same_bits(g["vertexOut"], o["vertexOut"])
    return g, info


@pytest.mark.parametrize("name", sorted(DECIMATE_CASES))
def test_pass_equals_sequential_restatement(name, device):
    meshes, frac, D, seed, noise, use_area, wgt_bnd = DECIMATE_CASES[name]
    d = decimate_inputs(meshes, frac, D, seed, noise)
    if name == "one_sample_skipped":
        d["remove"][1] = 0
    arrs = [d[k].numpy() for k in ("vertex", "face", "geometry", "nv_cum", "mf_cum", "remove")]
    check_against_oracle(device, arrs, use_area, wgt_bnd)


@pytest.mark.parametrize("name", sorted(DECIMATE_GOLDEN_CASES))
def test_reference_fixture(name, device):
    z = np.load(os.path.join(GOLDEN_DIR, name + ".npz"))
    use_area, wgt_bnd = bool(z["use_area"]), float(z["wgt_bnd"])
    for tag, pre in (("ref1_", "in_"), ("ref2_", "in2_")):
        g, _ = run_lib(device, z[pre + "vertex"], z[pre + "face"], z[pre + "geometry"], z[pre + "nv_cum"], z[pre + "mf_cum"],
                       z[pre + "remove"], use_area, wgt_bnd)
        for k in INT_OUTPUTS:
            assert np.array_equal(g[k], z[tag + k]), (tag, k)
        assert np.abs(g["vertexOut"] - z[tag + "vertexOut"]).max() <= 1e-6
    rep, mp = dm().combine_clusters(on(device, z["ref1_vtReplace"]), on(device, z["ref1_vtMap"]),
                                    on(device, z["ref2_vtReplace"]), on(device, z["ref2_vtMap"]))
    assert np.array_equal(rep.cpu().numpy(), z["ref_comb_rep"]) and np.array_equal(mp.cpu().numpy(), z["ref_comb_map"])


@pytest.mark.skipif(not ref_cuda.available(), reason="reference kernels not built")
def test_live_reference_kernels(device):
    meshes, frac, D, seed, noise, use_area, wgt_bnd = DECIMATE_GOLDEN_CASES["decim_two_sweeps"]
    d = decimate_inputs(meshes, 0.5, 4, seed + 100, noise)
    c = {k: v.to(device) for k, v in d.items()}
    r = ref_cuda.mesh_simplify(c["vertex"], c["face"], c["geometry"], c["nv_cum"], c["mf_cum"], c["remove"], use_area, wgt_bnd)
    outs = dm().simplify(c["vertex"], c["face"], c["geometry"], c["nv_cum"], c["mf_cum"], c["remove"], use_area, wgt_bnd)
    for k, t in zip(NAMES, outs):
        if k == "vertexOut":
            assert (t - r[k]).abs().max().item() <= 1e-6
        else:
            assert torch.equal(t, r[k]), k
    rep_b = torch.zeros(int(r["nvOut"].sum()), dtype=torch.int32, device=device)
    map_b = torch.arange(rep_b.shape[0], dtype=torch.int32, device=device)
    mine = dm().combine_clusters(r["vtReplace"], r["vtMap"], rep_b, map_b)
    ref = ref_cuda.combine_clusters(r["vtReplace"], r["vtMap"], rep_b, map_b)
    assert torch.equal(mine[0], ref[0]) and torch.equal(mine[1], ref[1])


def planar_grid(n):
    """n x n vertices in a plane, regular triangulation: every candidate has the same cost, so ranks follow
    the edge order and the greedy sweep is one long dependency chain along every row."""
    ii, jj = np.meshgrid(np.arange(n), np.arange(n), indexing="ij")
    v = np.stack([ii, jj, np.zeros_like(ii)], -1).reshape(-1, 3).astype(np.float32) / n
    idx = lambda i, j: i * n + j
    f = []
    for i in range(n - 1):
        for j in range(n - 1):
            f.append((idx(i, j), idx(i + 1, j), idx(i, j + 1)))
            f.append((idx(i + 1, j), idx(i + 1, j + 1), idx(i, j + 1)))
    return v, np.array(f, np.int32)


@pytest.mark.parametrize("n,frac", [(40, 0.75), (150, 0.75), (150, 0.1)])
def test_equal_costs_long_chains(n, frac, device):
    v, f = planar_grid(n)
    geo = c_oracle.triangle_geometry(v, f)
    arrs = [v, f, geo, np.array([v.shape[0]], np.int32), np.array([f.shape[0]], np.int32),
            np.array([int(v.shape[0] * frac)], np.int32)]
    g, info = check_against_oracle(device, arrs, True, 5.0)
    assert (g["vtReplace"] < 0).sum() > 0


def random_soup(rng, nv, nf, B):
    """B samples of random triangles over random points: non-manifold edges (shared by three and more faces),
    duplicate faces, faces that name a vertex twice, isolated vertices, many boundary edges."""
    vs, fs, nvs, mfs, off = [], [], [], [], 0
    for _ in range(B):
        n, m = int(rng.integers(nv // 2, nv + 1)), int(rng.integers(nf // 2, nf + 1))
        v = rng.standard_normal((n, 3)).astype(np.float32)
        f = rng.integers(0, n, size=(m, 3)).astype(np.int32)
        f[: m // 8] = f[m // 8: 2 * (m // 8)]                 # duplicates
        f[-3:, 1] = f[-3:, 0]                                 # a vertex named twice
        vs.append(v); fs.append(f + off); nvs.append(n); mfs.append(m); off += n
    return np.concatenate(vs), np.concatenate(fs), np.array(nvs, np.int32), np.array(mfs, np.int32)


@pytest.mark.parametrize("seed", range(6))
def test_random_triangle_soups(seed, device):
    rng = np.random.default_rng(100 + seed)
    B = int(rng.integers(1, 5))
    v, f, nv, mf = random_soup(rng, 120, 300, B)
    geo = c_oracle.triangle_geometry(v, f)
    frac = [0.05, 0.3, 0.6, 0.9, 0.5, 0.75][seed]
    remove = np.floor(nv * frac).astype(np.int32)
    if B > 1:
        remove[0] = 0                                          # one sample left alone
    arrs = [v, f, geo, np.cumsum(nv).astype(np.int32), np.cumsum(mf).astype(np.int32), remove]
    check_against_oracle(device, arrs, bool(seed % 2), [0.0, 1.0, 5.0][seed % 3])


def test_degenerate_sizes(device):
    # a batch whose second sample has no face at all, nothing to remove anywhere, a single triangle
    v = np.array([[0, 0, 0], [1, 0, 0], [0, 1, 0], [5, 5, 5], [6, 5, 5]], np.float32)
    f = np.array([[0, 1, 2]], np.int32)
    geo = c_oracle.triangle_geometry(v, f)
    for remove in ([0, 0], [1, 1], [3, 2]):
        arrs = [v, f, geo, np.array([3, 5], np.int32), np.array([1, 1], np.int32), np.array(remove, np.int32)]
        check_against_oracle(device, arrs, True, 5.0)


def oracle_decimation(d, nv_out, use_area, wgt_bnd):
    """The pass loop of picasso/mesh/pi_modules/decimate.py:30-46 on the restatement."""
    vertex, face, geo = d["vertex"].numpy(), d["face"].numpy(), d["geometry"].numpy()
    nv, mf = d["nv"].numpy().copy(), d["mf"].numpy().copy()
    remove = nv - nv_out
    rep = np.zeros(vertex.shape[0], np.int32)
    mp = np.arange(vertex.shape[0], dtype=np.int32)
    while (remove > 0).any():
        o = c_oracle.mesh_simplify(vertex, face, geo, np.cumsum(nv).astype(np.int32), np.cumsum(mf).astype(np.int32),
                                   remove.astype(np.int32), use_area, wgt_bnd)
        if not ((nv - o["nvOut"]) > 0).any():
            break
        face = o["faceOut"][~o["isDegenerate"]]
        vertex = o["vertexOut"][o["vtMap"] >= 0]
        geo = c_oracle.triangle_geometry(vertex[:, :3].copy(), face)
        remove = remove - (nv - o["nvOut"])
        rep, mp = c_oracle.combine_clusters(rep, mp, o["vtReplace"], o["vtMap"])
        nv, mf = o["nvOut"], o["mfOut"]
    return vertex, face, nv, mf, rep, mp


def test_whole_decimation_loop(device):
    meshes, frac, D, seed, noise, use_area, wgt_bnd = DECIMATE_CASES["larger"]
    d = decimate_inputs(meshes, frac, D, seed, noise)
    c = {k: v.to(device) for k, v in d.items()}
    nv_out = c["nv"] - c["remove"]
    # geometry as the library computes it (the loop recomputes it with the library after every pass)
    geo = dm().compute_triangle_geometry_(c["vertex"], c["face"])
    d["geometry"] = geo.cpu()
    res = dm().mesh_decimation_(c["vertex"], c["face"], geo, c["nv"], c["mf"], nv_out, use_area, wgt_bnd)
    vertex, face, geometry, nv, mf, rep, mp = [t.cpu().numpy() for t in res]
    assert (nv <= nv_out.cpu().numpy()).all() and (nv >= nv_out.cpu().numpy() - 8).all()
    assert face.max() < vertex.shape[0] and vertex.shape[0] == nv.sum() and face.shape[0] == mf.sum()
    # clusters over the input vertices: every representative maps to an output vertex, sizes add up
    removed = rep < 0
    roots = -rep[removed]
    assert np.array_equal(np.bincount(roots, minlength=rep.shape[0])[~removed], rep[~removed])
    assert (mp[removed] == -1).all() and np.array_equal(np.sort(mp[mp >= 0]), np.arange(vertex.shape[0]))
    assert geometry.shape == (face.shape[0], 5)


def test_bad_arguments(device):
    meshes, frac, D, seed, noise, use_area, wgt_bnd = DECIMATE_GOLDEN_CASES["decim_medium"]
    d = decimate_inputs(meshes, frac, D, seed, noise)
    c = {k: v.to(device) for k, v in d.items()}
    bad_face = c["face"].clone()
    bad_face[5, 1] = c["vertex"].shape[0] + 3
    with pytest.raises(RuntimeError, match="outside"):
        dm().simplify(c["vertex"], bad_face, c["geometry"], c["nv_cum"], c["mf_cum"], c["remove"], True, 5.0)
    with pytest.raises(RuntimeError, match="running totals"):
        dm().simplify(c["vertex"], c["face"], c["geometry"], c["nv"], c["mf_cum"], c["remove"], True, 5.0)
    with pytest.raises(RuntimeError, match="Nf, 5"):
        dm().simplify(c["vertex"], c["face"], c["geometry"][:, :4].contiguous(), c["nv_cum"], c["mf_cum"], c["remove"], True, 5.0)
    # the library still works afterwards
    outs = dm().simplify(c["vertex"], c["face"], c["geometry"], c["nv_cum"], c["mf_cum"], c["remove"], True, 5.0)
    assert int(outs[5].sum()) < c["vertex"].shape[0]
