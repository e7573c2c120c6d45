"""Mesh decimation: the sequential restatement (oracle/decimate_oracle.c) against fixtures recorded from
the reference's own kernels (decimate_gpu.cu, two chained passes and the cluster merge), and the
properties every clustering must have."""
import os

import numpy as np
import pytest

from cases import DECIMATE_CASES, DECIMATE_GOLDEN_CASES, decimate_inputs
from oracle import c_oracle

GOLDEN_DIR = os.path.join(os.path.dirname(os.path.abspath(__file__)), "golden")
INT_OUTPUTS = ("faceOut", "isDegenerate", "vtReplace", "vtMap", "nvOut", "mfOut")


def run_oracle(d, use_area, wgt_bnd):
    return c_oracle.mesh_simplify(d["vertex"].numpy(), d["face"].numpy(), d["geometry"].numpy(), d["nv_cum"].numpy(),
                                  d["mf_cum"].numpy(), d["remove"].numpy(), use_area, wgt_bnd)


@pytest.mark.parametrize("name", sorted(DECIMATE_GOLDEN_CASES))
def test_oracle_matches_reference_fixture(name):
    z = np.load(os.path.join(GOLDEN_DIR, name + ".npz"))
    meshes, frac, D, seed, noise, use_area, wgt_bnd = DECIMATE_GOLDEN_CASES[name]
    d = decimate_inputs(meshes, frac, D, seed, noise)
    for k, v in d.items():                                   # the fixture's inputs are the generator's
        assert np.array_equal(v.numpy(), z["in_" + k]), k
    for tag, pre in (("ref1_", "in_"), ("ref2_", "in2_")):
        o = c_oracle.mesh_simplify(z[pre + "vertex"], z[pre + "face"], z[pre + "geometry"], z[pre + "nv_cum"],
                                   z[pre + "mf_cum"], z[pre + "remove"], bool(z["use_area"]), float(z["wgt_bnd"]))
        for k in INT_OUTPUTS:
            assert np.array_equal(o[k], z[tag + k]), (tag, k)
        # the reference adds the members of a cluster with float atomics: last-bit differences
        assert np.abs(o["vertexOut"] - z[tag + "vertexOut"]).max() <= 1e-6
    rep, mp = c_oracle.combine_clusters(z["ref1_vtReplace"], z["ref1_vtMap"], z["ref2_vtReplace"], z["ref2_vtMap"])
    assert np.array_equal(rep, z["ref_comb_rep"]) and np.array_equal(mp, z["ref_comb_map"])


@pytest.mark.parametrize("name", sorted(DECIMATE_CASES))
def test_clustering_properties(name):
    meshes, frac, D, seed, noise, use_area, wgt_bnd = DECIMATE_CASES[name]
    d = decimate_inputs(meshes, frac, D, seed, noise)
    if name == "one_sample_skipped":
        d["remove"][1] = 0
    o = run_oracle(d, use_area, wgt_bnd)
    rep, vmap = o["vtReplace"], o["vtMap"]
    nv = d["nv"].numpy()
    bounds = np.concatenate([[0], np.cumsum(nv)])
    removed = rep < 0
    roots = -rep[removed]
    assert (rep[roots] > 0).all()                                            # contracted into representatives only
    assert np.array_equal(np.bincount(roots, minlength=rep.shape[0])[~removed], rep[~removed])   # sizes add up
    for s in range(nv.shape[0]):
        seg = slice(bounds[s], bounds[s + 1])
        assert removed[seg].sum() <= max(int(d["remove"][s]), 0)             # never more than asked
        assert ((roots[(np.nonzero(removed)[0] >= bounds[s]) & (np.nonzero(removed)[0] < bounds[s + 1])] >= bounds[s]).all())
        assert o["nvOut"][s] == (vmap[seg] >= 0).sum()
        kept_ids = vmap[seg][vmap[seg] >= 0]
        assert np.array_equal(kept_ids, np.arange(kept_ids.shape[0]) + (vmap[:bounds[s]] >= 0).sum())
    assert (vmap[removed] == -1).all()
    good = ~o["isDegenerate"]
    fo = o["faceOut"][good]
    assert fo.min() >= 0 and fo.max() < o["nvOut"].sum()
    assert (fo[:, 0] != fo[:, 1]).all() and (fo[:, 0] != fo[:, 2]).all() and (fo[:, 1] != fo[:, 2]).all()
    assert o["mfOut"].sum() == good.sum()
    if name == "one_sample_skipped":                                         # a sample with nothing to remove is untouched
        seg = slice(bounds[1], bounds[2])
        assert (rep[seg] == 0).all()
        assert np.array_equal(o["vertexOut"][seg], d["vertex"].numpy()[seg])
    # cluster means
    vin = d["vertex"].numpy().astype(np.float64)
    for r in np.unique(roots)[:50]:
        members = np.nonzero(rep == -r)[0]
        mean = (vin[members].sum(0) + vin[r]) / (members.shape[0] + 1)
        assert np.allclose(o["vertexOut"][r], mean, atol=1e-5)


def test_merge_composes_two_passes():
    meshes, frac, D, seed, noise, use_area, wgt_bnd = DECIMATE_CASES["two_sweeps"]
    d = decimate_inputs(meshes, frac, D, seed, noise)
    a = run_oracle(d, use_area, wgt_bnd)
    keep = a["vtMap"] >= 0
    v2 = a["vertexOut"][keep]
    f2 = a["faceOut"][~a["isDegenerate"]]
    g2 = c_oracle.triangle_geometry(v2[:, :3].copy(), f2)
    b = c_oracle.mesh_simplify(v2, f2, g2, np.cumsum(a["nvOut"]).astype(np.int32), np.cumsum(a["mfOut"]).astype(np.int32),
                               (a["nvOut"] // 2).astype(np.int32), use_area, wgt_bnd)
    rep, mp = c_oracle.combine_clusters(a["vtReplace"], a["vtMap"], b["vtReplace"], b["vtMap"])
    nA = rep.shape[0]
    for v in range(nA):
        ra = -a["vtReplace"][v] if a["vtReplace"][v] < 0 else v            # representative after the first pass
        vb = a["vtMap"][ra]
        if vb < 0:
            continue                                                        # dropped with its degenerate faces
        rb = -b["vtReplace"][vb] if b["vtReplace"][vb] < 0 else vb          # representative after the second
        coarse = b["vtMap"][rb]
        r = -rep[v] if rep[v] < 0 else v
        assert mp[r] == coarse, v
    removed = rep < 0
    roots = -rep[removed]
    assert np.array_equal(np.bincount(roots, minlength=nA)[~removed], rep[~removed])
