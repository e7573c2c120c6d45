"""CPU tests of the checkers themselves: the torch oracle and the plain-C oracle against
the fixtures recorded from the reference's own CUDA operators (tests/golden/*.npz), against
each other, against analytic known answers, and fp64 gradcheck of the backward formulas."""
import glob
import math
import os

import numpy as np
import pytest
import torch

from conftest import rel_err, max_abs
from cases import GOLDEN_CASES, conv_inputs
from oracle import mesh_oracle as mo, c_oracle as co

# fixtures of the reference's CUDA operators, one per case of GOLDEN_CASES (the fixture of the
# reference's Python modules has its own test file)
GOLDEN = sorted(p for p in glob.glob(os.path.join(os.path.dirname(__file__), "golden", "*.npz"))
                if os.path.basename(p)[:-4] in GOLDEN_CASES)
TOL = 1e-4


def _load(path):
    z = np.load(path)
    i = {k[3:]: torch.from_numpy(z[k]) for k in z.files if k.startswith("in_")}
    r = {k[4:]: torch.from_numpy(z[k]) for k in z.files if k.startswith("ref_")}
    return i, r, int(z["nv_out"])


def test_golden_fixtures_present():
    assert {os.path.basename(p)[:-4] for p in GOLDEN} == set(GOLDEN_CASES)


@pytest.mark.parametrize("path", GOLDEN, ids=lambda p: os.path.basename(p)[:-4])
def test_fixture_inputs_reproducible(path):
    """The committed inputs are what tests/cases.py generates from the seed."""
    i, _, nv_out = _load(path)
    kind, C, r, K, cout, seed = GOLDEN_CASES[os.path.basename(path)[:-4]]
    d = conv_inputs(kind, C, r, K, cout, seed)
    assert d["nv_out"] == nv_out
    for k, v in i.items():
        assert torch.equal(v, d[k]), k


@pytest.mark.parametrize("impl", ["torch", "c"])
@pytest.mark.parametrize("path", GOLDEN, ids=lambda p: os.path.basename(p)[:-4])
def test_oracle_matches_reference_outputs(path, impl):
    i, ref, nv_out = _load(path)
    if impl == "torch":
        f = dict(count=lambda: mo.count_vertex_adjface(i["face"], i["vt_map"], nv_out),
                 v2f=lambda: mo.vertex2facet_forward(i["x_v"], i["filt_v2f"], i["face"]),
                 v2f_b=lambda: mo.vertex2facet_backward(i["g_v2f"], i["x_v"], i["filt_v2f"], i["face"]),
                 f2v=lambda n: mo.facet2vertex_forward(i["x_f"], i["filt_f2v"], i["coeff"], i["face"], n, i["vt_map"]),
                 f2v_b=lambda n: mo.facet2vertex_backward(i["g_f2v"], i["x_f"], i["filt_f2v"], i["coeff"], i["face"], n,
                                                          i["vt_map"]),
                 f2f=lambda: mo.facet2facet_forward(i["tex"], i["filt_f2f"], i["bary"], i["cum"]),
                 f2f_b=lambda: mo.facet2facet_backward(i["g_f2f"], i["tex"], i["filt_f2f"], i["bary"], i["cum"]))
    else:
        n_ = {k: v.numpy() for k, v in i.items()}
        f = dict(count=lambda: co.count_vertex_adjface(n_["face"], n_["vt_map"], nv_out),
                 v2f=lambda: co.v2f_forward(n_["x_v"], n_["filt_v2f"], n_["face"]),
                 v2f_b=lambda: co.v2f_backward(n_["g_v2f"], n_["x_v"], n_["filt_v2f"], n_["face"]),
                 f2v=lambda n: co.f2v_forward(n_["x_f"], n_["filt_f2v"], n_["coeff"], n_["face"], np.asarray(n),
                                              n_["vt_map"]),
                 f2v_b=lambda n: co.f2v_backward(n_["g_f2v"], n_["x_f"], n_["filt_f2v"], n_["coeff"], n_["face"],
                                                 np.asarray(n), n_["vt_map"]),
                 f2f=lambda: co.f2f_forward(n_["tex"], n_["filt_f2f"], n_["bary"], n_["cum"]),
                 f2f_b=lambda: co.f2f_backward(n_["g_f2f"], n_["tex"], n_["filt_f2f"], n_["bary"], n_["cum"]))
    nfc = torch.as_tensor(f["count"]())
    assert torch.equal(nfc.to(torch.int32), ref["nf_count"])            # index output: bit-exact
    assert rel_err(f["v2f"](), ref["v2f_out"]) <= TOL
    for got, key in zip(f["v2f_b"](), ("v2f_gin", "v2f_gf")):
        assert rel_err(got, ref[key]) <= TOL, key
    assert rel_err(f["f2v"](nfc), ref["f2v_out"]) <= TOL
    for got, key in zip(f["f2v_b"](nfc), ("f2v_gin", "f2v_gf")):
        assert rel_err(got, ref[key]) <= TOL, key
    assert rel_err(f["f2f"](), ref["f2f_out"]) <= TOL
    for got, key in zip(f["f2f_b"](), ("f2f_gin", "f2f_gf")):
        assert rel_err(got, ref[key]) <= TOL, key


@pytest.mark.parametrize("kind,C,r,K,cout", [("ico1x2+drop", 6, 3, 4, 3), ("grid9x1", 4, 1, 25, 5),
                                              ("tet+iso", 3, 2, 1, 2), ("tri", 2, 1, 4, 2)])
def test_torch_and_c_oracles_agree(kind, C, r, K, cout):
    d = conv_inputs(kind, C, r, K, cout, seed=31)
    n = {k: (v.numpy() if isinstance(v, torch.Tensor) else v) for k, v in d.items()}
    nfc = mo.count_vertex_adjface(d["face"], d["vt_map"], d["nv_out"])
    assert np.array_equal(nfc.numpy(), co.count_vertex_adjface(n["face"], n["vt_map"], d["nv_out"]))
    for acc64 in (False, True):
        cast = (lambda t: t.double()) if acc64 else (lambda t: t)
        tol = 1e-6 if acc64 else 2e-6
        assert rel_err(co.v2f_forward(n["x_v"], n["filt_v2f"], n["face"], acc64),
                       mo.vertex2facet_forward(cast(d["x_v"]), cast(d["filt_v2f"]), d["face"])) <= tol
        a = co.v2f_backward(n["g_v2f"], n["x_v"], n["filt_v2f"], n["face"], acc64)
        b = mo.vertex2facet_backward(cast(d["g_v2f"]), cast(d["x_v"]), cast(d["filt_v2f"]), d["face"])
        assert rel_err(a[0], b[0]) <= tol and rel_err(a[1], b[1]) <= 5 * tol
        assert rel_err(co.f2v_forward(n["x_f"], n["filt_f2v"], n["coeff"], n["face"], nfc.numpy(), n["vt_map"], acc64),
                       mo.facet2vertex_forward(cast(d["x_f"]), cast(d["filt_f2v"]), cast(d["coeff"]), d["face"], nfc,
                                               d["vt_map"])) <= tol
        a = co.f2v_backward(n["g_f2v"], n["x_f"], n["filt_f2v"], n["coeff"], n["face"], nfc.numpy(), n["vt_map"], acc64)
        b = mo.facet2vertex_backward(cast(d["g_f2v"]), cast(d["x_f"]), cast(d["filt_f2v"]), cast(d["coeff"]),
                                     d["face"], nfc, d["vt_map"])
        assert rel_err(a[0], b[0]) <= tol and rel_err(a[1], b[1]) <= 5 * tol
        assert rel_err(co.f2f_forward(n["tex"], n["filt_f2f"], n["bary"], n["cum"], acc64),
                       mo.facet2facet_forward(cast(d["tex"]), cast(d["filt_f2f"]), cast(d["bary"]), d["cum"])) <= tol
        a = co.f2f_backward(n["g_f2f"], n["tex"], n["filt_f2f"], n["bary"], n["cum"], acc64)
        b = mo.facet2facet_backward(cast(d["g_f2f"]), cast(d["tex"]), cast(d["filt_f2f"]), cast(d["bary"]), d["cum"])
        assert rel_err(a[0], b[0]) <= tol and rel_err(a[1], b[1]) <= 5 * tol


def test_backward_formulas_gradcheck_fp64():
    d = conv_inputs("ico1x2+drop", 3, 2, 4, 3, seed=5)
    dd = lambda t: t.double()
    x = dd(d["x_v"]).requires_grad_()
    fl = dd(d["filt_v2f"]).requires_grad_()
    assert torch.autograd.gradcheck(lambda a, b: mo.vertex2facet(a, b, d["face"]), (x, fl))
    nfc = mo.count_vertex_adjface(d["face"], d["vt_map"], d["nv_out"])
    xf = dd(d["x_f"]).requires_grad_()
    ff = dd(d["filt_f2v"]).requires_grad_()
    assert torch.autograd.gradcheck(lambda a, b: mo.facet2vertex(a, b, dd(d["coeff"]), d["face"], nfc, d["vt_map"]),
                                    (xf, ff))
    tex = dd(d["tex"]).requires_grad_()
    W = dd(d["filt_f2f"]).requires_grad_()
    assert torch.autograd.gradcheck(lambda a, b: mo.facet2facet(a, b, dd(d["bary"]), d["cum"]), (tex, W))


def test_known_answers():
    # one triangle, one-hot filter / coefficient: outputs are single input values
    face = torch.tensor([[0, 1, 2]], dtype=torch.int32)
    x = torch.tensor([[1.0, 10.0], [2.0, 20.0], [3.0, 30.0]])
    filt = torch.zeros(3, 2, 1)
    filt[1] = 1.0
    assert torch.equal(mo.vertex2facet_forward(x, filt, face), torch.tensor([[2.0, 20.0]]))
    # closed mesh, constant features, filter == 1/K, coeff == 1: F2V returns the constant
    d = conv_inputs("ico1x2", 4, 1, 16, 4, seed=1)
    nfc = mo.count_vertex_adjface(d["face"], d["vt_map"], d["nv_out"])
    nf = d["face"].shape[0]
    out = mo.facet2vertex_forward(torch.full((nf, 4), 3.0), torch.full((16, 4, 1), 1 / 16), torch.ones(nf, 16),
                                  d["face"], nfc, d["vt_map"])
    assert torch.allclose(out, torch.full_like(out, 3.0), atol=1e-6)
    assert int(nfc.sum()) == 3 * nf and set(nfc.tolist()) <= {5, 6}      # icosphere valences
    # F2F with one sample per face and a filter that picks basis 0, channel 0
    cum = torch.arange(1, 6, dtype=torch.int32)
    tex = torch.arange(5, dtype=torch.float32).reshape(5, 1)
    W = torch.zeros(2, 1, 3)
    W[1, 0, 0] = 2.0
    bary = torch.tensor([[1.0, 0, 0]]).repeat(5, 1)
    assert torch.equal(mo.facet2facet_forward(tex, W, bary, cum), torch.stack([torch.zeros(5), 2 * tex[:, 0]], 1))


def test_sph_harm_known_values():
    # Y_0 = 1/2 sqrt(1/pi); degree-1 values on the axes; both restatements agree
    axes = torch.eye(3)
    sh = mo.sph_harm_coeff(1, axes)
    y0 = 0.5 * math.sqrt(1 / math.pi)
    assert torch.allclose(sh[:, 0], torch.full((3,), y0), atol=1e-7)
    c1 = 0.5 * math.sqrt(3 / (2 * math.pi))
    c2 = 0.5 * math.sqrt(3 / math.pi)
    want = torch.tensor([[c1, 0, 0], [0, 0, c1], [0, c2, 0]])
    assert torch.allclose(sh[:, 1:], want, atol=1e-6)
    g = torch.Generator().manual_seed(0)
    xyz = torch.randn(257, 3, generator=g)
    xyz[0] = 0
    for L in range(6):
        a = mo.sph_harm_coeff(L, xyz)
        assert a.shape == (257, (L + 1) ** 2)
        assert max_abs(a, co.sph_harm_coeff(L, xyz.numpy(), mo.sph_constants_f32())) <= 2e-6
        assert max_abs(a, mo.sph_harm_coeff(L, xyz.double())) <= 5e-6
    with pytest.raises(NotImplementedError):
        mo.sph_harm_coeff(6, xyz)
    # orthonormality of the real basis implied by the reference's normalisation:
    # sum over the sphere of Y_0^2 * 4pi == 1
    assert abs(y0 * y0 * 4 * math.pi - 1.0) < 1e-12


def test_triangle_geometry():
    d = conv_inputs("grid9x1", 4, 1, 4, 2, seed=1)
    geo = mo.triangle_geometry(d["vertex"], d["face"])
    assert max_abs(geo, co.triangle_geometry(d["vertex"].numpy(), d["face"].numpy())) <= 1e-6
    assert torch.allclose(geo[:, :3].norm(dim=1), torch.ones(geo.shape[0]), atol=1e-5)


def test_repeated_face_rows_fold_into_mean_weights():
    """The identity behind block.conv_block: facet2facet over rows repeated once per sample equals facet2facet over
    one row per face with the per-face mean of the sample weights and one sample per face -- output, filter gradient,
    and the input gradient summed over each face's samples (the backward of the repetition).  fp64, the oracle's own
    restatement of mesh_conv3d_gpu.cu:6-135; faces without samples included."""
    import numpy as np
    from oracle import mesh_oracle as mo
    rng = np.random.default_rng(3)
    nf, cin, cout, F = 57, 5, 4, 9
    counts = torch.from_numpy(rng.integers(0, 5, size=nf).astype(np.int64))
    cum = torch.cumsum(counts, 0).to(torch.int32)
    nik = int(counts.sum())
    y = torch.from_numpy(rng.standard_normal((nf, cin)))
    bary = torch.from_numpy(rng.standard_normal((nik, F)))
    w = torch.from_numpy(rng.standard_normal((cout, cin, F)))
    g = torch.from_numpy(rng.standard_normal((nf, cout)))
    seg = torch.repeat_interleave(torch.arange(nf), counts)
    tex = y[seg]
    out = mo.facet2facet_forward(tex, w, bary, cum)
    gin, gf = mo.facet2facet_backward(g, tex, w, bary, cum)
    gy = torch.zeros_like(y).index_add_(0, seg, gin)
    mean = torch.zeros(nf, F, dtype=torch.float64).index_add_(0, seg, bary) / counts.clamp(min=1)[:, None]
    one_each = torch.arange(1, nf + 1, dtype=torch.int32)
    out1 = mo.facet2facet_forward(y, w, mean, one_each)
    gy1, gf1 = mo.facet2facet_backward(g, y, w, mean, one_each)
    for a, b in ((out1, out), (gy1, gy), (gf1, gf)):
        assert float((a - b).abs().max()) <= 1e-12 * max(1.0, float(b.abs().max()))
    assert torch.all(out[counts == 0] == 0) and torch.all(out1[counts == 0] == 0)
