"""The oracle against outputs of the reference's own Python (picasso/math_utils.py,
picasso/mesh/layers.py, picasso/mesh/pi_modules/decimate.py run unmodified by
tests/golden/make_golden_modules.py): spherical-harmonic basis, triangle geometry, and the
V2VConv3d / F2FConv3d modules forward + backward."""
import torch

from conftest import max_abs, rel_err
from module_oracle import f2f_forward, group, load_fixture, v2v_forward
from oracle import c_oracle as co
from oracle import mesh_oracle as mo

FX = load_fixture()


def test_sph_harm_matches_reference_python():
    xyz = torch.from_numpy(FX["sh_xyz"])
    for L in range(6):
        want = torch.from_numpy(FX[f"sh_L{L}"])
        assert want.shape == (xyz.shape[0], (L + 1) ** 2)
        assert max_abs(mo.sph_harm_coeff(L, xyz), want) <= 2e-6                     # torch restatement, fp32
        assert max_abs(co.sph_harm_coeff(L, xyz.numpy(), mo.sph_constants_f32()), want) <= 2e-6   # C restatement
        assert max_abs(mo.sph_harm_coeff(L, xyz.double()), want) <= 5e-6            # fp64 evaluation


def test_triangle_geometry_matches_reference_python():
    vertex, face = torch.from_numpy(FX["geo_vertex"]), torch.from_numpy(FX["geo_face"])
    want = torch.from_numpy(FX["geo_out"])
    assert max_abs(mo.triangle_geometry(vertex, face), want) <= 1e-6
    assert max_abs(co.triangle_geometry(vertex.numpy(), face.numpy()), want) <= 1e-6


def test_v2v_module_matches_reference_python():
    cfg = [int(v) for v in FX["v2v_cfg"]]
    params = {k: v.double().requires_grad_() for k, v in group(FX, "v2v_param").items()}
    x = torch.from_numpy(FX["v2v_x"]).double().requires_grad_()
    out = v2v_forward(x, params, torch.from_numpy(FX["v2v_face"]), torch.from_numpy(FX["v2v_nf_count"]),
                      torch.from_numpy(FX["v2v_vt_map"]), torch.from_numpy(FX["v2v_coeff"]).double(), cfg)
    (out * torch.from_numpy(FX["v2v_G"]).double()).sum().backward()
    assert rel_err(out, FX["v2v_out"]) <= 1e-4
    assert rel_err(x.grad, FX["v2v_grad_x"]) <= 1e-4
    grads = group(FX, "v2v_grad")
    assert set(grads) == set(params)
    for name, g in grads.items():
        assert rel_err(params[name].grad, g) <= 1e-4, name


def test_f2f_module_matches_reference_python():
    params = {k: v.double().requires_grad_() for k, v in group(FX, "f2f_param").items()}
    tex = torch.from_numpy(FX["f2f_tex"]).double().requires_grad_()
    L = int(FX["f2f_cfg"][2])
    # the basis of the barycentric samples first: restated SH against the recorded one
    assert max_abs(mo.sph_harm_coeff(L, torch.from_numpy(FX["f2f_bary_xyz"])), FX["f2f_bary"]) <= 2e-6
    out = f2f_forward(tex, params, torch.from_numpy(FX["f2f_bary"]).double(), torch.from_numpy(FX["f2f_counts"]))
    (out * torch.from_numpy(FX["f2f_G"]).double()).sum().backward()
    assert rel_err(out, FX["f2f_out"]) <= 1e-4
    assert rel_err(tex.grad, FX["f2f_grad_tex"]) <= 1e-4
    for name, g in group(FX, "f2f_grad").items():
        assert rel_err(params[name].grad, g) <= 1e-4, name


def test_oriented_normals_match_reference_python():
    geo, vertex = torch.from_numpy(FX["orient_geometry"]), torch.from_numpy(FX["orient_vertex"])
    face, want = torch.from_numpy(FX["orient_face"]), torch.from_numpy(FX["orient_normals"])
    assert max_abs(mo.triangle_geometry(vertex, face), geo) <= 1e-6
    got = mo.oriented_normals(geo, vertex, face)
    assert torch.equal(got, want)
    assert (want != geo[:, :3]).any() and (want == geo[:, :3]).any()       # both orientations occur


def test_pcloud_module_matches_reference_python():
    from cases import pcloud_inputs
    d = pcloud_inputs(*[int(v) for v in FX["pc_args"]])
    params = {k: v.double().requires_grad_() for k, v in group(FX, "pc_param").items()}
    x = d["x"].double().requires_grad_()
    from module_oracle import tail
    f = mo.pcloud_conv3d_forward(x, params["spatial_weights"], d["nn_count"], d["nn_index"], d["bin_index"],
                                 d["bin_coeff"].double())
    out = tail(f @ params["depth_weights"], params["biases"], params["BatchNorm.weight"], params["BatchNorm.bias"])
    (out * torch.from_numpy(FX["pc_G"]).double()).sum().backward()
    assert rel_err(out, FX["pc_out"]) <= 1e-4 and rel_err(x.grad, FX["pc_grad_x"]) <= 1e-4
    for name, g in group(FX, "pc_grad").items():
        assert rel_err(params[name].grad, g) <= 1e-4, name
