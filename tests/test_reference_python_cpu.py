"""The oracle against outputs of the reference's own Python (picasso/math_utils.py,
picasso/mesh/layers.py, picasso/mesh/pi_modules/decimate.py run unmodified by
tests/golden/make_golden_modules.py): spherical-harmonic basis, triangle geometry, and the
V2VConv3d / F2FConv3d modules forward + backward."""
import pytest
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


LX = load_fixture("layers_ref_python.npz")


def _load_layer(module, prefix):
    sd = group(LX, prefix + "_param")
    sd.update(group(LX, prefix + "_buffer"))
    for k in list(sd):                                  # recorded after the reference's step: start from fresh ones
        if k.endswith("running_mean"):
            sd[k] = torch.zeros_like(sd[k])
        elif k.endswith("running_var"):
            sd[k] = torch.ones_like(sd[k])
        elif k.endswith("num_batches_tracked"):
            sd[k] = torch.zeros_like(sd[k])
    module.load_state_dict(sd, strict=True)


@pytest.mark.parametrize("tag,kw", [("pic_bn", {}), ("pic_plain", dict(with_bn=False, activation_fn=None))])
def test_per_item_conv_matches_reference_python(tag, kw):
    from picassoplus_b200.mesh.layers import PerItemConv3d
    cin, cout = [int(v) for v in LX[tag + "_cfg"]]
    mod = PerItemConv3d(cin, cout, **kw)
    _load_layer(mod, tag)
    mod = mod.to("cpu").train()
    x = torch.from_numpy(LX[tag + "_x"]).to("cpu").requires_grad_()
    out = mod(x)
    (out * torch.from_numpy(LX[tag + "_G"]).to("cpu")).sum().backward()
    assert rel_err(out, LX[tag + "_out"]) <= 1e-4
    assert rel_err(x.grad, LX[tag + "_grad_x"]) <= 1e-4
    params = dict(mod.named_parameters())
    for name, g in group(LX, tag + "_grad").items():
        assert rel_err(params[name].grad, g) <= 1e-4, name
    bufs = dict(mod.named_buffers())
    for name, b in group(LX, tag + "_buffer").items():
        if b.dtype.is_floating_point:
            assert rel_err(bufs[name], b) <= 1e-4, name


def test_build_f2v_coeff_matches_reference_python():
    from picassoplus_b200.mesh.layers import BuildF2VCoeff
    mod = BuildF2VCoeff(int(LX["f2vc_cfg"][0]), tau=float(LX["f2vc_cfg"][1]))
    mod.load_state_dict({"centers": torch.from_numpy(LX["f2vc_centers"])}, strict=True)
    out = mod.to("cpu")(torch.from_numpy(LX["f2vc_normals"]).to("cpu"))
    assert max_abs(out, LX["f2vc_out"]) <= 1e-6


def test_global_pool_against_plain_loops():
    from picassoplus_b200.mesh.layers import GlobalPool3d
    g = torch.Generator().manual_seed(3)
    x = torch.randn(37, 5, generator=g).to("cpu")
    nv = torch.tensor([10, 1, 26], dtype=torch.int32, device="cpu")
    avg = GlobalPool3d("avg")(x, nv)
    val, pos = GlobalPool3d("max")(x, nv)
    start = 0
    for s, n in enumerate([10, 1, 26]):
        seg = x[start:start + n]
        assert max_abs(avg[s], seg.mean(0)) <= 1e-6
        assert torch.equal(val[s], seg.max(0).values) and torch.equal(pos[s].cpu(), seg.argmax(0).cpu() + start)
        start += n
