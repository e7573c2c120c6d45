"""The CUDA path against outputs of the reference's own Python (fixture made by
tests/golden/make_golden_modules.py from picasso/math_utils.py, picasso/mesh/layers.py and
picasso/mesh/pi_modules/decimate.py, run unmodified): pb200_sph_harm_coeff,
pb200_triangle_geometry, and the V2VConv3d / F2FConv3d modules of this package loaded with
the reference module's state_dict (strict)."""
import pytest
import torch

from conftest import max_abs, rel_err
from module_oracle import group, load_fixture

pytestmark = pytest.mark.gpu
FX = load_fixture()


def test_sph_harm_kernel_matches_reference_python():
    from picassoplus_b200.math_utils import sph_harm_coeff
    xyz = torch.from_numpy(FX["sh_xyz"]).cuda()
    for L in range(6):
        got = sph_harm_coeff(L, xyz)
        assert max_abs(got, FX[f"sh_L{L}"]) <= 2e-6, L


def test_triangle_geometry_kernel_matches_reference_python():
    from picassoplus_b200.mesh.pi_modules import decimate
    geo = decimate.compute_triangle_geometry_(torch.from_numpy(FX["geo_vertex"]).cuda(),
                                              torch.from_numpy(FX["geo_face"]).cuda())
    assert max_abs(geo, FX["geo_out"]) <= 1e-6


def _load(module, prefix):
    sd = group(FX, prefix + "_param")
    sd.update(group(FX, prefix + "_buffer"))
    # the recorded buffers are the running statistics AFTER the reference's step: start from fresh ones
    for k in list(sd):
        if k.endswith("running_mean"):
            sd[k] = torch.zeros_like(sd[k])
        elif k.endswith("running_var"):
            sd[k] = torch.ones_like(sd[k])
        elif k.endswith("num_batches_tracked"):
            sd[k] = torch.zeros_like(sd[k])
    module.load_state_dict(sd, strict=True)            # same names and shapes as the reference module


def test_v2v_module_matches_reference_python():
    from picassoplus_b200.mesh.layers import V2VConv3d
    cin, mid, cout, L, m1, m2 = [int(v) for v in FX["v2v_cfg"]]
    mod = V2VConv3d(cin, [mid, cout], L, [m1, m2])
    _load(mod, "v2v")
    mod = mod.cuda().train()
    x = torch.from_numpy(FX["v2v_x"]).cuda().requires_grad_()
    out = mod(x, torch.from_numpy(FX["v2v_face"]).cuda(), torch.from_numpy(FX["v2v_nf_count"]).cuda(),
              torch.from_numpy(FX["v2v_vt_map"]).cuda(), torch.from_numpy(FX["v2v_coeff"]).cuda())
    (out * torch.from_numpy(FX["v2v_G"]).cuda()).sum().backward()
    assert rel_err(out, FX["v2v_out"]) <= 1e-4
    assert rel_err(x.grad, FX["v2v_grad_x"]) <= 1e-4
    params = dict(mod.named_parameters())
    for name, g in group(FX, "v2v_grad").items():
        assert rel_err(params[name].grad, g) <= 1e-4, name
    bufs = dict(mod.named_buffers())
    for name, b in group(FX, "v2v_buffer").items():    # running statistics after one training step
        if b.dtype.is_floating_point:
            assert rel_err(bufs[name], b) <= 1e-4, name


def test_f2f_module_matches_reference_python():
    from picassoplus_b200.mesh.layers import F2FConv3d, SphHarmCoeff
    cin, cout, L = [int(v) for v in FX["f2f_cfg"]]
    mod = F2FConv3d(cin, cout, L)
    _load(mod, "f2f")
    mod = mod.cuda().train()
    bary = SphHarmCoeff(L)(torch.from_numpy(FX["f2f_bary_xyz"]).cuda())
    assert max_abs(bary, FX["f2f_bary"]) <= 2e-6
    tex = torch.from_numpy(FX["f2f_tex"]).cuda().requires_grad_()
    out = mod(tex, bary, torch.from_numpy(FX["f2f_counts"]).cuda())
    (out * torch.from_numpy(FX["f2f_G"]).cuda()).sum().backward()
    assert rel_err(out, FX["f2f_out"]) <= 1e-4
    assert rel_err(tex.grad, FX["f2f_grad_tex"]) <= 1e-4
    params = dict(mod.named_parameters())
    for name, g in group(FX, "f2f_grad").items():
        assert rel_err(params[name].grad, g) <= 1e-4, name


def test_level_prepare_orientation_matches_reference_python():
    from picassoplus_b200 import topology
    vertex, face = torch.from_numpy(FX["orient_vertex"]).cuda(), torch.from_numpy(FX["orient_face"]).cuda()
    vt = torch.arange(vertex.shape[0], dtype=torch.int32, device="cuda")
    got = topology.prepare_level(vertex, face, vt, vertex.shape[0], 3, orient=True, want_normals=True)
    assert max_abs(got["geometry"], FX["orient_geometry"]) <= 1e-6
    assert max_abs(got["normals"], FX["orient_normals"]) <= 1e-6
    flipped_ref = FX["orient_normals"] != FX["orient_geometry"][:, :3]
    flipped = (got["normals"] != got["geometry"][:, :3]).cpu().numpy()
    assert (flipped == flipped_ref).all()                               # the same faces are re-oriented


def test_pcloud_module_matches_reference_python():
    from cases import pcloud_inputs
    from picassoplus_b200.point.layers import PCloudConv3d
    Np, Mp, knn, F, C, r, T, seed = [int(v) for v in FX["pc_args"]]
    d = pcloud_inputs(Np, Mp, knn, F, C, r, T, seed)
    mod = PCloudConv3d(C, FX["pc_out"].shape[1], F, depth_multiplier=r)
    _load(mod, "pc")
    mod = mod.cuda().train()
    x = d["x"].cuda().requires_grad_()
    out = mod(x, d["nn_count"].cuda(), d["nn_index"].cuda(), d["bin_index"].cuda(), d["bin_coeff"].cuda())
    (out * torch.from_numpy(FX["pc_G"]).cuda()).sum().backward()
    assert rel_err(out, FX["pc_out"]) <= 1e-4 and rel_err(x.grad, FX["pc_grad_x"]) <= 1e-4
    params = dict(mod.named_parameters())
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
    mod = mod.to("cuda").train()
    x = torch.from_numpy(LX[tag + "_x"]).to("cuda").requires_grad_()
    out = mod(x)
    (out * torch.from_numpy(LX[tag + "_G"]).to("cuda")).sum().backward()
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
    out = mod.to("cuda")(torch.from_numpy(LX["f2vc_normals"]).to("cuda"))
    assert max_abs(out, LX["f2vc_out"]) <= 1e-6


def test_global_pool_against_plain_loops():
    from picassoplus_b200.mesh.layers import GlobalPool3d
    g = torch.Generator().manual_seed(3)
    x = torch.randn(37, 5, generator=g).to("cuda")
    nv = torch.tensor([10, 1, 26], dtype=torch.int32, device="cuda")
    avg = GlobalPool3d("avg")(x, nv)
    val, pos = GlobalPool3d("max")(x, nv)
    start = 0
    for s, n in enumerate([10, 1, 26]):
        seg = x[start:start + n]
        assert max_abs(avg[s], seg.mean(0)) <= 1e-6
        assert torch.equal(val[s], seg.max(0).values) and torch.equal(pos[s].cpu(), seg.argmax(0).cpu() + start)
        start += n
