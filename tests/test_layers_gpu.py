"""The layer modules (same names / parameters as the reference's picasso/mesh/layers.py)
against a CPU composition of the oracle operators with the same parameters: operator ->
pointwise matmul -> + bias -> ReLU -> BatchNorm1d(eps=1e-3)  (batch norm after ReLU)."""
import pytest
import torch
import torch.nn as nn

from conftest import rel_err
from cases import conv_inputs

pytestmark = pytest.mark.gpu
TOL = 1e-4


def _tail(x, mod):
    x = x + mod.biases.detach().cpu().double()
    x = torch.relu(x)
    bn = mod.BatchNorm
    mean, var = x.mean(0), x.var(0, unbiased=False)
    return (x - mean) / torch.sqrt(var + bn.eps) * bn.weight.detach().cpu().double() + bn.bias.detach().cpu().double()


def test_v2v_and_f2f_modules_match_oracle_composition():
    from picassoplus_b200.mesh.layers import V2VConv3d, F2FConv3d, SphHarmCoeff
    from picassoplus_b200.mesh import utils as mesh_utils
    from oracle import mesh_oracle as mo
    torch.manual_seed(0)
    L, cin, mid, cout = 3, 16, 32, 24
    d = conv_inputs("ico2x3", cin, 1, (L + 1) ** 2, 8, seed=61)
    dev = torch.device("cuda")
    vertex, face, vt = d["vertex"].to(dev), d["face"].to(dev), d["vt_map"].to(dev)
    nfc = mesh_utils.count_vertex_adjface(face, vt, vertex)
    geo = mesh_utils.compute_triangle_geometry(vertex, face)
    coeff = SphHarmCoeff(L)(geo[:, :3].contiguous())

    conv = V2VConv3d(cin, [mid, cout], L, [1, 1]).to(dev).train()
    x = d["x_v"].to(dev).requires_grad_()
    out = conv(x, face, nfc, vt, coeff)
    G = torch.randn_like(out)
    (out * G).sum().backward()

    # the same computation with the oracle operators on the CPU, fp64
    v2f, f2v = conv.V2F_conv3d, conv.F2V_conv3d
    P = lambda t: t.detach().cpu().double()
    xo = P(d["x_v"]).requires_grad_()
    sw = P(v2f.spatial_weights).requires_grad_()
    sh_eye = mo.sph_harm_coeff(L, torch.eye(3)).double()
    y = mo.vertex2facet(xo, (sh_eye @ sw).reshape(3, cin, 1), d["face"])
    y = _tail(y @ P(v2f.depth_weights), v2f)
    geo_o = mo.triangle_geometry(d["vertex"], d["face"])
    coeff_o = mo.sph_harm_coeff(L, geo_o[:, :3]).double()
    nfc_o = mo.count_vertex_adjface(d["face"], d["vt_map"], d["nv_out"])
    fw = P(f2v.spatial_weights).requires_grad_()
    z = mo.facet2vertex(y, fw, coeff_o, d["face"], nfc_o, d["vt_map"])
    z = _tail(z @ P(f2v.depth_weights), f2v)
    (z * P(G)).sum().backward()

    assert rel_err(out, z) <= 2e-4
    assert rel_err(x.grad, xo.grad) <= 5e-4
    assert rel_err(v2f.spatial_weights.grad, sw.grad) <= 5e-4
    assert rel_err(f2v.spatial_weights.grad, fw.grad) <= 5e-4

    # F2FConv3d: takes per-face sample COUNTS (the module forms the running count itself)
    f2f = F2FConv3d(cin, cout, L).to(dev).train()
    bary_sh = SphHarmCoeff(L)(d["bary_xyz"].to(dev))
    tex = d["tex"].to(dev).requires_grad_()
    o2 = f2f(tex, bary_sh, d["counts"].to(dev))
    G2 = torch.randn_like(o2)
    (o2 * G2).sum().backward()
    texo = P(d["tex"]).requires_grad_()
    Wo = P(f2f.weights).requires_grad_()
    ref = mo.facet2facet(texo, Wo, mo.sph_harm_coeff(L, d["bary_xyz"]).double(), d["cum"])
    ref = _tail(ref, f2f)
    (ref * P(G2)).sum().backward()
    assert rel_err(o2, ref) <= 2e-4
    assert rel_err(tex.grad, texo.grad) <= 5e-4
    assert rel_err(f2f.weights.grad, Wo.grad) <= 5e-4


def test_state_dict_names_match_reference_layout():
    """Parameter names and shapes a reference checkpoint would carry."""
    from picassoplus_b200.mesh.layers import V2VConv3d, F2FConv3d
    m = V2VConv3d(8, [16, 12], 3, [1, 2])
    sd = {k: tuple(v.shape) for k, v in m.state_dict().items()}
    assert sd["V2F_conv3d.spatial_weights"] == (16, 8)
    assert sd["V2F_conv3d.depth_weights"] == (8, 16)
    assert sd["V2F_conv3d.biases"] == (1, 16)
    assert sd["F2V_conv3d.spatial_weights"] == (16, 16, 2)
    assert sd["F2V_conv3d.depth_weights"] == (32, 12)
    assert "V2F_conv3d.BatchNorm.running_mean" in sd and "F2V_conv3d.BatchNorm.weight" in sd
    f = F2FConv3d(3, 32, 3)
    assert tuple(f.weights.shape) == (32, 3, 16) and tuple(f.biases.shape) == (1, 32)
