"""Makes tests/golden/modules_ref_python.npz by running the reference's own, UNMODIFIED
Python for the parts of the path that are plain torch code:

  * SphHarmCoeff(L)(xyz), L = 0..5   (picasso/mesh/layers.py:331-356 over
                                      picasso/math_utils.py:10-62)
  * compute_triangle_geometry_       (picasso/mesh/pi_modules/decimate.py:70-85)
  * V2VConv3d and F2FConv3d, forward and backward with a seeded state_dict
  * PerItemConv3d (forward and backward) and BuildF2VCoeff, in layers_ref_python.npz
                                     (picasso/mesh/layers.py:18-195)
  * get_oriented_normals             (picasso/networks/scene_seg.py:117-124)
  * PCloudConv3d with fuzzy bins, forward and backward (picasso/point/layers.py:19-75)

    REF_ROOT=<reference checkout> python tests/golden/make_golden_modules.py [output_dir]

The reference tree is imported from where it lies (REF_ROOT); nothing of it is copied.  It
cannot be imported as it is on a machine without its compiled extensions, so this script
(and only this script) puts stand-ins into sys.modules for what the import needs but the
recorded functions never call: `torch_scatter` (used by GlobalPool3d only),
`scipy.special.sph_harm` (imported by math_utils, never called by torch_sph_harm_reorder),
`mesh_decimation`, `mesh_pool3d`, `mesh_unpool3d`, `open3d` and the point-cloud extensions other than
`point_conv3d` (imported by pi_modules / utils, not called here).
The extensions the modules do call, `mesh_conv3d` and `point_conv3d`, are bound to the reference's own CUDA
kernels (oracle/_ref, compiled from the reference sources) when a CUDA device is present,
else to the plain-C restatement in oracle/mesh_oracle.c, which is itself pinned against
those kernels by tests/golden/*.npz; the fixture records which one ran (`conv_backend`).
On a machine without CUDA the reference's `.to(x.get_device())` idiom (device index -1)
fails, so `Tensor.get_device` is wrapped to answer "cpu" for CPU tensors while the
reference code runs.
"""
from __future__ import annotations

import os
import sys
import types

import numpy as np
import torch

HERE = os.path.dirname(os.path.abspath(__file__))
ROOT = os.path.dirname(os.path.dirname(HERE))
sys.path.insert(0, ROOT)
sys.path.insert(0, os.path.join(ROOT, "tests"))

from cases import conv_inputs, pcloud_inputs  # noqa: E402


def _install_stand_ins(use_cuda: bool) -> str:
    ts = types.ModuleType("torch_scatter")
    ts.scatter_mean = ts.scatter_max = lambda *a, **k: (_ for _ in ()).throw(RuntimeError("stand-in"))
    sys.modules["torch_scatter"] = ts
    import scipy.special
    if not hasattr(scipy.special, "sph_harm"):
        scipy.special.sph_harm = lambda *a, **k: (_ for _ in ()).throw(RuntimeError("stand-in"))
    for name in ("mesh_decimation", "mesh_pool3d", "mesh_unpool3d", "open3d", "point_buildkernel", "point_nnquery",
                 "point_pool3d", "point_sample", "point_unpool3d"):
        sys.modules[name] = types.ModuleType(name)
    pconv = types.ModuleType("point_conv3d")

    conv = types.ModuleType("mesh_conv3d")
    if use_cuda:
        from oracle import ref_cuda as rc
        conv.facet2facet_forward = rc.f2f_forward
        conv.facet2facet_backward = lambda g, x, w, b, n: list(rc.f2f_backward(g, x, w, b, n))
        conv.vertex2facet_forward = rc.v2f_forward
        conv.vertex2facet_backward = lambda g, x, w, f: list(rc.v2f_backward(g, x, w, f))
        conv.facet2vertex_forward = rc.f2v_forward
        conv.facet2vertex_backward = lambda g, x, w, c, f, n, m: list(rc.f2v_backward(g, x, w, c, f, n, m))
        pconv.SPH3D_forward = lambda x, w, c, i, b: rc.pcloud_forward(x, w, c, i, b)
        pconv.SPH3D_backward = lambda g, x, w, c, i, b: list(rc.pcloud_backward(g, x, w, c, i, b))
        pconv.fuzzySPH3D_forward = lambda x, w, c, i, b, k: rc.pcloud_forward(x, w, c, i, b, k)
        pconv.fuzzySPH3D_backward = lambda g, x, w, c, i, b, k: list(rc.pcloud_backward(g, x, w, c, i, b, k))
        backend = "reference CUDA kernels (oracle/_ref)"
    else:
        from oracle import c_oracle as co
        t = torch.from_numpy
        n = lambda x: x.detach().cpu().numpy()                                   # noqa: E731
        conv.facet2facet_forward = lambda x, w, b, c: t(co.f2f_forward(n(x), n(w), n(b), n(c)))
        conv.facet2facet_backward = lambda g, x, w, b, c: [t(a) for a in co.f2f_backward(n(g), n(x), n(w), n(b), n(c))]
        conv.vertex2facet_forward = lambda x, w, f: t(co.v2f_forward(n(x), n(w), n(f)))
        conv.vertex2facet_backward = lambda g, x, w, f: [t(a) for a in co.v2f_backward(n(g), n(x), n(w), n(f))]
        conv.facet2vertex_forward = lambda x, w, c, f, nf, m: t(co.f2v_forward(n(x), n(w), n(c), n(f), n(nf), n(m)))
        conv.facet2vertex_backward = lambda g, x, w, c, f, nf, m: [
            t(a) for a in co.f2v_backward(n(g), n(x), n(w), n(c), n(f), n(nf), n(m))]
        pconv.SPH3D_forward = lambda x, w, c, i, b: t(co.pcloud_forward(n(x), n(w), n(c), n(i), n(b)))
        pconv.SPH3D_backward = lambda g, x, w, c, i, b: [t(a) for a in co.pcloud_backward(n(g), n(x), n(w), n(c), n(i), n(b))]
        pconv.fuzzySPH3D_forward = lambda x, w, c, i, b, k: t(co.pcloud_forward(n(x), n(w), n(c), n(i), n(b), n(k)))
        pconv.fuzzySPH3D_backward = lambda g, x, w, c, i, b, k: [
            t(a) for a in co.pcloud_backward(n(g), n(x), n(w), n(c), n(i), n(b), n(k))]
        backend = "plain-C restatement (oracle/mesh_oracle.c), fp32 accumulators"
        orig = torch.Tensor.get_device
        torch.Tensor.get_device = lambda self: orig(self) if self.is_cuda else "cpu"
    sys.modules["mesh_conv3d"] = conv
    sys.modules["point_conv3d"] = pconv
    return backend


def main(out_dir: str) -> None:
    ref_root = os.environ.get("REF_ROOT")
    assert ref_root and os.path.isdir(os.path.join(ref_root, "picasso")), "set REF_ROOT to the reference checkout"
    use_cuda = torch.cuda.is_available() and os.path.exists(os.path.join(ROOT, "oracle", "_ref", "libref_mesh_conv3d.so"))
    backend = _install_stand_ins(use_cuda)
    sys.path.insert(0, ref_root)
    from picasso.mesh import layers as ref_layers                      # the reference, unmodified
    from picasso.mesh.pi_modules import decimate as ref_decimate
    dev = torch.device("cuda:0" if use_cuda else "cpu")
    out = {"conv_backend": np.array(backend)}

    # ---- spherical-harmonic basis: seeded directions, the axes, the zero vector, phi < 0
    g = torch.Generator().manual_seed(2024)
    xyz = torch.randn(96, 3, generator=g)
    xyz[:8] = torch.tensor([[1., 0, 0], [0, 1., 0], [0, 0, 1.], [0, 0, 0], [-1., 0, 0], [0, -1., 0], [0, 0, -1.],
                            [0.3, -0.4, 0.5]])
    xyz[8:16] *= torch.tensor([1e-3, 1e3, 1e-6, 7.0, 1.0, 1.0, 1.0, 1.0]).reshape(-1, 1)    # un-normalised lengths
    out["sh_xyz"] = xyz.numpy()
    for L in range(6):
        out[f"sh_L{L}"] = ref_layers.SphHarmCoeff(L)(xyz.clone().to(dev)).cpu().numpy()

    # ---- triangle geometry on a seeded heightfield with deleted faces (vertex rows carry extra columns)
    d = conv_inputs("grid17x2", 4, 1, 4, 2, seed=71)
    vert6 = torch.cat([d["vertex"], torch.rand(d["vertex"].shape[0], 3, generator=g)], dim=1)
    out["geo_vertex"], out["geo_face"] = vert6.numpy(), d["face"].numpy()
    out["geo_out"] = ref_decimate.compute_triangle_geometry_(vert6.to(dev), d["face"].to(dev)).cpu().numpy()

    # ---- V2VConv3d (V2F then F2V, depth multipliers 2 and 1) and F2FConv3d, training-mode batch norm
    L, cin, mid, cout = 3, 6, 10, 8
    K = (L + 1) ** 2
    d = conv_inputs("ico1x3", cin, 1, K, cout, seed=72)
    face, vt_map = d["face"], d["vt_map"]
    nf_count = torch.bincount(face.reshape(-1).long(), minlength=d["nv_out"]).to(torch.int32)
    geo = ref_decimate.compute_triangle_geometry_(d["vertex"].to(dev), face.to(dev))
    coeff = ref_layers.SphHarmCoeff(L)(geo[:, :3]).detach()
    torch.manual_seed(7)
    v2v = ref_layers.V2VConv3d(cin, [mid, cout], L, [2, 1]).to(dev)
    with torch.no_grad():
        for n_, p_ in v2v.named_parameters():
            if n_.endswith("biases"):
                p_.copy_(torch.randn(p_.shape, generator=g) * 0.1)
    v2v.train()
    x = d["x_v"].clone().to(dev).requires_grad_()
    G = torch.randn(d["nv_out"], cout, generator=g)
    y = v2v(x, face.to(dev), nf_count.to(dev), vt_map.to(dev), coeff)
    (y * G.to(dev)).sum().backward()
    out.update(v2v_x=d["x_v"].numpy(), v2v_face=face.numpy(), v2v_vt_map=vt_map.numpy(), v2v_nf_count=nf_count.numpy(),
               v2v_coeff=coeff.cpu().numpy(), v2v_G=G.numpy(), v2v_out=y.detach().cpu().numpy(),
               v2v_grad_x=x.grad.cpu().numpy(), v2v_cfg=np.array([cin, mid, cout, L, 2, 1]))
    for n_, p_ in v2v.named_parameters():
        out["v2v_param/" + n_] = p_.detach().cpu().numpy()
        out["v2v_grad/" + n_] = p_.grad.cpu().numpy()
    for n_, b_ in v2v.named_buffers():
        out["v2v_buffer/" + n_] = b_.detach().cpu().numpy()          # running statistics after the step

    cin_t, cout_t = 3, 12                                             # the networks' texture entry: RGB in
    dt = conv_inputs("ico1x3", cin_t, 1, K, cout_t, seed=73)
    bary = ref_layers.SphHarmCoeff(L)(dt["bary_xyz"].to(dev)).detach()
    torch.manual_seed(8)
    f2f = ref_layers.F2FConv3d(cin_t, cout_t, L).to(dev)
    f2f.train()
    tex = dt["tex"].clone().to(dev).requires_grad_()
    Gt = torch.randn(dt["counts"].shape[0], cout_t, generator=g)
    z = f2f(tex, bary, dt["counts"].to(dev))
    (z * Gt.to(dev)).sum().backward()
    out.update(f2f_tex=dt["tex"].numpy(), f2f_bary_xyz=dt["bary_xyz"].numpy(), f2f_bary=bary.cpu().numpy(),
               f2f_counts=dt["counts"].numpy(), f2f_G=Gt.numpy(), f2f_out=z.detach().cpu().numpy(),
               f2f_grad_tex=tex.grad.cpu().numpy(), f2f_cfg=np.array([cin_t, cout_t, L]))
    for n_, p_ in f2f.named_parameters():
        out["f2f_param/" + n_] = p_.detach().cpu().numpy()
        out["f2f_grad/" + n_] = p_.grad.cpu().numpy()
    for n_, b_ in f2f.named_buffers():
        out["f2f_buffer/" + n_] = b_.detach().cpu().numpy()

    # ---- oriented normals (origin as viewpoint) on meshes centred on the origin, so that both signs occur
    from picasso.networks.scene_seg import PicassoNetII
    dn = conv_inputs("grid17x2", 4, 1, 4, 2, seed=74)
    vert_c = (dn["vertex"] - 0.5).to(dev)
    geo_c = ref_decimate.compute_triangle_geometry_(vert_c, dn["face"].to(dev))
    out.update(orient_vertex=vert_c.cpu().numpy(), orient_face=dn["face"].numpy(), orient_geometry=geo_c.cpu().numpy(),
               orient_normals=PicassoNetII.get_oriented_normals(None, geo_c, vert_c, dn["face"].to(dev)).cpu().numpy())

    # ---- PCloudConv3d with fuzzy filter bins, depth multiplier 2
    from picasso.point import layers as ref_point_layers
    pc_args = (120, 70, 8, 9, 6, 2, 3, 75)                      # Np, Mp, knn, F, C, r, T, seed
    dp = pcloud_inputs(*pc_args)
    torch.manual_seed(9)
    pconv = ref_point_layers.PCloudConv3d(6, 10, 9, depth_multiplier=2).to(dev)
    pconv.train()
    xp = dp["x"].clone().to(dev).requires_grad_()
    Gp = torch.randn(70, 10, generator=g)
    yp = pconv(xp, dp["nn_count"].to(dev), dp["nn_index"].to(dev), dp["bin_index"].to(dev), dp["bin_coeff"].to(dev))
    (yp * Gp.to(dev)).sum().backward()
    out.update(pc_args=np.array(pc_args), pc_G=Gp.numpy(), pc_out=yp.detach().cpu().numpy(), pc_grad_x=xp.grad.cpu().numpy())
    for n_, p_ in pconv.named_parameters():
        out["pc_param/" + n_] = p_.detach().cpu().numpy()
        out["pc_grad/" + n_] = p_.grad.cpu().numpy()
    for n_, b_ in pconv.named_buffers():
        out["pc_buffer/" + n_] = b_.detach().cpu().numpy()

    os.makedirs(out_dir, exist_ok=True)
    path = os.path.join(out_dir, "modules_ref_python.npz")
    np.savez_compressed(path, **out)
    print("wrote", path, f"({os.path.getsize(path) / 1024:.0f} KB), mesh_conv3d bound to:", backend)

    # ---- the remaining layer modules, in a file of their own: PerItemConv3d (with and without batch norm /
    # activation, forward and backward) and BuildF2VCoeff (picasso/mesh/layers.py:198-240, 299-328)
    more = {}
    for tag, (cin_p, cout_p, rows_p, kw) in {"pic_bn": (16, 24, 300, {}),
                                             "pic_plain": (40, 12, 257, dict(with_bn=False, activation_fn=None))}.items():
        torch.manual_seed(11)
        pic = ref_layers.PerItemConv3d(cin_p, cout_p, **kw).to(dev)
        with torch.no_grad():
            pic.biases.copy_(torch.randn(pic.biases.shape, generator=g) * 0.1)
        pic.train()
        xin = torch.randn(rows_p, cin_p, generator=g)
        xq = xin.clone().to(dev).requires_grad_()
        Gq = torch.randn(rows_p, cout_p, generator=g)
        yq = pic(xq)
        (yq * Gq.to(dev)).sum().backward()
        more.update({f"{tag}_cfg": np.array([cin_p, cout_p]), f"{tag}_x": xin.numpy(), f"{tag}_G": Gq.numpy(),
                     f"{tag}_out": yq.detach().cpu().numpy(), f"{tag}_grad_x": xq.grad.cpu().numpy()})
        for n_, p_ in pic.named_parameters():
            more[f"{tag}_param/" + n_] = p_.detach().cpu().numpy()
            more[f"{tag}_grad/" + n_] = p_.grad.cpu().numpy()
        for n_, b_ in pic.named_buffers():
            more[f"{tag}_buffer/" + n_] = b_.detach().cpu().numpy()
    torch.manual_seed(12)
    if dev.type == "cpu":
        torch.Tensor.get_device = lambda self: self.device          # the reference asks a CPU tensor for its device
    f2vc = ref_layers.BuildF2VCoeff(9, tau=0.2).to(dev)
    normals = torch.nn.functional.normalize(torch.randn(200, 3, generator=g), dim=1)
    more.update(f2vc_normals=normals.numpy(), f2vc_centers=f2vc.centers.detach().cpu().numpy(),
                f2vc_out=f2vc(normals.to(dev)).detach().cpu().numpy(), f2vc_cfg=np.array([9, 0.2]))
    path2 = os.path.join(out_dir, "layers_ref_python.npz")
    np.savez_compressed(path2, **more)
    print("wrote", path2, f"({os.path.getsize(path2) / 1024:.0f} KB)")


if __name__ == "__main__":
    main(sys.argv[1] if len(sys.argv) > 1 else HERE)
