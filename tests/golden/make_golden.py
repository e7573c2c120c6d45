"""Makes the fixtures in this folder by running the reference's own, unmodified CUDA
operators (oracle/_ref, see oracle/Makefile target `ref`) on a CUDA device:

    python tests/golden/make_golden.py [output_dir]

For every case of tests/cases.py:GOLDEN_CASES it stores the inputs and the reference's
outputs (all three operators forward and backward, and nfCount) in <case>.npz, and for
every case of POOL_GOLDEN_CASES / PCLOUD_GOLDEN_CASES the reference's mesh pooling / unpooling and
point-cloud convolution outputs, for every case of DECIMATE_GOLDEN_CASES two passes of the reference's
mesh decimation and the merge of their clusters.  The parts
of the path that are plain Python in the reference (spherical-harmonic basis, triangle
geometry, layer modules) have their own generator, make_golden_modules.py.
"""
from __future__ import annotations

import os
import sys

import numpy as np
import torch

ROOT = os.path.dirname(os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
sys.path.insert(0, ROOT)
sys.path.insert(0, os.path.join(ROOT, "tests"))

from cases import (DECIMATE_GOLDEN_CASES, GOLDEN_CASES, PCLOUD_GOLDEN_CASES, POOL_GOLDEN_CASES, cluster_inputs,  # noqa: E402
                   conv_inputs, decimate_inputs, pcloud_inputs)
from oracle import c_oracle  # noqa: E402
from oracle import ref_cuda  # noqa: E402


def main(out_dir):
    assert ref_cuda.available(), "needs oracle/_ref/libref_mesh_conv3d.so and a CUDA device"
    os.makedirs(out_dir, exist_ok=True)
    dev = torch.device("cuda:0")
    for name, (kind, C, r, K, cout, seed) in GOLDEN_CASES.items():
        d = conv_inputs(kind, C, r, K, cout, seed)
        c = {k: (v.to(dev) if isinstance(v, torch.Tensor) else v) for k, v in d.items()}
        nf_count = ref_cuda.count_vertex_adjface(c["face"], c["vt_map"], d["nv_out"])
        out = dict(nf_count=nf_count)
        out["v2f_out"] = ref_cuda.v2f_forward(c["x_v"], c["filt_v2f"], c["face"])
        out["v2f_gin"], out["v2f_gf"] = ref_cuda.v2f_backward(c["g_v2f"], c["x_v"], c["filt_v2f"], c["face"])
        out["f2v_out"] = ref_cuda.f2v_forward(c["x_f"], c["filt_f2v"], c["coeff"], c["face"], nf_count, c["vt_map"])
        out["f2v_gin"], out["f2v_gf"] = ref_cuda.f2v_backward(c["g_f2v"], c["x_f"], c["filt_f2v"], c["coeff"],
                                                              c["face"], nf_count, c["vt_map"])
        out["f2f_out"] = ref_cuda.f2f_forward(c["tex"], c["filt_f2f"], c["bary"], c["cum"])
        out["f2f_gin"], out["f2f_gf"] = ref_cuda.f2f_backward(c["g_f2f"], c["tex"], c["filt_f2f"], c["bary"], c["cum"])
        arrays = {("in_" + k): v.numpy() for k, v in d.items() if isinstance(v, torch.Tensor)}
        arrays.update({("ref_" + k): v.cpu().numpy() for k, v in out.items()})
        arrays["nv_out"] = np.array(d["nv_out"])
        np.savez_compressed(os.path.join(out_dir, name + ".npz"), **arrays)
        print("wrote", name, {k: tuple(v.shape) for k, v in arrays.items() if k.startswith("ref_")})
    # mesh pool / unpool (mesh_pool3d_gpu.cu, mesh_unpool3d_gpu.cu); inputs without ties, so the
    # reference's max index does not depend on its thread order
    for name, (nv_in, nv_out, C, seed) in POOL_GOLDEN_CASES.items():
        d = cluster_inputs(nv_in, nv_out, C, seed)
        c = {k: (v.to(dev) if isinstance(v, torch.Tensor) else v) for k, v in d.items()}
        out = {}
        out["max_out"], out["max_index"] = ref_cuda.max_pool_forward(c["x"], c["vt_replace"], c["vt_map"], nv_out)
        out["max_gin"] = ref_cuda.max_pool_backward(c["g_coarse"], nv_in, out["max_index"])
        out["avg_out"] = ref_cuda.avg_pool_forward(c["x"], c["vt_replace"], c["vt_map"], nv_out)
        out["avg_gin"] = ref_cuda.avg_pool_backward(c["g_coarse"], c["vt_replace"], c["vt_map"])
        out["unpool_out"] = ref_cuda.unpool_forward(c["x_coarse"], c["vt_replace"], c["vt_map"])
        out["unpool_gin"] = ref_cuda.unpool_backward(c["g_fine"], nv_out, c["vt_replace"], c["vt_map"])
        arrays = {("in_" + k): v.numpy() for k, v in d.items() if isinstance(v, torch.Tensor)}
        arrays.update({("ref_" + k): v.cpu().numpy() for k, v in out.items()})
        np.savez_compressed(os.path.join(out_dir, name + ".npz"), **arrays)
        print("wrote", name, {k: tuple(v.shape) for k, v in arrays.items() if k.startswith("ref_")})
    # point-cloud depthwise convolution, hard and fuzzy bins (pcloud_conv3d_gpu.cu)
    for name, args in PCLOUD_GOLDEN_CASES.items():
        d = pcloud_inputs(*args)
        c = {k: (v.to(dev) if isinstance(v, torch.Tensor) else v) for k, v in d.items()}
        out = {"out": ref_cuda.pcloud_forward(c["x"], c["filt"], c["nn_count"], c["nn_index"], c["bin_index"], c["bin_coeff"])}
        out["gin"], out["gf"] = ref_cuda.pcloud_backward(c["g_out"], c["x"], c["filt"], c["nn_count"], c["nn_index"],
                                                         c["bin_index"], c["bin_coeff"])
        arrays = {("in_" + k): v.numpy() for k, v in d.items() if isinstance(v, torch.Tensor)}
        arrays.update({("ref_" + k): v.cpu().numpy() for k, v in out.items()})
        np.savez_compressed(os.path.join(out_dir, name + ".npz"), **arrays)
        print("wrote", name, {k: tuple(v.shape) for k, v in arrays.items() if k.startswith("ref_")})
    # mesh decimation (decimate_gpu.cu): two passes as decimate.py:30-46 chains them, and the cluster merge
    names = ("vertexOut", "faceOut", "isDegenerate", "vtReplace", "vtMap", "nvOut", "mfOut")
    for name, (meshes, frac, D, seed, noise, use_area, wgt_bnd) in DECIMATE_GOLDEN_CASES.items():
        d = decimate_inputs(meshes, frac, D, seed, noise)
        c = {k: v.to(dev) for k, v in d.items()}
        arrays = {("in_" + k): v.numpy() for k, v in d.items()}
        arrays["use_area"], arrays["wgt_bnd"] = np.array(use_area), np.array(wgt_bnd, np.float32)
        r1 = ref_cuda.mesh_simplify(c["vertex"], c["face"], c["geometry"], c["nv_cum"], c["mf_cum"], c["remove"],
                                    use_area, wgt_bnd)
        again = ref_cuda.mesh_simplify(c["vertex"], c["face"], c["geometry"], c["nv_cum"], c["mf_cum"], c["remove"],
                                       use_area, wgt_bnd)
        assert all(torch.equal(r1[k], again[k]) for k in names if k != "vertexOut"), "reference not repeatable on " + name
        arrays.update({("ref1_" + k): r1[k].cpu().numpy() for k in names})
        # second pass on the compacted mesh: every sample sheds a third of what it has left
        face2 = r1["faceOut"][~r1["isDegenerate"]].contiguous()
        vertex2 = r1["vertexOut"][r1["vtMap"] >= 0].contiguous()
        geo2 = torch.from_numpy(c_oracle.triangle_geometry(vertex2[:, :3].cpu().numpy().copy(), face2.cpu().numpy())).to(dev)
        nv2, mf2 = r1["nvOut"], r1["mfOut"]
        nv_cum2 = torch.cumsum(nv2, 0, dtype=torch.int32)
        mf_cum2 = torch.cumsum(mf2, 0, dtype=torch.int32)
        remove2 = (nv2 // 3).to(torch.int32)
        r2 = ref_cuda.mesh_simplify(vertex2, face2, geo2, nv_cum2, mf_cum2, remove2, use_area, wgt_bnd)
        arrays.update(in2_vertex=vertex2.cpu().numpy(), in2_face=face2.cpu().numpy(), in2_geometry=geo2.cpu().numpy(),
                      in2_nv_cum=nv_cum2.cpu().numpy(), in2_mf_cum=mf_cum2.cpu().numpy(), in2_remove=remove2.cpu().numpy())
        arrays.update({("ref2_" + k): r2[k].cpu().numpy() for k in names})
        rep, mp = ref_cuda.combine_clusters(r1["vtReplace"], r1["vtMap"], r2["vtReplace"], r2["vtMap"])
        arrays["ref_comb_rep"], arrays["ref_comb_map"] = rep.cpu().numpy(), mp.cpu().numpy()
        np.savez_compressed(os.path.join(out_dir, name + ".npz"), **arrays)
        print("wrote", name, "nvOut", r1["nvOut"].tolist(), "->", r2["nvOut"].tolist())


if __name__ == "__main__":
    main(sys.argv[1] if len(sys.argv) > 1 else os.path.dirname(os.path.abspath(__file__)))
