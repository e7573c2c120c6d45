"""Times the reference's own CUDA kernels (oracle/_ref, built unmodified for sm_100a by
`make -C oracle ref`) on the benchmark block V2F -> F2F -> F2V, forward + backward, on the
same seeded synthetic inputs bench.py uses.  TEST INFRASTRUCTURE: a second baseline beside
the CPU oracle, run by hand on a GPU box; nothing in the product imports it.

    python -m oracle.time_ref_cuda --config c1 [--meshes N] [--steps 3]

Prints one JSON line.  The reference ops run on the legacy default stream and the wrapper
synchronises before every call, so sub-millisecond configs include that host overhead.
"""
from __future__ import annotations

import argparse
import json
import os
import sys

import torch

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
sys.path.insert(0, ROOT)

from oracle import mesh_oracle, ref_cuda  # noqa: E402
from picassoplus_b200 import synth  # noqa: E402
import bench  # noqa: E402  (input generators only)


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--config", default="c1")
    ap.add_argument("--meshes", type=int, default=0)
    ap.add_argument("--steps", type=int, default=3)
    args = ap.parse_args()
    if not ref_cuda.available():
        print(json.dumps({"impl": "reference-cuda", "unavailable": "oracle/_ref not built or no GPU"}))
        return
    cfg = dict(synth.CONFIGS[args.config])
    count = args.meshes or cfg["batch"]
    h = bench.host_inputs(cfg, 0, count)
    Wv, Wf, Wo = bench.make_params(cfg)
    dev = torch.device("cuda", 0)
    L = h["L"]
    vertex, face, x, cum, bary_xyz = (h[k].to(dev) for k in ("vertex", "face", "x", "cum", "bary_xyz"))
    counts = h["counts"].to(dev).long()
    vt_map = torch.arange(h["Nv"], dtype=torch.int32, device=dev)
    Wv, Wf, Wo = Wv.to(dev), Wf.to(dev), Wo.to(dev)
    # per-batch preparation with the oracle's formulas (not timed)
    nfc = mesh_oracle.count_vertex_adjface(h["face"], torch.arange(h["Nv"], dtype=torch.int32), h["Nv"]).to(dev)
    geo = mesh_oracle.triangle_geometry(h["vertex"], h["face"])
    coeff = mesh_oracle.sph_harm_coeff(L, geo[:, :3].contiguous()).to(dev)
    bary_sh = mesh_oracle.sph_harm_coeff(L, h["bary_xyz"]).to(dev)
    sh_eye = mesh_oracle.sph_harm_coeff(L, torch.eye(3)).to(dev)
    spatial = (sh_eye @ Wv).reshape(3, cfg["cin"], 1).contiguous()
    seg = torch.repeat_interleave(torch.arange(h["Nf"], device=dev), counts)
    G = torch.randn(h["Nv"], cfg["cout"], device=dev, generator=torch.Generator(device=dev).manual_seed(1))

    def step():
        y = ref_cuda.v2f_forward(x, spatial, face)
        tex = y.index_select(0, seg)
        z = ref_cuda.f2f_forward(tex, Wf, bary_sh, cum)
        o = ref_cuda.f2v_forward(z, Wo, coeff, face, nfc, vt_map)
        gz, gWo = ref_cuda.f2v_backward(G, z, Wo, coeff, face, nfc, vt_map)
        gtex, gWf = ref_cuda.f2f_backward(gz.contiguous(), tex, Wf, bary_sh, cum)
        gy = torch.zeros_like(y).index_add_(0, seg, gtex)
        gx, gWv = ref_cuda.v2f_backward(gy, x, spatial, face)
        return o, gx, gWf

    step()
    torch.cuda.synchronize()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    for _ in range(args.steps):
        step()
    e1.record()
    torch.cuda.synchronize()
    ms = e0.elapsed_time(e1) / args.steps
    print(json.dumps({"impl": "reference-cuda", "config": args.config, "meshes": count, "faces": h["Nf"],
                      "ms_per_step": ms, "faces_per_s": h["Nf"] / (ms / 1e3), "steps": args.steps,
                      "note": "reference kernels of picasso/mesh/pi_modules/source/mesh_conv3d_gpu.cu compiled for "
                              "sm_100a; block glue (repeat/segment-sum) in torch"}))


if __name__ == "__main__":
    main()
