#!/usr/bin/env python
"""Benchmark of the mesh-convolution block (vertex2facet -> facet2facet -> facet2vertex,
forward + backward, + all-reduce of filter gradients when N > 1).

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl ours|reference]
                    [--config c5] [--precision fp32|tf32|bf16] [--meshes M]

Under torchrun (N > 1) one rank drives one GPU; rank 0 prints ONE JSON line.
Metric: faces per second of one fwd+bwd pass of the block over the whole batch.
  value     inputs resident in HBM, timed with CUDA events, max over ranks
  e2e       the same step through the public operator API starting from pinned HOST buffers:
            H2D of the batch (vertices, faces, features, texture samples), on-device
            per-batch preparation (nfCount, normals, SH coefficients, CSR), fwd+bwd, D2H of
            the loss
  roofline  the dominant kernel of the step: algorithmic bytes (or flops) / measured duration
  cpu_baseline  the CPU oracle (PyTorch composition of the same formulas) on a bounded sample
`--impl reference` times that CPU composition alone (the reference has no CPU code path of
its own; its operators are CUDA-only).
"""
from __future__ import annotations

import argparse
import json
import os
import statistics
import subprocess
import sys
import threading
import time

import numpy as np
import torch

ROOT = os.path.dirname(os.path.abspath(__file__))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)

from picassoplus_b200 import synth  # noqa: E402

METRIC = "mesh_conv_block_fwd_bwd_faces_per_sec"
UNIT = "faces/s"
# max|a-b| / max|b| per tensor that each precision mode of facet2facet must meet
GATES = {"fp32": 1e-4, "fp32_tf32x3": 1e-4, "tf32": 2e-3, "bf16": 2e-2}


def parse_args():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=10)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--config", default="c5", choices=sorted(synth.CONFIGS) + ["c4", "decimate", "aux"])
    ap.add_argument("--precision", default="fp32", choices=["fp32", "fp32_tf32x3", "tf32", "bf16"])
    ap.add_argument("--meshes", type=int, default=0, help="total meshes of the batch (0 = the configuration's)")
    ap.add_argument("--no-e2e", action="store_true")
    ap.add_argument("--graph", action="store_true", help="also time the step replayed from a CUDA graph "
                    "(done by default when a step takes less than 3 ms)")
    ap.add_argument("--e2e-groups", type=int, default=0,
                    help="mesh groups of the end-to-end step (host-to-device copy of one overlaps compute of another); "
                         "0 = one group per 256 MB of host input, at most 4")
    ap.add_argument("--no-cpu-baseline", action="store_true")
    ap.add_argument("--no-variants", action="store_true")
    ap.add_argument("--no-cpu-binding", action="store_true",
                    help="multi-GPU runs: leave the ranks' CPU affinity alone (default: bind each rank to the cores near its GPU)")
    ap.add_argument("--no-parity", action="store_true")
    ap.add_argument("--hierarchy", default="decimate", choices=["decimate", "grid"],
                    help="config c4: mesh levels by the library's quadric-error decimation (stride 4 per level) or by "
                         "halving the height-field grid")
    ap.add_argument("--no-fusion", action="store_true", help="config c4: run the layer modules as operator + separate "
                    "pointwise kernels instead of the fused operator + pointwise kernels")
    ap.add_argument("--cpu-seconds", type=float, default=15.0, help="target CPU time of one baseline step")
    return ap.parse_args()


def workload_name(cfg, total_meshes):
    if cfg["kind"] == "heightfield":
        shape = f"{total_meshes} heightfield meshes {cfg['n']}x{cfg['n']} (10% faces deleted)"
    else:
        shape = f"{total_meshes} icospheres level {cfg['level']} ({cfg['mode']})"
    return f"{shape}, V2F->F2F->F2V block, Cin={cfg['cin']} Cout={cfg['cout']} L={cfg['L']}"


# ------------------------------------------------------------------------------ inputs
def host_inputs(cfg, first, count, seed_shift=0):
    """Host-side batch of meshes [first, first+count).  Features and texture samples are seeded
    PER MESH (by the mesh's index in the whole batch), so a mesh carries the same data whatever
    the number of ranks or mesh groups it is dealt to."""
    mb = synth.make_batch(cfg, count, first)
    L = cfg["L"]
    K = (L + 1) ** 2
    counts, bary_xyz, xs = [], [], []
    for j in range(count):
        i = first + j
        cj, bj = synth.texture_samples(int(mb.mf[j]), cfg["seed"] * 7919 + i)
        counts.append(cj)
        bary_xyz.append(bj)
        g = torch.Generator().manual_seed(cfg["seed"] * 104729 + i + seed_shift)
        xs.append(torch.randn(int(mb.nv[j]), cfg["cin"], generator=g))
    counts = np.concatenate(counts)
    bary_xyz = np.concatenate(bary_xyz)
    return dict(vertex=torch.from_numpy(mb.vertex), face=torch.from_numpy(mb.face),
                counts=torch.from_numpy(counts), cum=torch.cumsum(torch.from_numpy(counts), 0, dtype=torch.int32),
                bary_xyz=torch.from_numpy(bary_xyz), x=torch.cat(xs), K=K, L=L,
                Nv=mb.num_vertices, Nf=mb.num_faces, NiK=int(counts.sum()), nmesh=count,
                nv=[int(v) for v in mb.nv], mf=[int(f) for f in mb.mf])


def upstream_gradient(cfg, first, nv_per_mesh, dev):
    """The block's upstream gradient, seeded per mesh like the inputs (device generator)."""
    parts = []
    for j, nv in enumerate(nv_per_mesh):
        gen = torch.Generator(device=dev).manual_seed(cfg["seed"] * 31 + first + j)
        parts.append(torch.randn(nv, cfg["cout"], generator=gen, device=dev))
    return torch.cat(parts)


def make_params(cfg):
    """Xavier-normal filters, identical on every rank."""
    rng = np.random.default_rng(cfg["seed"] + 12345)
    K = (cfg["L"] + 1) ** 2
    Wv = torch.from_numpy(synth.xavier_normal((K, cfg["cin"]), rng))
    Wf = torch.from_numpy(synth.xavier_normal((cfg["cout"], cfg["cin"], K), rng))
    Wo = torch.from_numpy(synth.xavier_normal((K, cfg["cout"], 1), rng))
    return Wv, Wf, Wo


# ------------------------------------------------------------------------------ clocks
class ClockSampler:
    """nvidia-smi in loop mode beside the timed region.  Entering waits until the first sample has arrived
    (so the sampler is already running when the timed region starts, however short that is), and the summary
    counts only samples whose own timestamps lie inside the region."""
    FIELDS = ("timestamp,uuid,clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.hw_slowdown,"
              "clocks_event_reasons.hw_thermal_slowdown,clocks_event_reasons.sw_thermal_slowdown,"
              "clocks_event_reasons.sw_power_cap")

    def __init__(self, uuid, active=True):
        self.uuid = uuid
        self.active = active                                   # only rank 0 samples (its own GPU)
        self.lines = []
        self.proc = None
        self.t0 = self.t1 = None

    def __enter__(self):
        if not self.active:
            return self
        try:
            self.proc = subprocess.Popen(["nvidia-smi", f"--query-gpu={self.FIELDS}", "--format=csv,noheader,nounits",
                                          "-lms", "25"], stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True)
            self.thread = threading.Thread(target=self._pump, daemon=True)
            self.thread.start()
            deadline = time.time() + 2.0
            while not self.lines and time.time() < deadline:
                time.sleep(0.005)
        except OSError:
            self.proc = None
        self.t0 = time.time()
        return self

    def _pump(self):
        for line in self.proc.stdout:
            self.lines.append(line)

    def __exit__(self, *exc):
        self.t1 = time.time()
        if self.proc is not None:
            time.sleep(0.03)                                   # let the sample taken at the end arrive
            self.proc.terminate()
            try:
                self.proc.wait(timeout=5)
            except subprocess.TimeoutExpired:
                self.proc.kill()

    @staticmethod
    def _stamp(text):
        import datetime
        try:
            return datetime.datetime.strptime(text.strip(), "%Y/%m/%d %H:%M:%S.%f").timestamp()
        except ValueError:
            return None

    def summary(self):
        names = ["hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"]
        rows = []
        for line in self.lines:
            parts = [p.strip() for p in line.split(",")]
            if len(parts) < 9 or (self.uuid and self.uuid not in parts[1]):
                continue
            try:
                rows.append((self._stamp(parts[0]), float(parts[2]), float(parts[3]), parts[5:9]))
            except ValueError:
                continue
        inside = [r for r in rows if r[0] is not None and self.t0 is not None and self.t0 - 0.005 <= r[0] <= self.t1 + 0.005]
        note = None
        if not inside and rows and self.t0 is not None:
            # a region shorter than the sampling interval: the sample closest to it
            mid = 0.5 * (self.t0 + self.t1)
            stamped = [r for r in rows if r[0] is not None]
            if stamped:
                inside = [min(stamped, key=lambda r: abs(r[0] - mid))]
                note = "timed region shorter than the sampling interval: nearest sample"
        if not inside:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": [], "samples": 0}
        reasons = set()
        for r in inside:
            for n, v in zip(names, r[3]):
                if v == "Active":
                    reasons.add(n)
        out = {"sm_mhz": statistics.median(r[1] for r in inside), "sm_max_mhz": max(r[2] for r in inside),
               "reasons": sorted(reasons), "samples": len(inside)}
        if note:
            out["note"] = note
        return out


def gpu_uuid(dev):
    try:
        return "GPU-" + str(torch.cuda.get_device_properties(dev).uuid)
    except Exception:
        return ""


# ---------------------------------------------------------------------- kernel models
def kernel_models(d):
    """Algorithmic (compulsory) bytes and contraction flops of one launch set per step,
    by kernel label: every operand read once, every result written once; fp32 / int32."""
    Nv, Nf, NiK, Ci, Co, K = d["Nv"], d["Nf"], d["NiK"], d["cin"], d["cout"], d["K"]
    Q = K * Ci
    # sample rows that facet2facet itself sees: one per face when the block folds the repetition of the face rows
    # into per-face mean weights (face_mean_rows), every sample when the block runs as written
    Ns = d.get("f2f_samples", NiK)
    m = {
        "v2f_fwd": dict(bytes=4 * Ci * Nv + 12 * Nf + 4 * Ci * Nf),
        "v2f_bwd": dict(bytes=4 * Ci * Nf + 8 * Ci * Nv + 12 * Nf + 4 * Nv),
        "expand_rows_fwd": dict(bytes=4 * Ci * Nf + 4 * Nf + 4 * Ci * NiK),
        "expand_rows_bwd": dict(bytes=4 * Ci * Nf + 4 * Nf + 4 * Ci * NiK),
        # facet2vertex forward = per-face products (wx) + CSR gather
        "f2v_fwd_face": dict(bytes=8 * Co * Nf + 4 * K * Nf),
        "f2v_fwd_gather": dict(bytes=4 * Co * Nf + 12 * Nf + 8 * Nv + 4 * Co * Nv),
        "f2v_bwd": dict(bytes=4 * Co * Nv + 8 * Co * Nf + 4 * K * Nf + 12 * Nf + 4 * Nv),
        # fp32 FFMA path of facet2facet (chunked through workspace)
        "f2f_build_A": dict(bytes=4 * Ci * NiK + 4 * K * NiK + 4 * Nf + 4 * Q * Nf),
        "f2f_fwd_sgemm": dict(bytes=4 * Q * Nf + 4 * Co * Nf, flops=2 * Q * Co * Nf),
        "f2f_gfilter_sgemm": dict(bytes=4 * Q * Nf + 4 * Co * Nf, flops=2 * Q * Co * Nf),
        "f2f_gA_sgemm": dict(bytes=4 * Q * Nf + 4 * Co * Nf, flops=2 * Q * Co * Nf),
        "f2f_gin_from_gA": dict(bytes=4 * Q * Nf + 4 * K * NiK + 4 * Ci * NiK),
        # fused tensor-core path of facet2facet
        "f2f_fwd_tc": dict(bytes=4 * Ci * Ns + 4 * K * Ns + 4 * Nf + 4 * Co * Nf,
                           flops=2 * Q * Ns + 2 * Q * Co * Nf),
        "f2f_bwd_gin_tc": dict(bytes=4 * Co * Nf + 4 * K * Ns + 4 * Nf + 4 * Ci * Ns,
                               flops=2 * Q * Ns + 2 * Q * Co * Nf),
        "f2f_bwd_gfilter_tc": dict(bytes=4 * Ci * Ns + 4 * K * Ns + 4 * Nf + 4 * Co * Nf,
                                   flops=2 * Q * Ns + 2 * Q * Co * Nf),
        "face_mean_rows": dict(bytes=4 * K * NiK + 4 * Nf + 4 * K * Nf),
        # forward for one sample per face: a plain product over the input rows, the sum over the bases in the epilogue
        "f2f_fwd_one_sample_tc": dict(bytes=4 * Ci * Nf + 4 * K * Nf + 4 * Co * Nf, flops=2 * Q * Co * Nf + 2 * K * Co * Nf),
    }
    return m


# DRAM bytes per face of one launch (dram__bytes_read.sum + dram__bytes_write.sum of an ncu
# capture on a 2-mesh case of the same shapes, divided by its face count; traffic grows in
# proportion to the faces).  Source: the summaries under profiles/.
MEASURED_DRAM_BYTES_PER_FACE = {
    # the block with the repetition of the face rows folded in (one sample per face reaches facet2facet)
    ("c5", "f2f_fwd_one_sample_tc"): 1041.0,
    ("c5", "f2f_bwd_gin_tc"): 1043.0,
    ("c5", "f2f_bwd_gfilter_tc"): 1858.0,
    # the general forward kernel over every sample (variants.block_as_written)
    ("c5", "f2f_fwd_tc"): 2001.0,
}


MMAS_PER_PRODUCT = {"fp32": 3, "fp32_tf32x3": 3, "tf32": 1, "bf16": 1}


def load_peaks():
    p = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.exists(p):
        j = json.load(open(p))
        return dict(hbm_gbs=float(j["hbm_gbs"]), tflops=float(j.get("bf16_tflops_sustained", j["bf16_tflops"])),
                    source="measured (MEASURED_PEAKS.json; tensor = sustained bf16)")
    return dict(hbm_gbs=6650.0, tflops=1400.0, source="fallback (6.65 TB/s, 1.4 PFLOP/s sustained bf16)")


def roofline_from_profile(records, steps, dims):
    """records: [(label, launches, total_ms)] over `steps` steps.  The dominant kernel label
    (largest total time) gets: achieved = algorithmic bytes|flops per step / its time per step."""
    models = kernel_models(dims)
    peaks = load_peaks()
    total = sum(r[2] for r in records) or 1.0
    table = []
    for name, launches, ms in records:
        row = dict(kernel=name, launches_per_step=launches / steps, ms_per_step=ms / steps, share=ms / total)
        mdl = models.get(name)
        if mdl:
            sec = ms / steps / 1e3
            gbs = mdl["bytes"] / sec / 1e9
            row["hbm_gbs"] = gbs
            row["hbm_frac"] = gbs / peaks["hbm_gbs"]
            if "flops" in mdl:
                tf = mdl["flops"] / sec / 1e12
                row["tflops"] = tf
                row["tensor_frac"] = tf / peaks["tflops"]
                # what the tensor cores are asked to do for those flops: three bf16 (or tf32) products per term in
                # the two hi + lo modes, one in the single-operand modes
                mmas = MMAS_PER_PRODUCT.get(dims.get("precision"), 1) if name.endswith("_tc") else 1
                row["mmas_per_product"] = mmas
                row["tensor_issued_frac"] = mmas * tf / peaks["tflops"]
        table.append(row)
    top = table[0] if table else None
    roof = None
    if top and top["kernel"] in models:
        mdl = models[top["kernel"]]
        t_hbm = mdl["bytes"] / (peaks["hbm_gbs"] * 1e9)
        t_tc = mdl.get("flops", 0) / (peaks["tflops"] * 1e12)
        if t_tc > t_hbm:
            roof = dict(bound="tensor", achieved=top["tflops"], peak=peaks["tflops"], unit="TFLOP/s",
                        frac=top["tensor_frac"], traffic=None, mmas_per_product=top.get("mmas_per_product", 1),
                        issued_frac=top.get("tensor_issued_frac"),
                        issued_note="frac counts algorithmic flops; the fp32-faithful mode issues mmas_per_product "
                                    "tensor-core products per term (bf16 hi + lo operands), issued_frac counts those")
        else:
            roof = dict(bound="hbm", achieved=top["hbm_gbs"], peak=peaks["hbm_gbs"], unit="GB/s",
                        frac=top["hbm_frac"], traffic=None)
        roof.update(kernel=top["kernel"], peak_source=peaks["source"], ms_per_launch_set=top["ms_per_step"],
                    share_of_step=top["share"])
        per_face = MEASURED_DRAM_BYTES_PER_FACE.get((dims.get("config"), top["kernel"]))
        if per_face is not None:
            roof["traffic"] = per_face * dims["Nf"]
            roof["traffic_note"] = "ncu dram bytes of a 2-mesh capture scaled by faces (profiles/)"
    return roof, table


# ------------------------------------------------------------------------------- ours
def run_ours(args):
    import torch.distributed as dist
    from picassoplus_b200 import _lib
    from picassoplus_b200.block import conv_block, conv_block_expanded
    from picassoplus_b200.math_utils import sph_harm_coeff
    from picassoplus_b200.mesh import utils as mesh_utils
    from picassoplus_b200.mesh.pi_modules import conv3d
    from picassoplus_b200.parallel import FilterGradAllReduce, HostBatchFeed, bind_to_gpu_cpus, partition_meshes

    rank = int(os.environ.get("RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    local = int(os.environ.get("LOCAL_RANK", "0"))
    if not torch.cuda.is_available():
        raise SystemExit("bench.py needs a CUDA device (there is no CPU fallback for --impl ours)")
    torch.cuda.set_device(local)
    dev = torch.device("cuda", local)
    # several ranks on one host: keep each rank's pinned staging buffers on the socket of its GPU
    near_cpus = bind_to_gpu_cpus(local) if world > 1 and not args.no_cpu_binding else 0
    if world > 1:
        dist.init_process_group("nccl", device_id=dev)
    assert world == args.gpus or world == 1, f"WORLD_SIZE={world} but --gpus {args.gpus}"

    cfg = dict(synth.CONFIGS[args.config])
    total_meshes = args.meshes or cfg["batch"]
    cfg["batch"] = total_meshes
    first, count = partition_meshes([1] * total_meshes, world)[rank]
    conv3d.set_f2f_precision(args.precision)

    h = host_inputs(cfg, first, count)
    L, K = h["L"], h["K"]
    Wv, Wf, Wo = make_params(cfg)
    pin = {k: h[k].pin_memory() for k in ("vertex", "face", "x", "cum", "bary_xyz")}
    d = {k: v.to(dev) for k, v in pin.items()}
    vt_map = torch.arange(h["Nv"], dtype=torch.int32, device=dev)
    G = upstream_gradient(cfg, first, h["nv"], dev)
    params = [w.to(dev).requires_grad_() for w in (Wv, Wf, Wo)]
    allreduce = FilterGradAllReduce(params)
    sh_eye = sph_harm_coeff(L, torch.eye(3, device=dev))

    def prepare():
        nfc = mesh_utils.count_vertex_adjface(d["face"], vt_map, d["vertex"])
        geo = mesh_utils.compute_triangle_geometry(d["vertex"], d["face"])
        coeff = sph_harm_coeff(L, geo[:, :3].contiguous())
        bary_sh = sph_harm_coeff(L, d["bary_xyz"])
        return nfc, coeff, bary_sh

    nfc, coeff, bary_sh = prepare()
    xd = d["x"].requires_grad_()

    block_fn = [conv_block]            # the variants swap in the block as written

    def step_resident():
        for p in params:
            p.grad = None
        xd.grad = None
        o = block_fn[0](xd, params[0], params[1], params[2], d["face"], d["cum"], bary_sh, coeff, nfc, vt_map, sh_eye)
        o.backward(G)
        allreduce()

    # End to end: the rank's meshes are fed from pinned host memory in groups; the copy of
    # group g+1 overlaps the fwd+bwd of group g (filter gradients accumulate over the groups).
    host_bytes = sum(h[k].numel() * h[k].element_size() for k in ("vertex", "face", "x", "cum", "bary_xyz"))
    # one group per 300 MB of host input, at most four.  Every group costs about 0.6 ms of fixed work (preparation,
    # CSR build, launches), and the feed is double-buffered across steps as well (the first group of the next step
    # is copied while the last group of this one is computed), so a small shard goes in one piece.
    want_groups = args.e2e_groups if args.e2e_groups > 0 else max(1, min(4, host_bytes // (300 << 20)))
    ngroups = max(1, min(want_groups, count))
    feed = None
    if not args.no_e2e:
        pinned_groups, group_G = [], []
        for gfirst, gcount in [(first + a, b) for a, b in partition_meshes([1] * count, ngroups) if b > 0]:
            hg = h if ngroups == 1 else host_inputs(cfg, gfirst, gcount)
            pinned_groups.append({k: hg[k].pin_memory() for k in ("vertex", "face", "x", "cum", "bary_xyz")})
            group_G.append(upstream_gradient(cfg, gfirst, hg["nv"], dev))
        feed = HostBatchFeed(pinned_groups, dev, depth=2)
    h2d_bytes = feed.bytes_per_pass if feed is not None else 0
    # step after step over the same pinned groups: the first group of the next step is copied while
    # the last group of the current one is computed
    feed_cycle = feed.cycle() if feed is not None else None

    from picassoplus_b200 import topology

    def step_e2e():
        # index validation without a host round trip per group: the status words of the CSR builds are
        # read after the step's own synchronisation (the loss read-back)
        topology.set_validation("deferred")
        for p in params:
            p.grad = None
        total = torch.zeros((), device=dev)
        for gi in range(len(group_G)):                     # fresh copies: topology is rebuilt per group
            b = next(feed_cycle)
            nv = b["vertex"].shape[0]
            vt = vt_map[:nv]
            # nfCount, face normals, their SH coefficients and the vertex CSR in one library call
            lvl = topology.prepare_level(b["vertex"], b["face"], vt, nv, L, want_geometry=False)
            nfc_, coeff_ = lvl["nf_count"], lvl["coeff"]
            # SH components of the texture samples, averaged per face in the same kernel (all the folded block needs)
            bary_ = topology.face_means_sph_harm(L, b["bary_xyz"], b["cum"])
            xe = b["x"].detach().requires_grad_()
            o = conv_block(xe, params[0], params[1], params[2], b["face"], b["cum"], bary_, coeff_, nfc_, vt, sh_eye)
            # loss = sum(o * G): its value by one dot product, its gradient with respect to o is G itself
            with torch.no_grad():
                total = total + torch.dot(o.reshape(-1), group_G[gi].reshape(-1))
            o.backward(group_G[gi])
        allreduce()
        out = float(total.item())
        topology.check_deferred()
        topology.set_validation("sync")
        return out

    def barrier():
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()

    def timed(fn, steps):
        barrier()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        n0 = _lib.launch_count()
        e0.record()
        for _ in range(steps):
            fn()
        e1.record()
        barrier()
        ms = torch.tensor([e0.elapsed_time(e1)], device=dev)
        if world > 1:
            dist.all_reduce(ms, op=dist.ReduceOp.MAX)
        return float(ms.item()), _lib.launch_count() - n0

    # total faces over all ranks
    nf_all = torch.tensor([h["Nf"], h["Nv"], h["NiK"]], device=dev, dtype=torch.float64)
    if world > 1:
        dist.all_reduce(nf_all)
    faces_total = float(nf_all[0].item())

    for _ in range(max(args.warmup, 3)):
        step_resident()
    with ClockSampler(gpu_uuid(dev), active=(rank == 0)) as clk:
        ms, launches = timed(step_resident, args.steps)
    clocks = clk.summary()
    ms_per_step = ms / args.steps
    value = faces_total / (ms_per_step / 1e3)

    if _lib.async_error():
        raise SystemExit(f"a tensor-core kernel gave up waiting (code {_lib.async_error()}): the timed steps are invalid")
    # checksum of the all-reduced filter gradients of the last step: the batch is seeded per mesh, so
    # the values agree across GPU counts up to fp32 re-association of the sum over meshes
    gsum = sum(float(p.grad.double().sum().item()) for p in params)
    gl2 = float(sum(float((p.grad.double() ** 2).sum().item()) for p in params) ** 0.5)
    checksum = dict(sum=gsum, l2=gl2, note="sum and L2 norm over the three all-reduced filter gradients "
                    "(fp64 accumulation of the fp32 results)")

    # per-kernel durations of the same step, measured live with CUDA events on the launch stream
    prof_steps = min(args.steps, 3)
    _lib.prof_reset()
    _lib.prof_enable(True)
    for _ in range(prof_steps):
        step_resident()
    torch.cuda.synchronize()
    _lib.prof_enable(False)
    records = _lib.prof_read(64)
    _lib.prof_reset()
    dims = dict(Nv=h["Nv"], Nf=h["Nf"], NiK=h["NiK"], f2f_samples=h["Nf"], cin=cfg["cin"], cout=cfg["cout"], K=K,
                config=args.config, precision=args.precision)
    roof, table = roofline_from_profile(records, prof_steps, dims)

    # per-batch preparation, reported apart (amortised over the convolutions of a level): nfCount,
    # triangle geometry, the two SH bases and the vertex CSR build with its index validation
    prep_ms = []
    for _ in range(3):
        topology.clear_cache()
        torch.cuda.synchronize()
        p0, p1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        p0.record()
        _, _, bsh = prepare()
        topology.vertex_csr(d["face"], vt_map, h["Nv"], h["Nv"])
        topology.face_means(bsh, d["cum"])
        p1.record()
        torch.cuda.synchronize()
        prep_ms.append(p0.elapsed_time(p1))
    prep = dict(ms=sorted(prep_ms)[1], includes="count_vertex_adjface, triangle geometry, SH_L(normals), "
                "SH_L(texture barycentrics) and its per-face means, vertex CSR build + index validation; not part of `value` "
                "(cached per topology), part of `e2e`")

    # the single-MMA operand variants of the facet2facet contraction, same step, same inputs
    variants = None
    if args.precision == "fp32" and not args.no_variants:
        variants = {}
        notes = {"tf32": "facet2facet operands rounded to tf32 (1 MMA per product), fp32 accumulation; relative error gate 2e-3",
                 "bf16": "facet2facet operands rounded to bf16 (1 MMA per product), fp32 accumulation; relative error gate 2e-2"}
        vsteps = max(2, min(args.steps, 5))
        for vname in ("tf32", "bf16"):
            conv3d.set_f2f_precision(vname)
            for _ in range(2):
                step_resident()
            vms, _ = timed(step_resident, vsteps)
            variants[vname] = dict(value=faces_total / (vms / vsteps / 1e3), unit=UNIT, ms_per_step=vms / vsteps,
                                   note=notes[vname])
        conv3d.set_f2f_precision(args.precision)
        block_fn[0] = conv_block_expanded
        for _ in range(2):
            step_resident()
        vms, _ = timed(step_resident, vsteps)
        block_fn[0] = conv_block
        variants["block_as_written"] = dict(
            value=faces_total / (vms / vsteps / 1e3), unit=UNIT, ms_per_step=vms / vsteps,
            note="the face rows written once per sample (expand_rows) and the general facet2facet over every sample, "
                 "instead of per-face mean weights and one sample per face; same result")

    # accuracy of the timed precision mode on this batch's first mesh (outside every timed region):
    # the whole block in the timed mode against the library's fp32 FFMA path on identical inputs
    parity = None
    if rank == 0 and not args.no_parity:
        nv0, mf0 = h["nv"][0], h["mf"][0]
        nik0 = int(h["cum"][mf0 - 1])
        sl = dict(x=d["x"][:nv0].detach(), face=d["face"][:mf0], cum=d["cum"][:mf0], bary=bary_sh[:nik0],
                  coeff=coeff[:mf0], nfc=nfc[:nv0], vt=vt_map[:nv0], G=G[:nv0])

        def one_mesh(mode, block):
            conv3d.set_f2f_precision(mode)
            x0 = sl["x"].clone().requires_grad_()
            ws = [p.detach().clone().requires_grad_() for p in params]
            o = block(x0, ws[0], ws[1], ws[2], sl["face"], sl["cum"], sl["bary"], sl["coeff"], sl["nfc"], sl["vt"],
                      sh_eye)
            o.backward(sl["G"])
            return [o.detach(), x0.grad] + [w.grad for w in ws]

        got, want = one_mesh(args.precision, conv_block), one_mesh("fp32_ffma", conv_block_expanded)
        conv3d.set_f2f_precision(args.precision)
        names = ["out", "grad_x", "grad_Wv", "grad_Wf", "grad_Wo"]
        parity = {"mode": args.precision,
                  "against": "the block as written (face rows expanded per sample, general facet2facet) on the fp32_ffma "
                             "path of the same library, same inputs",
                  "sample": f"first mesh of the batch ({mf0} faces)", "gate_max_rel": GATES[args.precision]}
        for n, a, b in zip(names, got, want):
            diff = (a.double() - b.double())
            parity[n] = dict(max_rel=float(diff.abs().max() / b.double().abs().max()),
                             rms_rel=float((diff ** 2).mean().sqrt() / (b.double() ** 2).mean().sqrt()))
        # the filter gradients sum over every face of the batch: check them on the rank's whole batch too
        # (a sum that long is where an accumulator that truncates would show)

        def whole_batch(mode, block):
            conv3d.set_f2f_precision(mode)
            ws = [p.detach().clone().requires_grad_() for p in params]
            x0 = d["x"].detach().clone().requires_grad_()
            o = block(x0, ws[0], ws[1], ws[2], d["face"], d["cum"], bary_sh, coeff, nfc, vt_map, sh_eye)
            o.backward(G)
            return [w.grad for w in ws]

        got_b, want_b = whole_batch(args.precision, conv_block), whole_batch("fp32_ffma", conv_block_expanded)
        conv3d.set_f2f_precision(args.precision)
        parity["whole_batch"] = {"sample": f"the rank's whole batch ({h['Nf']} faces)"}
        for n, a, b in zip(names[2:], got_b, want_b):
            diff = (a.double() - b.double())
            parity["whole_batch"][n] = dict(
                max_rel=float(diff.abs().max() / b.double().abs().max()),
                rms_rel=float((diff ** 2).mean().sqrt() / (b.double() ** 2).mean().sqrt()),
                scale=float((a.double() * b.double()).sum() / (b.double() ** 2).sum()) - 1.0)
        del got_b, want_b
        parity["ok"] = (all(parity[n]["max_rel"] <= GATES[args.precision] for n in names) and
                        all(parity["whole_batch"][n]["max_rel"] <= GATES[args.precision] for n in names[2:]))

    # launch-bound batches: the same resident step captured once into a CUDA graph and replayed
    graph = None
    if world == 1 and (args.graph or ms_per_step < 3.0):
        try:
            from picassoplus_b200.graph import GraphedStep
            for p in params:
                p.grad = None
            xd.grad = None

            def step_graph():
                # gradients are written in place (no `p.grad = None`): static addresses for the replay
                for p in params:
                    if p.grad is not None:
                        p.grad.zero_()
                if xd.grad is not None:
                    xd.grad.zero_()
                o = conv_block(xd, params[0], params[1], params[2], d["face"], d["cum"], bary_sh, coeff, nfc, vt_map,
                               sh_eye)
                o.backward(G)

            gstep = GraphedStep(step_graph)
            gsteps = max(args.steps, 10)
            for _ in range(3):
                gstep()
            gms, _ = timed(gstep, gsteps)
            graph = dict(value=faces_total / (gms / gsteps / 1e3), unit=UNIT, ms_per_step=gms / gsteps, steps=gsteps,
                         note="forward + backward of the resident step replayed from one CUDA graph")
        except Exception as exc:                     # a capture failure must not lose the measurement
            graph = dict(value=None, error=f"{type(exc).__name__}: {exc}"[:200])

    e2e = None
    if not args.no_e2e:
        for _ in range(max(args.warmup, 3)):
            step_e2e()
        e_steps = max(2, min(args.steps, 5))
        ems, _ = timed(step_e2e, e_steps)
        e2e = dict(value=faces_total / (ems / e_steps / 1e3), unit=UNIT, ms_per_step=ems / e_steps,
                   h2d_bytes_per_step=int(h2d_bytes), d2h_bytes_per_step=4, steps=e_steps,
                   mesh_groups=len(feed.batches),
                   includes="H2D of vertices/faces/features/texture samples (per mesh group, double-buffered: "
                            "the copy of one group overlaps the compute of the previous one, across steps too), nfCount + normals "
                            "+ SH + CSR rebuild, fwd+bwd, loss D2H")

    cpu = None
    if rank == 0 and world == 1 and not args.no_cpu_baseline:
        cpu = cpu_baseline(cfg, args.cpu_seconds)

    if world > 1:
        dist.barrier()
    if rank == 0:
        line = {
            "metric": METRIC, "value": value, "unit": UNIT, "n_gpus": world, "steps": args.steps,
            "warmup": max(args.warmup, 3), "ms_per_step": ms_per_step, "higher_is_better": True,
            "scaling": "strong", "vs_baseline": None, "dtype": "f32", "data": "synthetic",
            "config": {"workload": workload_name(cfg, total_meshes), "name": args.config},
            "workload_detail": {"faces": int(faces_total), "vertices": int(nf_all[1].item()),
                                "texture_samples": int(nf_all[2].item()), "f2f_precision": args.precision,
                                "parallelism": f"mesh-dp{world}", "meshes_per_gpu": count,
                                "cpus_bound_near_gpu": near_cpus,
                                "block": "V2F -> F2F -> F2V with the repetition of the face rows folded into facet2facet "
                                         "(per-face mean sample weights, one sample per face); variants.block_as_written "
                                         "times the row expansion + general facet2facet",
                                "l2_policy": "inputs larger than L2 (no flush)" if h["Nf"] * cfg["cin"] * 4 > 256e6
                                else "inputs smaller than L2, no flush"},
            "parity": parity, "grad_checksum": checksum,
            "roofline": roof, "cpu_baseline": cpu, "e2e": e2e, "graph_replay": graph, "prepare": prep, "gpu_launches": int(launches),
            "clocks": clocks, "variants": variants, "kernels": table[:12],
            "allreduce_bytes": allreduce.nbytes if world > 1 else 0,
        }
        print(json.dumps(line))
    if world > 1:
        dist.destroy_process_group()


# --------------------------------------------------------------- encoder stack (config c4)
C4 = dict(n=700, batch=2, levels=4, channels=[64, 128, 256, 384], L=3, seed=3)


def c4_hierarchy(cfg):
    """The batch's mesh hierarchy on the host: per level the concatenated (vertex, face), per
    transition the concatenated cluster encoding (ids re-based to the batch)."""
    per_mesh = [synth.heightfield_hierarchy(cfg["n"], cfg["seed"] * 1000 + i, cfg["levels"]) for i in range(cfg["batch"])]
    levels, trans = [], []
    for lvl in range(cfg["levels"]):
        levels.append(synth.concat_meshes([pm[0][lvl] for pm in per_mesh]))
    for t in range(cfg["levels"] - 1):
        reps, maps, voff, coff = [], [], 0, 0
        for pm in per_mesh:
            r, m = pm[1][t]
            reps.append(np.where(r < 0, r - voff, r).astype(np.int32))       # -(representative + offset)
            maps.append(np.where(m >= 0, m + coff, m).astype(np.int32))
            voff += r.shape[0]
            coff += int(m.max()) + 1
        trans.append((np.concatenate(reps), np.concatenate(maps)))
    return levels, trans


def run_c4(args):
    """BASELINE configuration 4: encoder stack over four mesh levels, forward + backward.  Per level
    one V2VConv3d module (vertex2facet -> pointwise -> facet2vertex -> pointwise, ReLU, batch norm in
    training mode) followed by a max pool to the next level; channels 64 -> 128 -> 256 -> 384, L = 3.
    The levels come from the library's quadric-error decimation (stride 4 per level; --hierarchy grid
    halves the height-field grid instead: face ratios 1 / 0.25 / 0.062 / 0.015 either way); they are
    built once, timed on their own (hierarchy_build_ms), and held fixed over the steps."""
    from picassoplus_b200 import _lib, topology
    from picassoplus_b200.mesh import layers as mesh_layers
    from picassoplus_b200.mesh.layers import Pool3d, V2VConv3d
    from picassoplus_b200.mesh.pi_modules import conv3d, fused
    if not torch.cuda.is_available():
        raise SystemExit("bench.py needs a CUDA device (there is no CPU fallback for --impl ours)")
    assert int(os.environ.get("WORLD_SIZE", "1")) == 1, "config c4 is a single-GPU measurement"
    mesh_layers.set_fusion(not args.no_fusion)
    fused.set_pointwise_precision("bf16" if args.precision == "bf16" else "fp32")
    dev = torch.device("cuda", 0)
    torch.cuda.set_device(dev)
    cfg = C4
    conv3d.set_f2f_precision(args.precision)
    hierarchy_ms = None
    if args.hierarchy == "grid":
        levels, trans = c4_hierarchy(cfg)
    else:
        # levels by decimation, as the reference's networks build them per batch (picasso/mesh/utils.py:32-58,
        # networks/scene_seg.py:131): stride 4 per level, the reference's hyper-parameters (scene_seg.py:23)
        from picassoplus_b200.mesh.utils import MeshHierarchy
        mb0 = synth.concat_meshes([synth.heightfield(cfg["n"], cfg["seed"] * 1000 + i) for i in range(cfg["batch"])])
        t_in = [torch.from_numpy(a).to(dev) for a in (mb0.vertex, mb0.face, mb0.nv.astype(np.int32), mb0.mf.astype(np.int32))]
        build = MeshHierarchy([4] * (cfg["levels"] - 1), [16] * (cfg["levels"] - 1), True, 1.0)
        build(*t_in)
        torch.cuda.synchronize()
        t0 = time.perf_counter()
        hier = build(*t_in)
        torch.cuda.synchronize()
        hierarchy_ms = (time.perf_counter() - t0) * 1e3
        levels = [synth.MeshBatch(h[0][:, :3].cpu().numpy(), h[1].cpu().numpy(), h[3].cpu().numpy(), h[4].cpu().numpy())
                  for h in hier]
        trans = [(h[5].cpu().numpy(), h[6].cpu().numpy()) for h in hier[1:]]
    L, ch = cfg["L"], cfg["channels"]
    rng = np.random.default_rng(cfg["seed"] + 77)
    v0 = levels[0].vertex
    xyz = (v0 - v0.min(0)) / (v0.max(0) - v0.min(0) + 1e-9)
    feats6 = np.concatenate([xyz, rng.uniform(0, 1, size=xyz.shape)], axis=1).astype(np.float32)
    x0 = torch.from_numpy(feats6 @ synth.xavier_normal((6, ch[0]), rng)).to(dev).requires_grad_()
    torch.manual_seed(cfg["seed"])
    convs = [V2VConv3d(ch[i], [ch[i + 1], ch[i + 1]], L, [1, 1]).to(dev).train() for i in range(3)]
    pool = Pool3d("max")
    lv = []
    for mb in levels:
        vertex, face = torch.from_numpy(mb.vertex).to(dev), torch.from_numpy(mb.face).to(dev)
        vt = torch.arange(mb.num_vertices, dtype=torch.int32, device=dev)
        prep = topology.prepare_level(vertex, face, vt, mb.num_vertices, L, want_geometry=False)
        lv.append(dict(vertex=vertex, face=face, vt=vt, nfc=prep["nf_count"], coeff=prep["coeff"]))
    tr = [(torch.from_numpy(r).to(dev), torch.from_numpy(m).to(dev)) for r, m in trans]
    G = torch.randn(levels[3].num_vertices, ch[3], device=dev, generator=torch.Generator(device=dev).manual_seed(9))
    params = [p for c in convs for p in c.parameters()]

    def step():
        for p in params:
            p.grad = None
        x0.grad = None
        x = x0
        for i in range(3):
            x = convs[i](x, lv[i]["face"], lv[i]["nfc"], lv[i]["vt"], lv[i]["coeff"])
            x = pool(x, tr[i][0], tr[i][1], lv[i + 1]["vertex"])
        x.backward(G)

    for _ in range(max(args.warmup, 3)):
        step()
    torch.cuda.synchronize()
    with ClockSampler(gpu_uuid(dev)) as clk:
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        n0 = _lib.launch_count()
        e0.record()
        for _ in range(args.steps):
            step()
        e1.record()
        torch.cuda.synchronize()
    ms = e0.elapsed_time(e1) / args.steps
    launches = _lib.launch_count() - n0
    _lib.prof_reset()
    _lib.prof_enable(True)
    step()
    torch.cuda.synchronize()
    _lib.prof_enable(False)
    records = _lib.prof_read(64)
    _lib.prof_reset()
    lib_ms = sum(r[2] for r in records)
    faces = levels[0].num_faces
    # algorithmic bytes of the library's operators per level (the formulas of kernel_models), summed
    peaks = load_peaks()
    alg = 0
    for i in range(3):
        Nv, Nf, Ci, Co, K = levels[i].num_vertices, levels[i].num_faces, ch[i], ch[i + 1], (L + 1) ** 2
        alg += 12 * Ci * Nv + 8 * Ci * Nf + 24 * Nf                                         # V2F fwd+bwd
        alg += 12 * Co * Nf + 8 * K * Nf + 24 * Nf + 8 * Co * Nv + 16 * Nv                  # F2V fwd+bwd
        alg += 4 * Co * (2 * Nv + 3 * levels[i + 1].num_vertices)                           # max pool fwd+bwd
        if not args.no_fusion:
            # backward of the two pointwise stages (rows x C -> Cout): masked product reads gradient + activation,
            # writes the masked gradient and the operator-output gradient; the contraction over rows reads both
            for rows, C, Cout in ((Nf, Ci, Co), (Nv, Co, Co)):
                alg += 4 * rows * (3 * Cout + C) + 4 * rows * (C + Cout)
    line = {
        "metric": METRIC, "value": faces / (ms / 1e3), "unit": UNIT, "n_gpus": 1, "steps": args.steps,
        "warmup": max(args.warmup, 3), "ms_per_step": ms, "higher_is_better": True, "scaling": "strong",
        "vs_baseline": None, "dtype": "f32", "data": "synthetic",
        "config": {"workload": f"encoder stack, {cfg['batch']} heightfield meshes {cfg['n']}x{cfg['n']} over 4 levels "
                               f"(faces {[m.num_faces for m in levels]}), channels 64->128->256->384, L=3", "name": "c4"},
        "workload_detail": {"faces_level0": faces, "vertices_per_level": [m.num_vertices for m in levels],
                            "hierarchy": ("grid halving of the height fields" if args.hierarchy == "grid" else
                                          "quadric-error decimation by the library, stride 4 per level (pb200_mesh_simplify)"),
                            "hierarchy_build_ms": hierarchy_ms,
                            "pointwise_stage": ("torch.matmul + bias + ReLU (cuBLAS / torch kernels), BatchNorm1d in torch"
                                                if args.no_fusion else
                                                "fused with the operator in one tcgen05 kernel (forward; "
                                                f"{'bf16' if args.precision == 'bf16' else 'bf16 hi+lo'} operands), "
                                                "BatchNorm1d in torch; backward = recompute of the operator output + masked product and "
                                                "contraction over rows on the tensor cores + operator backward")},
        "roofline": {"bound": "hbm", "achieved": alg / (lib_ms / 1e3) / 1e9, "peak": peaks["hbm_gbs"], "unit": "GB/s",
                     "frac": alg / (lib_ms / 1e3) / 1e9 / peaks["hbm_gbs"], "traffic": None,
                     "note": "all library kernels of one step together: algorithmic bytes of V2F, F2V, max pool and (fused "
                             "mode) the two backward products of every pointwise stage over the three conv levels / "
                             "their summed duration", "peak_source": peaks["source"]},
        "library_kernel_ms_per_step": lib_ms, "other_ms_per_step": ms - lib_ms,
        "gpu_launches": int(launches), "clocks": clk.summary(),
        "kernels": [dict(kernel=n, launches_per_step=c, ms_per_step=t) for n, c, t in records[:14]],
    }
    print(json.dumps(line))


# ------------------------------------------------------------------------ decimation
DECIMATE = dict(n=360, batch=32, stride=4, seed=5, use_area=True, wgt_bnd=1.0)
DECIMATE_METRIC, DECIMATE_UNIT = "mesh_decimation_input_faces_per_sec", "faces/s"


def decimate_batch(cfg, meshes):
    mb = synth.concat_meshes([synth.heightfield(cfg["n"], cfg["seed"] * 1000 + i) for i in range(meshes)])
    return mb, (mb.nv // cfg["stride"]).astype(np.int32)


def decimate_workload(cfg, meshes, mb):
    return (f"decimation of {meshes} heightfield meshes {cfg['n']}x{cfg['n']} ({mb.num_vertices} vertices, {mb.num_faces} "
            f"faces) to 1/{cfg['stride']} of their vertices: triangle geometry + all passes of the quadric-error "
            "clustering + cluster merges")


def run_decimate(args):
    """One step = the whole decimation of the batch to a quarter of its vertices (geometry, every pass of
    pb200_mesh_simplify, compaction, cluster merges), as the reference's networks run it once per batch and
    level (picasso/mesh/utils.py:42-58).  The workload (4.1 M vertices) is larger than L2."""
    from picassoplus_b200 import _lib
    from picassoplus_b200.mesh.pi_modules import decimate as dm
    if not torch.cuda.is_available():
        raise SystemExit("bench.py needs a CUDA device (there is no CPU fallback for --impl ours)")
    assert int(os.environ.get("WORLD_SIZE", "1")) == 1, "config decimate is a single-GPU measurement"
    dev = torch.device("cuda", 0)
    torch.cuda.set_device(dev)
    cfg = DECIMATE
    meshes = args.meshes or cfg["batch"]
    mb, target = decimate_batch(cfg, meshes)
    host = [torch.from_numpy(a).pin_memory() for a in (mb.vertex, mb.face, mb.nv.astype(np.int32), mb.mf.astype(np.int32), target)]
    resident = [t.to(dev) for t in host]

    def step(inputs):
        vertex, face, nv, mf, nv_out = inputs
        geo = dm.compute_triangle_geometry_(vertex, face)
        return dm.mesh_decimation_(vertex, face, geo, nv, mf, nv_out, cfg["use_area"], cfg["wgt_bnd"])

    def step_e2e():
        res = step([t.to(dev, non_blocking=True) for t in host])
        return res[3].cpu(), res[4].cpu()

    warm = max(args.warmup, 3)
    for _ in range(warm):
        res = step(resident)
    torch.cuda.synchronize()
    with ClockSampler(gpu_uuid(dev)) as clk:
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        n0 = _lib.launch_count()
        e0.record()
        for _ in range(args.steps):
            res = step(resident)
        e1.record()
        torch.cuda.synchronize()
        launches = _lib.launch_count() - n0
    ms = e0.elapsed_time(e1) / args.steps
    for _ in range(2):
        step_e2e()
    torch.cuda.synchronize()
    t0 = time.perf_counter()
    for _ in range(args.steps):
        nv_res, mf_res = step_e2e()
    torch.cuda.synchronize()
    ms_e2e = (time.perf_counter() - t0) * 1e3 / args.steps
    # the dominant kernel of the first (largest) pass: the radix-sort scatter
    vertex, face, nv, mf, nv_out = resident
    geo = dm.compute_triangle_geometry_(vertex, face)
    nv_cum, mf_cum = torch.cumsum(nv, 0, dtype=torch.int32), torch.cumsum(mf, 0, dtype=torch.int32)
    _lib.prof_reset()
    _lib.prof_enable(True)
    _, info, _ = dm.simplify(vertex, face, geo, nv_cum, mf_cum, (nv - nv_out).to(torch.int32), cfg["use_area"], cfg["wgt_bnd"],
                             return_info=True)
    torch.cuda.synchronize()
    _lib.prof_enable(False)
    records = _lib.prof_read(64)
    _lib.prof_reset()
    peaks = load_peaks()
    Nv, Nf, nu = mb.num_vertices, mb.num_faces, int(info[0])
    edge_passes = -(-2 * max(Nv, 1).bit_length() // 8)
    cost_passes = -(-(32 + meshes.bit_length()) // 8)
    scatter_bytes = 24 * (edge_passes * 3 * Nf + cost_passes * nu)            # key + payload, read and written
    scatter = [r for r in records if r[0] == "dec_sort_scatter"]
    sc_ms = scatter[0][2] if scatter else float("nan")
    pass_ms = sum(r[2] for r in records)
    line = {
        "metric": DECIMATE_METRIC, "value": Nf / (ms / 1e3), "unit": DECIMATE_UNIT, "n_gpus": 1, "steps": args.steps,
        "warmup": warm, "ms_per_step": ms, "higher_is_better": True, "scaling": "strong", "vs_baseline": None,
        "dtype": "f32", "data": "synthetic",
        "config": {"workload": decimate_workload(cfg, meshes, mb), "name": "decimate", "l2": "inputs larger than L2"},
        "e2e": dict(value=Nf / (ms_e2e / 1e3), unit=DECIMATE_UNIT, ms_per_step=ms_e2e,
                    h2d_bytes_per_step=int(sum(t.numel() * t.element_size() for t in host)),
                    d2h_bytes_per_step=int(nv_res.numel() * 4 + mf_res.numel() * 4)),
        "roofline": {"bound": "hbm", "achieved": scatter_bytes / (sc_ms / 1e3) / 1e9, "peak": peaks["hbm_gbs"], "unit": "GB/s",
                     "frac": scatter_bytes / (sc_ms / 1e3) / 1e9 / peaks["hbm_gbs"], "traffic": None,
                     "kernel": "dec_sort_scatter", "launches": scatter[0][1] if scatter else 0,
                     "note": "first pass only: (key 8 B + payload 4 B) read and written per element and radix pass, "
                             f"{edge_passes} passes over {3 * Nf} edge instances + {cost_passes} over {nu} candidates",
                     "peak_source": peaks["source"]},
        "first_pass": {"kernel_ms": pass_ms, "distinct_edges": nu, "grid_rounds": int(info[1]), "tail_edges": int(info[2])},
        "result": {"vertices_out": int(res[3].sum()), "faces_out": int(res[4].sum())},
        "gpu_launches": int(launches), "clocks": clk.summary(),
        "kernels": [dict(kernel=n, launches=c, ms=t, share=t / pass_ms) for n, c, t in records[:12]],
    }
    if not args.no_cpu_baseline:
        line["cpu_baseline"] = decimate_cpu_baseline(cfg, min(meshes, 8))
    print(json.dumps(line))


def decimate_cpu_baseline(cfg, meshes):
    """The sequential C restatement of the same loop on one host core, on `meshes` meshes of the workload."""
    from oracle import c_oracle
    mb, target = decimate_batch(cfg, meshes)
    vertex, face, nv, mf = mb.vertex, mb.face, mb.nv.astype(np.int32), mb.mf.astype(np.int32)
    t0 = time.perf_counter()
    geo = c_oracle.triangle_geometry(vertex, face)
    remove = nv - target
    rep, mp = np.zeros(vertex.shape[0], np.int32), np.arange(vertex.shape[0], dtype=np.int32)
    while (remove > 0).any():
        o = c_oracle.mesh_simplify(vertex, face, geo, np.cumsum(nv).astype(np.int32), np.cumsum(mf).astype(np.int32),
                                   remove.astype(np.int32), cfg["use_area"], cfg["wgt_bnd"])
        if not ((nv - o["nvOut"]) > 0).any():
            break
        face, vertex = o["faceOut"][~o["isDegenerate"]], o["vertexOut"][o["vtMap"] >= 0]
        geo = c_oracle.triangle_geometry(vertex[:, :3].copy(), face)
        remove = remove - (nv - o["nvOut"])
        rep, mp = c_oracle.combine_clusters(rep, mp, o["vtReplace"], o["vtMap"])
        nv, mf = o["nvOut"], o["mfOut"]
    dt = time.perf_counter() - t0
    return dict(value=mb.num_faces / dt, unit=DECIMATE_UNIT, cores=1, kind="port", seconds=dt,
                sample=f"{meshes} of the workload's meshes ({mb.num_faces} faces), the whole loop, sequential C restatement")


def run_reference_decimate(args):
    """Reference arm of config decimate.  The reference's decimation is a CUDA program with a host loop; where its
    sources were compiled (oracle/_ref) and a GPU is present it is run unmodified on a sample its per-vertex host
    stack array allows (decimate_gpu.cu:663), otherwise the sequential C restatement is timed on the host."""
    if int(os.environ.get("RANK", "0")) != 0:
        return
    cfg = DECIMATE
    from oracle import ref_cuda
    if ref_cuda.available():
        from oracle import c_oracle
        sub = dict(cfg, n=200)
        mb, target = decimate_batch(sub, 4)
        dev = torch.device("cuda", 0)
        geo = torch.from_numpy(c_oracle.triangle_geometry(mb.vertex, mb.face)).to(dev)
        vertex, face = torch.from_numpy(mb.vertex).to(dev), torch.from_numpy(mb.face).to(dev)
        nv_cum = torch.from_numpy(np.cumsum(mb.nv).astype(np.int32)).to(dev)
        mf_cum = torch.from_numpy(np.cumsum(mb.mf).astype(np.int32)).to(dev)
        remove = torch.from_numpy((mb.nv - target).astype(np.int32)).to(dev)

        def step():
            ref_cuda.mesh_simplify(vertex, face, geo, nv_cum, mf_cum, remove, cfg["use_area"], cfg["wgt_bnd"])
        kind, cores = "reference", 1
        sample = (f"first pass only on 4 heightfield meshes 200x200 ({mb.num_faces} faces): the reference's own CUDA kernels "
                  "and host loop, unmodified, on this GPU (its per-vertex host stack array bounds the size)")
        nf = mb.num_faces
    else:
        def step():
            step.out = decimate_cpu_baseline(cfg, 4)
        kind, cores, nf = "port", 1, None
        sample = "4 of the workload's meshes, the whole loop, sequential C restatement on one host core"
    for _ in range(args.warmup):
        step()
    t0 = time.perf_counter()
    for _ in range(args.steps):
        step()
    if kind == "reference":
        torch.cuda.synchronize()
    dt = (time.perf_counter() - t0) / args.steps
    if nf is None:
        nf = decimate_batch(cfg, 4)[0].num_faces
    value = nf / dt
    print(json.dumps({
        "impl": "reference", "metric": DECIMATE_METRIC, "value": value, "unit": DECIMATE_UNIT, "n_gpus": args.gpus,
        "steps": args.steps, "warmup": args.warmup, "ms_per_step": dt * 1e3, "higher_is_better": True, "scaling": "strong",
        "vs_baseline": None, "dtype": "f32", "data": "synthetic", "config": {"name": "decimate", "workload": sample},
        "cpu_baseline": dict(value=value, unit=DECIMATE_UNIT, cores=cores, kind=kind, sample=sample),
        "e2e": dict(value=value, unit=DECIMATE_UNIT, h2d_bytes_per_step=0, d2h_bytes_per_step=0),
    }))


# ------------------------------------------------------------------ auxiliary kernels
AUX = dict(n=700, batch=2, C=128, L=3, seed=3, pc_points=1 << 20, pc_out=1 << 18, pc_knn=16, pc_bins=17, pc_fuzzy=3, pc_C=64)
AUX_METRIC, AUX_UNIT = "aux_kernels_hbm_fraction_geomean", "fraction of measured copy bandwidth"


def aux_pcloud_inputs(cfg, dev):
    """Neighbour pairs as a radius search emits them (grouped by output point, up to knn each), fuzzy bins."""
    rng = np.random.default_rng(cfg["seed"] + 9)
    Np, Mp, knn, F, T = cfg["pc_points"], cfg["pc_out"], cfg["pc_knn"], cfg["pc_bins"], cfg["pc_fuzzy"]
    counts = rng.integers(knn // 2, knn + 1, size=Mp)
    out_idx = np.repeat(np.arange(Mp), counts)
    in_idx = rng.integers(0, Np, size=out_idx.shape[0])
    w = rng.random((out_idx.shape[0], T)).astype(np.float32) + 0.05
    t = lambda a: torch.from_numpy(a).to(dev)
    return dict(nn_index=t(np.stack([out_idx, in_idx], 1).astype(np.int32)), nn_count=t(counts.astype(np.int32)),
                bin_index=t(rng.integers(0, F, size=(out_idx.shape[0], T)).astype(np.int32)),
                bin_coeff=t(w / w.sum(1, keepdims=True)), npairs=int(out_idx.shape[0]))


def aux_cases(cfg, dev, impl):
    """[(name, callable, algorithmic bytes)] for one level-0 -> level-1 transition of the config-4 hierarchy
    (980 000 -> 245 000 vertices, C = 128) and a point-cloud convolution; impl = 'ours' or 'reference'."""
    from picassoplus_b200.mesh.utils import MeshHierarchy
    mb0 = synth.concat_meshes([synth.heightfield(cfg["n"], cfg["seed"] * 1000 + i) for i in range(cfg["batch"])])
    t_in = [torch.from_numpy(a).to(dev) for a in (mb0.vertex, mb0.face, mb0.nv.astype(np.int32), mb0.mf.astype(np.int32))]
    hier = MeshHierarchy([4], [16], True, 1.0)(*t_in)
    rep, vmap, vout = hier[1][5], hier[1][6], hier[1][0][:, :3].contiguous()
    nv_in, nv_out, C = rep.shape[0], vout.shape[0], cfg["C"]
    gen = torch.Generator(device=dev).manual_seed(cfg["seed"])
    x = torch.randn(nv_in, C, device=dev, generator=gen)
    xc = torch.randn(nv_out, C, device=dev, generator=gen)
    pc = aux_pcloud_inputs(cfg, dev)
    Cp, F, T, Np, Mp, P = cfg["pc_C"], cfg["pc_bins"], cfg["pc_fuzzy"], cfg["pc_points"], cfg["pc_out"], pc["npairs"]
    xp = torch.randn(Np, Cp, device=dev, generator=gen)
    gp = torch.randn(Mp, Cp, device=dev, generator=gen)
    filt = torch.randn(F, Cp, 1, device=dev, generator=gen)
    if impl == "ours":
        from picassoplus_b200.mesh.pi_modules import pool3d, unpool3d
        from picassoplus_b200.point.pi_modules import conv3d as pconv
        from picassoplus_b200 import topology
        mx, idx, clusters = pool3d.max_forward(x, rep, vmap, vout, return_clusters=True)
        L = cfg["L"]
        vt = torch.arange(nv_in, dtype=torch.int32, device=dev)
        cases = [
            ("mesh_max_pool_fwd", lambda: pool3d.max_forward(x, rep, vmap, vout), 4 * C * nv_in + 8 * C * nv_out),
            ("mesh_max_pool_bwd", lambda: pool3d.max_backward(xc, x, idx, clusters), 8 * C * nv_out + 4 * C * nv_in),
            ("mesh_max_pool_bwd (reference's signature: zero fill + scatter)", lambda: pool3d.max_backward(xc, x, idx),
             8 * C * nv_out + 4 * C * nv_in),
            ("mesh_avg_pool_fwd", lambda: pool3d.avg_forward(x, rep, vmap, vout), 4 * C * nv_in + 4 * C * nv_out),
            ("mesh_avg_pool_bwd", lambda: pool3d.avg_backward(xc, x, rep, vmap), 4 * C * nv_out + 4 * C * nv_in),
            ("mesh_unpool_fwd", lambda: unpool3d.forward(xc, rep, vmap), 4 * C * nv_out + 4 * C * nv_in),
            ("mesh_unpool_bwd", lambda: unpool3d.backward(x, xc, rep, vmap), 4 * C * nv_in + 4 * C * nv_out),
            ("pcloud_conv_fwd", lambda: pconv.fuzzySPH3D_forward(xp, filt, pc["nn_count"], pc["nn_index"], pc["bin_index"],
                                                                 pc["bin_coeff"]),
             4 * Cp * P + 4 * Cp * Mp + (8 + 8 * T) * P),
            ("pcloud_conv_bwd", lambda: pconv.fuzzySPH3D_backward(gp, xp, filt, pc["nn_count"], pc["nn_index"], pc["bin_index"],
                                                                  pc["bin_coeff"]),
             8 * Cp * P + 4 * Cp * Np + (8 + 8 * T) * P),
            ("level_prepare (geometry + normals + SH + nfCount + CSR)",
             lambda: topology.prepare_level(t_in[0], t_in[1], vt, nv_in, L, want_geometry=True),
             12 * nv_in + 12 * mb0.num_faces * 3 + (20 + 4 * (L + 1) ** 2) * mb0.num_faces + 12 * mb0.num_faces),
        ]
    else:
        from oracle import ref_cuda
        mx, idx = ref_cuda.max_pool_forward(x, rep, vmap, nv_out)
        cases = [
            ("mesh_max_pool_fwd", lambda: ref_cuda.max_pool_forward(x, rep, vmap, nv_out), 4 * C * nv_in + 8 * C * nv_out),
            ("mesh_max_pool_bwd", lambda: ref_cuda.max_pool_backward(xc, nv_in, idx), 8 * C * nv_out + 4 * C * nv_in),
            ("mesh_avg_pool_fwd", lambda: ref_cuda.avg_pool_forward(x, rep, vmap, nv_out), 4 * C * nv_in + 4 * C * nv_out),
            ("mesh_avg_pool_bwd", lambda: ref_cuda.avg_pool_backward(xc, rep, vmap), 4 * C * nv_out + 4 * C * nv_in),
            ("mesh_unpool_fwd", lambda: ref_cuda.unpool_forward(xc, rep, vmap), 4 * C * nv_out + 4 * C * nv_in),
            ("mesh_unpool_bwd", lambda: ref_cuda.unpool_backward(x, nv_out, rep, vmap), 4 * C * nv_in + 4 * C * nv_out),
            ("pcloud_conv_fwd", lambda: ref_cuda.pcloud_forward(xp, filt, pc["nn_count"], pc["nn_index"], pc["bin_index"],
                                                                pc["bin_coeff"]),
             4 * Cp * P + 4 * Cp * Mp + (8 + 8 * T) * P),
            ("pcloud_conv_bwd", lambda: ref_cuda.pcloud_backward(gp, xp, filt, pc["nn_count"], pc["nn_index"], pc["bin_index"],
                                                                 pc["bin_coeff"]),
             8 * Cp * P + 4 * Cp * Np + (8 + 8 * T) * P),
        ]
    what = (f"one level transition of the config-4 hierarchy ({nv_in} -> {nv_out} vertices by the library's decimation, "
            f"C = {C}) and a fuzzy point-cloud convolution ({Np} -> {Mp} points, {P} pairs, {F} bins x {T}, C = {Cp})")
    return cases, what


def run_aux(args):
    """Auxiliary kernels around the convolutions (mesh pool / unpool, point-cloud convolution, per-level
    preparation): each timed alone with CUDA events over `steps` calls (inputs larger than L2), reported with
    its algorithmic bytes against the measured copy bandwidth.  --impl reference times the reference's own
    CUDA kernels of the same operators (oracle/_ref) on the same inputs."""
    if int(os.environ.get("RANK", "0")) != 0:
        return
    if not torch.cuda.is_available():
        raise SystemExit("bench.py --config aux needs a CUDA device")
    dev = torch.device("cuda", 0)
    torch.cuda.set_device(dev)
    impl = args.impl
    if impl == "reference":
        from oracle import ref_cuda
        if not ref_cuda.available():
            print(json.dumps({"impl": "reference", "unavailable": "the reference's CUDA sources were not compiled (oracle/_ref missing)"}))
            return
    cases, what = aux_cases(AUX, dev, impl)
    peaks = load_peaks()
    rows = []
    warm = max(args.warmup, 3)
    with ClockSampler(gpu_uuid(dev)) as clk:
        for name, fn, nbytes in cases:
            for _ in range(warm):
                fn()
            torch.cuda.synchronize()
            e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            e0.record()
            for _ in range(args.steps):
                fn()
            e1.record()
            torch.cuda.synchronize()
            ms = e0.elapsed_time(e1) / args.steps
            rows.append(dict(kernel=name, ms=ms, algorithmic_bytes=int(nbytes), gbs=nbytes / (ms / 1e3) / 1e9,
                             hbm_frac=nbytes / (ms / 1e3) / 1e9 / peaks["hbm_gbs"]))
    geo = float(np.exp(np.mean([np.log(r["hbm_frac"]) for r in rows])))
    total_ms = sum(r["ms"] for r in rows)
    line = {"metric": AUX_METRIC, "value": geo, "unit": AUX_UNIT, "n_gpus": 1, "steps": args.steps, "warmup": warm,
            "ms_per_step": total_ms, "higher_is_better": True, "scaling": "strong", "vs_baseline": None, "dtype": "f32",
            "data": "synthetic", "config": {"name": "aux", "workload": what, "l2": "inputs larger than L2"},
            "roofline": {"bound": "hbm", "achieved": geo * peaks["hbm_gbs"], "peak": peaks["hbm_gbs"], "unit": "GB/s",
                         "frac": geo, "traffic": None, "note": "geometric mean over the kernels; per-call time includes "
                         "the host side of the call (allocation of the outputs, cached cluster / pair groupings)",
                         "peak_source": peaks["source"]},
            "kernels": rows, "clocks": clk.summary()}
    if impl == "reference":
        line["impl"] = "reference"
        line["cpu_baseline"] = dict(value=geo, unit=AUX_UNIT, cores=1, kind="reference",
                                    sample="the reference's own CUDA kernels of the same operators on the same inputs and GPU")
        line["e2e"] = dict(value=geo, unit=AUX_UNIT, h2d_bytes_per_step=0, d2h_bytes_per_step=0)
    print(json.dumps(line))


# ------------------------------------------------------------------- CPU oracle timing
def _oracle_step_fn(cfg, n_or_level, seed_shift=0):
    """One mesh of the configuration's kind (heightfield n x n or icosphere level) and a
    closure that runs fwd+bwd of the block with the CPU oracle."""
    from oracle import mesh_oracle as mo
    c = dict(cfg)
    c["batch"] = 1
    if c["kind"] == "heightfield":
        c["n"] = n_or_level
    else:
        c["level"] = n_or_level
    h = host_inputs(c, 0, 1, seed_shift)
    L = h["L"]
    Wv, Wf, Wo = make_params(cfg)
    vt = torch.arange(h["Nv"], dtype=torch.int32)
    nfc = mo.count_vertex_adjface(h["face"], vt, h["Nv"])
    geo = mo.triangle_geometry(h["vertex"], h["face"])
    coeff = mo.sph_harm_coeff(L, geo[:, :3])
    bary_sh = mo.sph_harm_coeff(L, h["bary_xyz"])
    sh_eye = mo.sph_harm_coeff(L, torch.eye(3))
    G = torch.randn(h["Nv"], cfg["cout"], generator=torch.Generator().manual_seed(1))
    params = [w.clone().requires_grad_() for w in (Wv, Wf, Wo)]
    x = h["x"].clone().requires_grad_()

    def step():
        for p in params:
            p.grad = None
        x.grad = None
        o = mo.conv_block(x, params[0], params[1], params[2], h["face"], h["counts"], h["cum"], bary_sh, coeff, nfc,
                          vt, sh_eye)
        o.backward(G)

    return step, h["Nf"]


def _calibrated_sample(cfg, target_seconds):
    """Pick the sample mesh so that one CPU step takes about `target_seconds` (at most one
    full mesh of the configuration)."""
    if cfg["kind"] == "heightfield":
        small, full = 48, cfg["n"]
    else:
        small, full = 1, cfg["level"]
    step, nf = _oracle_step_fn(cfg, small)
    step()
    t0 = time.perf_counter()
    step()
    per_face = (time.perf_counter() - t0) / nf
    if cfg["kind"] == "heightfield":
        n = int((target_seconds / per_face / 1.8) ** 0.5) + 1
        return max(small, min(full, n))
    lvl = small
    while lvl < full and per_face * 20 * 4 ** (lvl + 1) <= target_seconds:
        lvl += 1
    return lvl


def cpu_baseline(cfg, target_seconds):
    torch.set_num_threads(os.cpu_count() or 1)
    size = _calibrated_sample(cfg, target_seconds)
    step, nf = _oracle_step_fn(cfg, size)
    t0 = time.perf_counter()
    step()
    dt = time.perf_counter() - t0
    what = f"one {size}x{size} heightfield mesh" if cfg["kind"] == "heightfield" else f"one icosphere level {size}"
    return dict(value=nf / dt, unit=UNIT, cores=torch.get_num_threads(), kind="port",
                sample=f"{what} of the workload ({nf} faces), 1 fwd+bwd step of the CPU oracle "
                       f"(PyTorch index_add_/matmul composition, fp32), {dt:.2f} s")


def run_reference(args):
    rank = int(os.environ.get("RANK", "0"))
    if rank != 0:
        return
    cfg = dict(synth.CONFIGS[args.config])
    total_meshes = args.meshes or cfg["batch"]
    torch.set_num_threads(os.cpu_count() or 1)
    n_steps = args.steps + args.warmup
    size = _calibrated_sample(cfg, min(args.cpu_seconds, 120.0 / max(n_steps, 1)))
    step, nf = _oracle_step_fn(cfg, size)
    for _ in range(args.warmup):
        step()
    t0 = time.perf_counter()
    for _ in range(args.steps):
        step()
    dt = (time.perf_counter() - t0) / args.steps
    value = nf / dt
    what = f"one {size}x{size} heightfield mesh" if cfg["kind"] == "heightfield" else f"one icosphere level {size}"
    sample = (f"{what} ({nf} faces) per step; CPU oracle = PyTorch index_add_/matmul composition of the "
              "reference formulas, fp32 (the reference's own operators are CUDA-only)")
    print(json.dumps({
        "impl": "reference", "metric": METRIC, "value": value, "unit": UNIT, "n_gpus": args.gpus,
        "steps": args.steps, "warmup": args.warmup, "ms_per_step": dt * 1e3, "higher_is_better": True,
        "scaling": "strong", "vs_baseline": None, "dtype": "f32", "data": "synthetic",
        "config": {"workload": workload_name(cfg, total_meshes), "name": args.config},
        "cpu_baseline": dict(value=value, unit=UNIT, cores=torch.get_num_threads(), kind="port", sample=sample),
        "e2e": dict(value=value, unit=UNIT, h2d_bytes_per_step=0, d2h_bytes_per_step=0),
    }))


if __name__ == "__main__":
    a = parse_args()
    if a.config == "aux":
        run_aux(a)
    elif a.impl == "reference" and a.config == "decimate":
        run_reference_decimate(a)
    elif a.impl == "reference":
        run_reference(a)
    elif a.config == "decimate":
        run_decimate(a)
    elif a.config == "c4":
        run_c4(a)
    else:
        run_ours(a)
