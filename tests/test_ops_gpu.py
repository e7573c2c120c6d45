"""Parity of the CUDA operators, called through the C ABI (via the ctypes operator API),
against the CPU oracle and, when its build is present, the reference's own CUDA kernels
on identical seeded inputs.  Gate: max|a-b|/max|b| <= 1e-4 per fp32 tensor, index outputs
bit-exact (north-star tolerances)."""
import numpy as np
import pytest
import torch

from conftest import rel_err, max_abs
from cases import conv_inputs

pytestmark = pytest.mark.gpu

TOL = 1e-4
# tensor-core operand splits against the reference's fp32 FFMA, both measured against fp64
ARB_FP32 = 64.0      # bf16 hi+lo
ARB_TF32X3 = 64.0  # tf32 hi+lo (lo is cut to tf32 by the tensor core)

CASES = [
    # topology, C, r, K, Cout
    ("ico2x3", 32, 1, 16, 64),
    ("ico2x3+drop", 32, 1, 16, 8),
    ("ico1x2", 5, 2, 9, 7),
    ("ico1x2+drop", 6, 3, 4, 3),
    ("grid17x2", 128, 1, 25, 16),
    ("grid17x2+drop", 64, 1, 25, 16),
    ("grid9x1", 12, 1, 36, 5),
    ("grid9x1", 8, 1, 7, 5),        # K without a register-resident variant
    ("grid9x1", 160, 1, 16, 4),     # more than one 128-channel chunk
    ("grid17x2+drop", 256, 1, 9, 8),   # two whole 128-channel chunks: register-blocked facet2vertex kernels
    ("tri", 4, 1, 4, 2),
    ("tet+iso", 3, 1, 1, 2),
]


def _dev(d):
    return {k: (v.cuda() if isinstance(v, torch.Tensor) else v) for k, v in d.items()}


@pytest.fixture(scope="module")
def mods():
    from picassoplus_b200.mesh.pi_modules import conv3d, decimate
    from oracle import mesh_oracle, ref_cuda
    return conv3d, decimate, mesh_oracle, ref_cuda


@pytest.mark.parametrize("kind,C,r,K,cout", CASES)
def test_adjacency_bit_exact(mods, kind, C, r, K, cout):
    conv3d, decimate, mo, ref = mods
    d = conv_inputs(kind, C, r, K, cout, seed=3)
    c = _dev(d)
    vout = torch.zeros(d["nv_out"], 3, device="cuda")
    got = decimate.count_vertex_adjface_(c["face"], c["vt_map"], vout)
    want = mo.count_vertex_adjface(d["face"], d["vt_map"], d["nv_out"])
    assert got.dtype == torch.int32 and torch.equal(got.cpu(), want)
    from picassoplus_b200.topology import build_vertex_csr
    csr = build_vertex_csr(c["face"], c["vt_map"], d["vt_map"].shape[0], d["nv_out"])
    rowptr = csr.rowptr.cpu()
    assert torch.equal(rowptr[1:] - rowptr[:-1], want)          # row lengths == nfCount, bit for bit
    ent = csr.entries.cpu()[: int(rowptr[-1])].long()
    # every row ascending, and the multiset of entries equals all kept corners
    for v in range(d["nv_out"]):
        row = ent[rowptr[v]:rowptr[v + 1]]
        assert torch.all(row[1:] > row[:-1])
        f, j = row >> 2, row & 3
        assert torch.all(d["vt_map"].long()[d["face"].long()[f, j]] == v)
    if ref.available() and "+drop" not in kind:
        assert torch.equal(ref.count_vertex_adjface(c["face"], c["vt_map"], d["nv_out"]).cpu(), want)


@pytest.mark.parametrize("kind,C,r,K,cout", CASES)
def test_vertex2facet(mods, kind, C, r, K, cout):
    conv3d, _, mo, ref = mods
    d = conv_inputs(kind, C, r, K, cout, seed=4)
    c = _dev(d)
    out = conv3d.vertex2facet_forward(c["x_v"], c["filt_v2f"], c["face"])
    want = mo.vertex2facet_forward(d["x_v"], d["filt_v2f"], d["face"])
    assert out.shape == want.shape and rel_err(out, want) <= TOL
    gin, gf = conv3d.vertex2facet_backward(c["g_v2f"], c["x_v"], c["filt_v2f"], c["face"])
    wgin, wgf = mo.vertex2facet_backward(d["g_v2f"].double(), d["x_v"].double(), d["filt_v2f"].double(), d["face"])
    assert rel_err(gin, wgin) <= TOL and rel_err(gf, wgf) <= TOL
    if ref.available():
        r_out = ref.v2f_forward(c["x_v"], c["filt_v2f"], c["face"])
        assert rel_err(out, r_out) <= TOL
        r_gin, r_gf = ref.v2f_backward(c["g_v2f"], c["x_v"], c["filt_v2f"], c["face"])
        assert rel_err(gin, r_gin) <= TOL and rel_err(gf, r_gf) <= TOL
        # the fp64 oracle arbitrates: we must not be further from it than the reference is (plus slack)
        assert max_abs(gf, wgf) <= max_abs(r_gf, wgf) * 4 + 1e-5 * float(wgf.abs().max())


@pytest.mark.parametrize("kind,C,r,K,cout", CASES)
def test_facet2vertex(mods, kind, C, r, K, cout):
    conv3d, _, mo, ref = mods
    d = conv_inputs(kind, C, r, K, cout, seed=5)
    c = _dev(d)
    nfc = mo.count_vertex_adjface(d["face"], d["vt_map"], d["nv_out"])
    nfc_c = nfc.cuda()
    out = conv3d.facet2vertex_forward(c["x_f"], c["filt_f2v"], c["coeff"], c["face"], nfc_c, c["vt_map"])
    want = mo.facet2vertex_forward(d["x_f"].double(), d["filt_f2v"].double(), d["coeff"].double(), d["face"], nfc,
                                   d["vt_map"])
    assert out.shape == want.shape and rel_err(out, want) <= TOL
    assert torch.all(out[nfc_c == 0] == 0)            # vertices no face maps to stay exactly zero
    gin, gf = conv3d.facet2vertex_backward(c["g_f2v"], c["x_f"], c["filt_f2v"], c["coeff"], c["face"], nfc_c,
                                           c["vt_map"])
    wgin, wgf = mo.facet2vertex_backward(d["g_f2v"].double(), d["x_f"].double(), d["filt_f2v"].double(),
                                         d["coeff"].double(), d["face"], nfc, d["vt_map"])
    assert rel_err(gin, wgin) <= TOL and rel_err(gf, wgf) <= TOL
    if ref.available() and "+drop" not in kind:       # the reference reads nfCount[-1] for dropped vertices
        r_out = ref.f2v_forward(c["x_f"], c["filt_f2v"], c["coeff"], c["face"], nfc_c, c["vt_map"])
        assert rel_err(out, r_out) <= TOL
        r_gin, r_gf = ref.f2v_backward(c["g_f2v"], c["x_f"], c["filt_f2v"], c["coeff"], c["face"], nfc_c, c["vt_map"])
        assert rel_err(gin, r_gin) <= TOL and rel_err(gf, r_gf) <= TOL


@pytest.mark.parametrize("kind,C,r,K,cout", CASES)
def test_facet2facet_fp32(mods, kind, C, r, K, cout):
    conv3d, _, mo, ref = mods
    d = conv_inputs(kind, C, r, K, cout, seed=6)
    c = _dev(d)
    conv3d.set_f2f_precision("fp32")
    out = conv3d.facet2facet_forward(c["tex"], c["filt_f2f"], c["bary"], c["cum"])
    want = mo.facet2facet_forward(d["tex"].double(), d["filt_f2f"].double(), d["bary"].double(), d["cum"])
    assert out.shape == want.shape and rel_err(out, want) <= TOL
    zero_faces = (d["counts"] == 0).nonzero().flatten()
    assert torch.all(out[zero_faces.cuda()] == 0)
    gin, gf = conv3d.facet2facet_backward(c["g_f2f"], c["tex"], c["filt_f2f"], c["bary"], c["cum"])
    wgin, wgf = mo.facet2facet_backward(d["g_f2f"].double(), d["tex"].double(), d["filt_f2f"].double(),
                                        d["bary"].double(), d["cum"])
    assert rel_err(gin, wgin) <= TOL and rel_err(gf, wgf) <= TOL
    if ref.available() and d["tex"].shape[0] * C * cout < 5e7:
        r_out = ref.f2f_forward(c["tex"], c["filt_f2f"], c["bary"], c["cum"])
        assert rel_err(out, r_out) <= TOL
        r_gin, r_gf = ref.f2f_backward(c["g_f2f"], c["tex"], c["filt_f2f"], c["bary"], c["cum"])
        assert rel_err(gin, r_gin) <= TOL and rel_err(gf, r_gf) <= TOL
        # The fp64 oracle arbitrates: our distance to fp64 against the reference's distance to fp64.
        # The FFMA path must be as close as the reference (factor 4 covers the different summation
        # order).  The tensor-core modes of "fp32" keep 16 (bf16 hi+lo) or 21 (tf32 hi+lo) mantissa bits
        # per operand and drop the lo*lo product, so they sit further from fp64 than an FFMA chain
        # while staying inside the 1e-4 gate: bounded by the factors below, with a floor of 2e-5 of the
        # tensor's largest value (operand rounding does not shrink with the length of the sum, the
        # reference's accumulation error does).  The FFMA path's floor covers tensors the reference
        # gets exactly right.
        for mode, k, flo in (("fp32", ARB_FP32, 2e-5), ("fp32_tf32x3", ARB_TF32X3, 2e-5), ("fp32_ffma", 4.0, 2e-6)):
            conv3d.set_f2f_precision(mode)
            o_m = conv3d.facet2facet_forward(c["tex"], c["filt_f2f"], c["bary"], c["cum"])
            gi_m, gf_m = conv3d.facet2facet_backward(c["g_f2f"], c["tex"], c["filt_f2f"], c["bary"], c["cum"])
            for name, ours, theirs, truth in (("out", o_m, r_out, want), ("gin", gi_m, r_gin, wgin), ("gf", gf_m, r_gf, wgf)):
                floor = flo * float(truth.abs().max()) if truth.numel() else 0.0
                assert max_abs(ours, truth) <= k * max_abs(theirs, truth) + floor, (mode, name, max_abs(ours, truth),
                                                                                   max_abs(theirs, truth))
        conv3d.set_f2f_precision("fp32")


def _ref_block(ref, x, Wv, Wf, Wo, face, counts, cum, bary_sh, coeff, nfc, vt_map, sh_eye, G):
    """The benchmark block chained by hand through the reference's own CUDA kernels (forward and
    backward), with torch for the glue the reference leaves to user code."""
    cin = x.shape[1]
    spatial = (sh_eye @ Wv).reshape(3, cin, 1).contiguous()
    y = ref.v2f_forward(x, spatial, face)
    tex = torch.repeat_interleave(y, counts.long(), dim=0)
    z = ref.f2f_forward(tex, Wf, bary_sh, cum)
    o = ref.f2v_forward(z, Wo, coeff, face, nfc, vt_map)
    gz, gWo = ref.f2v_backward(G, z, Wo, coeff, face, nfc, vt_map)
    gtex, gWf = ref.f2f_backward(gz, tex, Wf, bary_sh, cum)
    fid = torch.repeat_interleave(torch.arange(face.shape[0], device=x.device), counts.long())
    gy = torch.zeros_like(y).index_add_(0, fid, gtex)
    gx, gsp = ref.v2f_backward(gy, x, spatial, face)
    gWv = sh_eye.t() @ gsp.reshape(3, cin)
    return o, gx, [gWv, gWf, gWo]


def test_baseline_config_c1_block_exact(mods):
    """BASELINE configuration 1 as written: 4 icospheres of level 4 (2562 vertices, 5120 faces each),
    radial jitter N(0, 0.02), 32 -> 64 channels, L = 3, whole V2F -> F2F -> F2V block forward and
    backward, against the reference's live CUDA kernels and against the fp64 oracle."""
    conv3d, _, mo, ref = mods
    from picassoplus_b200 import synth
    from picassoplus_b200.block import conv_block
    from picassoplus_b200.math_utils import sph_harm_coeff
    cfg = synth.CONFIGS["c1"]
    L, cin, cout = cfg["L"], cfg["cin"], cfg["cout"]
    K = (L + 1) ** 2
    mb = synth.make_batch(cfg)
    assert mb.num_vertices == 4 * 2562 and mb.num_faces == 4 * 5120
    counts_np, bary_xyz = synth.texture_samples(mb.num_faces, seed=101)
    g = torch.Generator().manual_seed(102)
    rng = __import__("numpy").random.default_rng(103)
    x = torch.randn(mb.num_vertices, cin, generator=g)
    Wv = torch.from_numpy(synth.xavier_normal((K, cin), rng))
    Wf = torch.from_numpy(synth.xavier_normal((cout, cin, K), rng))
    Wo = torch.from_numpy(synth.xavier_normal((K, cout, 1), rng))
    G = torch.randn(mb.num_vertices, cout, generator=g)
    vertex, face = torch.from_numpy(mb.vertex), torch.from_numpy(mb.face)
    counts = torch.from_numpy(counts_np)
    cum = torch.cumsum(counts, 0, dtype=torch.int32)
    vt_map = torch.arange(mb.num_vertices, dtype=torch.int32)
    nfc = mo.count_vertex_adjface(face, vt_map, mb.num_vertices)
    coeff = mo.sph_harm_coeff(L, mo.triangle_geometry(vertex, face)[:, :3])
    bary_sh = mo.sph_harm_coeff(L, torch.from_numpy(bary_xyz))
    sh_eye = mo.sph_harm_coeff(L, torch.eye(3))

    xo = x.double().requires_grad_()
    wo = [w.double().requires_grad_() for w in (Wv, Wf, Wo)]
    oo = mo.conv_block(xo, wo[0], wo[1], wo[2], face, counts, cum, bary_sh.double(), coeff.double(), nfc, vt_map,
                       sh_eye.double())
    (oo * G.double()).sum().backward()
    truth = [oo.detach(), xo.grad] + [w.grad for w in wo]

    conv3d.set_f2f_precision("fp32")
    xd = x.cuda().requires_grad_()
    wd = [w.cuda().requires_grad_() for w in (Wv, Wf, Wo)]
    o = conv_block(xd, wd[0], wd[1], wd[2], face.cuda(), cum.cuda(), bary_sh.cuda(), coeff.cuda(), nfc.cuda(),
                   vt_map.cuda(), sh_eye.cuda())
    o.backward(G.cuda())
    ours = [o.detach(), xd.grad] + [w.grad for w in wd]
    names = ["out", "grad_x", "grad_Wv", "grad_Wf", "grad_Wo"]
    for n, a, b in zip(names, ours, truth):
        assert rel_err(a, b) <= TOL, (n, rel_err(a, b))
    if ref.available():
        ro, rgx, rgw = _ref_block(ref, x.cuda(), Wv.cuda(), Wf.cuda(), Wo.cuda(), face.cuda(), counts.cuda(), cum.cuda(),
                                  bary_sh.cuda(), coeff.cuda(), nfc.cuda(), vt_map.cuda(), sh_eye.cuda(), G.cuda())
        for n, a, b, t in zip(names, ours, [ro, rgx] + rgw, truth):
            assert rel_err(a, b) <= TOL, (n, rel_err(a, b))
            assert rel_err(b, t) <= TOL, ("reference vs fp64", n, rel_err(b, t))


@pytest.mark.parametrize("precision", ["fp32", "bf16", "fp32_ffma"])
def test_block_with_folded_repetition_equals_the_expanded_block(mods, precision):
    """conv_block folds 'repeat the face row once per sample' into facet2facet (per-face mean of the sample
    weights, one sample per face); conv_block_expanded runs the block as written.  Same output and gradients
    within the mode's gate; a face without samples gives 0 in both; two runs give identical bits."""
    conv3d, _, mo, _ = mods
    from picassoplus_b200 import synth, topology
    from picassoplus_b200.block import conv_block, conv_block_expanded
    L, cin, cout = 4, 32, 48
    K = (L + 1) ** 2
    mb = synth.concat_meshes([synth.heightfield(40, 7), synth.icosphere(3), synth.heightfield(33, 9)])
    nf, nv = mb.face.shape[0], mb.vertex.shape[0]
    counts_np, _ = synth.texture_samples(nf, seed=55)
    counts_np[5::29] = 6                                    # more samples than the kernels keep in registers
    counts_np[::17] = 0                                     # faces without a sample
    rng = np.random.default_rng(56)
    nik = int(counts_np.sum())
    bary = rng.dirichlet((1.0, 1.0, 1.0), size=nik).astype(np.float32)
    g = torch.Generator().manual_seed(57)
    dev = "cuda"
    x = torch.randn(nv, cin, generator=g).to(dev)
    Wv = torch.from_numpy(synth.xavier_normal((K, cin), rng)).to(dev)
    Wf = torch.from_numpy(synth.xavier_normal((cout, cin, K), rng)).to(dev)
    Wo = torch.from_numpy(synth.xavier_normal((K, cout, 1), rng)).to(dev)
    G = torch.randn(nv, cout, generator=g).to(dev)
    vertex, face = torch.from_numpy(mb.vertex), torch.from_numpy(mb.face)
    cum = torch.cumsum(torch.from_numpy(counts_np), 0, dtype=torch.int32).to(dev)
    vt_map = torch.arange(nv, dtype=torch.int32)
    nfc = mo.count_vertex_adjface(face, vt_map, nv).to(dev)
    coeff = mo.sph_harm_coeff(L, mo.triangle_geometry(vertex, face)[:, :3]).to(dev)
    bary_sh = mo.sph_harm_coeff(L, torch.from_numpy(bary)).to(dev)
    sh_eye = mo.sph_harm_coeff(L, torch.eye(3)).to(dev)
    face, vt_map = face.to(dev), vt_map.to(dev)

    fm = topology.face_means(bary_sh, cum)
    seg = torch.repeat_interleave(torch.arange(nf, device=dev), torch.from_numpy(counts_np).to(dev).long())
    want = torch.zeros(nf, K, dtype=torch.float64, device=dev).index_add_(0, seg, bary_sh.double())
    want = want / torch.from_numpy(counts_np).to(dev).clamp(min=1)[:, None]
    assert rel_err(fm.rows, want) <= 1e-6 and torch.all(fm.rows[::17] == 0)
    assert torch.equal(fm.one_each.cpu(), torch.arange(1, nf + 1, dtype=torch.int32))

    def run(block):
        xd = x.clone().requires_grad_()
        wd = [w.clone().requires_grad_() for w in (Wv, Wf, Wo)]
        o = block(xd, wd[0], wd[1], wd[2], face, cum, bary_sh, coeff, nfc, vt_map, sh_eye)
        o.backward(G)
        return [o.detach(), xd.grad] + [w.grad for w in wd]

    conv3d.set_f2f_precision(precision)
    try:
        folded, expanded, again = run(conv_block), run(conv_block_expanded), run(conv_block)
    finally:
        conv3d.set_f2f_precision("fp32")
    gate = {"fp32": TOL, "fp32_ffma": 2e-5, "bf16": 2e-2}[precision]
    for n, a, b, c in zip(["out", "grad_x", "grad_Wv", "grad_Wf", "grad_Wo"], folded, expanded, again):
        assert rel_err(a, b) <= gate, (n, rel_err(a, b))
        assert torch.equal(a, c), n


@pytest.mark.parametrize("nf,cin,cout,F", [(3000, 64, 64, 25), (1234, 128, 96, 16), (777, 32, 300, 9), (500, 3, 32, 16),
                                            (650, 48, 40, 7), (129, 272, 64, 4)])
@pytest.mark.parametrize("precision", ["fp32", "bf16", "tf32", "fp32_ffma"])
def test_one_sample_forward_equals_the_general_forward(mods, nf, cin, cout, F, precision):
    """pb200_facet2facet_one_sample_forward against pb200_facet2facet_forward with numInterior = 1..Nf and against
    the fp64 formula; shapes on the exchanged-roles tensor-core kernel, on its chunked form (more than 256 input
    channels), and on the fallbacks (F = 7, fp32_ffma)."""
    conv3d, _, mo, _ = mods
    from picassoplus_b200.block import one_sample_forward
    g = torch.Generator().manual_seed(nf + cin)
    x = torch.randn(nf, cin, generator=g).cuda()
    w = (torch.randn(cout, cin, F, generator=g) / (cin * F) ** 0.5).cuda()
    b = torch.randn(nf, F, generator=g).cuda()
    one_each = torch.arange(1, nf + 1, dtype=torch.int32, device="cuda")
    truth = torch.einsum("fd,fc,ocd->fo", b.double(), x.double(), w.double())
    conv3d.set_f2f_precision(precision)
    try:
        from picassoplus_b200 import topology
        got = one_sample_forward(x, w, b)
        general = conv3d.facet2facet_forward(x, w, b, one_each)
        again = one_sample_forward(x, w, b)
        # the caller-kept padded copy of the weight rows changes nothing but the work done per call
        bp = topology.pad_rows(b)
        assert (bp is None) == (F % 4 == 0)
        kept = one_sample_forward(x, w, b, bp)
        go = torch.randn(nf, cout, generator=g).cuda()
        back, back_kept = conv3d.facet2facet_backward(go, x, w, b, one_each), conv3d.facet2facet_backward(go, x, w, b, one_each, bp)
    finally:
        conv3d.set_f2f_precision("fp32")
    gate = {"fp32": TOL, "fp32_ffma": 2e-5, "bf16": 2e-2, "tf32": 2e-3}[precision]
    assert rel_err(got, truth) <= gate and rel_err(general, truth) <= gate, (rel_err(got, truth), rel_err(general, truth))
    assert torch.equal(got, again) and torch.equal(got, kept)
    assert torch.equal(back[0], back_kept[0]) and torch.equal(back[1], back_kept[1])


@pytest.mark.parametrize("L", [0, 2, 3, 4, 5])
def test_face_means_of_sh_components_in_one_kernel(mods, L):
    """pb200_face_mean_sph_harm against pb200_sph_harm_coeff followed by pb200_face_mean_rows (same bits) and against the
    fp64 oracle; faces without samples, a long run of samples on one face, and the conv_block call that takes the means."""
    _, _, mo, _ = mods
    from picassoplus_b200 import topology
    from picassoplus_b200.math_utils import sph_harm_coeff
    rng = np.random.default_rng(70 + L)
    nf = 1000
    counts = rng.integers(0, 5, size=nf)
    counts[123] = 37
    nik = int(counts.sum())
    xyz = torch.from_numpy(rng.dirichlet((1.0, 1.0, 1.0), size=nik).astype(np.float32)).cuda()
    cum = torch.cumsum(torch.from_numpy(counts), 0, dtype=torch.int32).cuda()
    fused = topology.face_means_sph_harm(L, xyz, cum)
    two_step = topology.face_means(sph_harm_coeff(L, xyz), cum)
    assert torch.equal(fused.rows, two_step.rows) and torch.equal(fused.one_each, two_step.one_each)
    sh = mo.sph_harm_coeff(L, xyz.cpu()).double()
    seg = torch.repeat_interleave(torch.arange(nf), torch.from_numpy(counts))
    want = torch.zeros(nf, (L + 1) ** 2, dtype=torch.float64).index_add_(0, seg, sh) / torch.from_numpy(counts).clamp(min=1)[:, None]
    assert max_abs(fused.rows, want) <= 5e-6
    assert torch.all(fused.rows[torch.from_numpy(counts == 0).cuda()] == 0)


def test_one_benchmark_mesh_against_fp64(mods):
    """One 360 x 360 heightfield mesh of the headline configuration (128 -> 128 channels, L = 4,
    ~232 k faces): facet2facet forward and backward in every tensor-core mode against the fp64
    formulas of the oracle (evaluated with torch in fp64 on the device, in face chunks)."""
    conv3d, _, mo, _ = mods
    from picassoplus_b200 import synth
    cfg = synth.CONFIGS["c5"]
    mb = synth.make_batch(cfg, 1, 0)
    counts_np, _ = synth.texture_samples(mb.num_faces, 3)
    g = torch.Generator().manual_seed(5)
    cum = torch.cumsum(torch.from_numpy(counts_np), 0, dtype=torch.int32).cuda()
    nik = int(counts_np.sum())
    C, F, cout = cfg["cin"], (cfg["L"] + 1) ** 2, cfg["cout"]
    tex = torch.randn(nik, C, generator=g).cuda()
    bary = torch.randn(nik, F, generator=g).cuda()
    W = (torch.randn(cout, C, F, generator=g) / (C * F) ** 0.5).cuda()
    go = torch.randn(mb.num_faces, cout, generator=g).cuda()
    want = mo.facet2facet_forward(tex.double(), W.double(), bary.double(), cum, chunk=16384)
    wgin, wgf = mo.facet2facet_backward(go.double(), tex.double(), W.double(), bary.double(), cum, chunk=16384)
    gates = {"fp32": 1e-4, "fp32_tf32x3": 1e-4, "tf32": 2e-3, "bf16": 2e-2}
    try:
        for mode, gate in gates.items():
            conv3d.set_f2f_precision(mode)
            out = conv3d.facet2facet_forward(tex, W, bary, cum)
            gin, gf = conv3d.facet2facet_backward(go, tex, W, bary, cum)
            errs = dict(out=rel_err(out, want), gin=rel_err(gin, wgin), gf=rel_err(gf, wgf))
            assert max(errs.values()) <= gate, (mode, errs)
    finally:
        conv3d.set_f2f_precision("fp32")


def test_filter_gradient_over_a_long_batch_against_fp64(mods):
    """Eight meshes of the headline configuration (1.86 M faces): the filter gradient sums over all faces,
    a CTA of the tensor-core kernel walks 100 000 of them.  The tensor core adds into its accumulator with
    truncation, so without the periodic flush of the accumulator into a round-to-nearest running sum the result
    drifts towards zero with the length of that walk (-3.1e-4 here, -1.2e-3 on the 32-mesh batch): the gate
    must hold at this size too."""
    conv3d, _, mo, _ = mods
    from picassoplus_b200 import synth
    cfg = dict(synth.CONFIGS["c5"])
    mb = synth.make_batch(cfg, 8, 0)
    counts_np = np.concatenate([synth.texture_samples(int(m), 11 + i)[0] for i, m in enumerate(mb.mf)])
    g = torch.Generator(device="cuda").manual_seed(6)
    cum = torch.cumsum(torch.from_numpy(counts_np), 0, dtype=torch.int32).cuda()
    nik = int(counts_np.sum())
    C, F, cout = cfg["cin"], (cfg["L"] + 1) ** 2, cfg["cout"]
    tex = torch.randn(nik, C, generator=g, device="cuda")
    bary = torch.randn(nik, F, generator=g, device="cuda")
    W = torch.randn(cout, C, F, generator=g, device="cuda") / (C * F) ** 0.5
    go = torch.randn(mb.num_faces, cout, generator=g, device="cuda")
    # fp64 filter gradient in face chunks (the input gradient has no long sum and is covered elsewhere)
    _, wgf = mo.facet2facet_backward(go.double(), tex.double(), W.double(), bary.double(), cum, chunk=16384)
    gates = {"fp32": 1e-4, "tf32": 2e-3, "bf16": 2e-2}
    try:
        for mode, gate in gates.items():
            conv3d.set_f2f_precision(mode)
            _, gf = conv3d.facet2facet_backward(go, tex, W, bary, cum)
            err = rel_err(gf, wgf)
            scale = float((gf.double() * wgf).sum() / (wgf * wgf).sum()) - 1.0
            assert err <= gate, (mode, err)
            assert abs(scale) <= 5e-5, (mode, "systematic scale error", scale)
    finally:
        conv3d.set_f2f_precision("fp32")


def test_autograd_functions_match_oracle_block(mods):
    """The three autograd Functions chained as the benchmark block, against the oracle's
    autograd over the same formula (fp64)."""
    conv3d, _, mo, _ = mods
    from picassoplus_b200.math_utils import sph_harm_coeff
    d = conv_inputs("ico2x3", 16, 1, 16, 24, seed=9)
    L, cin, cout = 3, 16, 24
    g = torch.Generator().manual_seed(1)
    Wv = torch.randn(16, cin, generator=g) * 0.2
    Wf = d["filt_f2f"]
    Wo = torch.randn(16, cout, 1, generator=g) * 0.2
    geo = mo.triangle_geometry(d["vertex"], d["face"])
    coeff = mo.sph_harm_coeff(L, geo[:, :3])
    bary_sh = mo.sph_harm_coeff(L, d["bary_xyz"])
    nfc = mo.count_vertex_adjface(d["face"], d["vt_map"], d["nv_out"])
    G = torch.randn(d["nv_out"], cout, generator=g)

    def run_oracle():
        x = d["x_v"].double().requires_grad_()
        ws = [w.double().requires_grad_() for w in (Wv, Wf, Wo)]
        o = mo.conv_block(x, ws[0], ws[1], ws[2], d["face"], d["counts"], d["cum"], bary_sh.double(),
                          coeff.double(), nfc, d["vt_map"], mo.sph_harm_coeff(L, torch.eye(3)).double())
        (o * G.double()).sum().backward()
        return o.detach(), x.grad, [w.grad for w in ws]

    def run_gpu():
        from picassoplus_b200.block import conv_block
        x = d["x_v"].cuda().requires_grad_()
        ws = [w.cuda().requires_grad_() for w in (Wv, Wf, Wo)]
        o = conv_block(x, ws[0], ws[1], ws[2], d["face"].cuda(), d["cum"].cuda(), bary_sh.cuda(), coeff.cuda(),
                       nfc.cuda(), d["vt_map"].cuda(), sph_harm_coeff(L, torch.eye(3, device="cuda")))
        (o * G.cuda()).sum().backward()
        return o.detach(), x.grad, [w.grad for w in ws]

    o1, gx1, gw1 = run_oracle()
    o2, gx2, gw2 = run_gpu()
    assert rel_err(o2, o1) <= TOL and rel_err(gx2, gx1) <= TOL
    for a, b in zip(gw2, gw1):
        assert rel_err(a, b) <= TOL


def test_run_to_run_deterministic(mods):
    conv3d, _, mo, _ = mods
    d = conv_inputs("grid33x2", 64, 1, 16, 32, seed=21)
    c = _dev(d)
    nfc = mo.count_vertex_adjface(d["face"], d["vt_map"], d["nv_out"]).cuda()

    def once():
        from picassoplus_b200.topology import clear_cache
        clear_cache()
        a = conv3d.vertex2facet_backward(c["g_v2f"], c["x_v"], c["filt_v2f"], c["face"])
        b = conv3d.facet2vertex_forward(c["x_f"], c["filt_f2v"], c["coeff"], c["face"], nfc, c["vt_map"])
        e = conv3d.facet2vertex_backward(c["g_f2v"], c["x_f"], c["filt_f2v"], c["coeff"], c["face"], nfc, c["vt_map"])
        f = conv3d.facet2facet_backward(c["g_f2f"], c["tex"], c["filt_f2f"], c["bary"], c["cum"])
        return [*a, b, *e, *f]

    first = once()
    for _ in range(3):
        for x, y in zip(first, once()):
            assert torch.equal(x, y)


def test_sph_harm_and_geometry(mods):
    _, decimate, mo, _ = mods
    from picassoplus_b200.math_utils import sph_harm_coeff
    g = torch.Generator().manual_seed(2)
    xyz = torch.randn(5000, 3, generator=g)
    xyz[:4] = torch.tensor([[1., 0, 0], [0, 1., 0], [0, 0, 1.], [0, 0, 0]])
    for L in range(6):
        got = sph_harm_coeff(L, xyz.cuda())
        want = mo.sph_harm_coeff(L, xyz)
        assert got.shape == want.shape
        assert rel_err(got, mo.sph_harm_coeff(L, xyz.double())) <= 1e-5
        assert max_abs(got, want) <= 2e-6
    with pytest.raises(NotImplementedError):
        sph_harm_coeff(6, xyz.cuda())
    d = conv_inputs("grid17x2", 4, 1, 4, 2, seed=1)
    geo = decimate.compute_triangle_geometry_(d["vertex"].cuda(), d["face"].cuda())
    assert max_abs(geo, mo.triangle_geometry(d["vertex"], d["face"])) <= 1e-6


def test_error_behaviour(mods):
    conv3d, _, _, _ = mods
    d = _dev(conv_inputs("ico1x2", 8, 1, 16, 4, seed=1))
    with pytest.raises(RuntimeError):
        conv3d.vertex2facet(d["x_v"].cpu(), d["filt_v2f"], d["face"])              # not CUDA
    with pytest.raises(RuntimeError):
        conv3d.vertex2facet(d["x_v"].t().contiguous().t(), d["filt_v2f"], d["face"])  # not contiguous
    with pytest.raises(RuntimeError):
        conv3d.vertex2facet(d["x_v"], d["filt_v2f"][:2].contiguous(), d["face"])    # needs 3 filters
    with pytest.raises(RuntimeError):
        conv3d.vertex2facet(d["x_v"], d["filt_v2f"], d["face"].long())              # int32 indices only
    with pytest.raises(RuntimeError):
        conv3d.facet2facet(d["tex"], torch.zeros(4, 8, 51, device="cuda"), torch.zeros(d["tex"].shape[0], 51,
                           device="cuda"), d["cum"])                                 # F <= 50
    with pytest.raises(RuntimeError):
        conv3d.facet2vertex(d["x_f"], d["filt_f2v"][:, :4].contiguous(), d["coeff"], d["face"],
                            torch.ones(d["nv_out"], dtype=torch.int32, device="cuda"), d["vt_map"])
    bad = d["face"].clone()
    bad[0, 0] = 10 ** 6                                                              # index out of range: reported, not dereferenced
    with pytest.raises(RuntimeError):
        conv3d.vertex2facet_backward(d["g_v2f"], d["x_v"], d["filt_v2f"], bad)
    # the context is still usable afterwards
    assert torch.isfinite(conv3d.vertex2facet(d["x_v"], d["filt_v2f"], d["face"])).all()


def test_error_behaviour_of_the_shared_rows_entries(mods):
    """Bad arguments to the one-sample forward, the padded-copy arguments, the per-face means and the cluster form of the
    max-pool gradient are answered with an error (RuntimeError from the wrappers, an error code from the C ABI), and the
    context keeps working."""
    conv3d, _, _, _ = mods
    from picassoplus_b200 import _lib, topology
    from picassoplus_b200.block import one_sample_forward
    from picassoplus_b200.topology import ptr, stream_ptr
    nf, cin, cout, F = 300, 32, 16, 25
    g = torch.Generator().manual_seed(5)
    x = torch.randn(nf, cin, generator=g).cuda()
    w = torch.randn(cout, cin, F, generator=g).cuda()
    b = torch.randn(nf, F, generator=g).cuda()
    with pytest.raises(RuntimeError):
        one_sample_forward(x, w[:, :8].contiguous(), b)                        # filter input channels
    with pytest.raises(RuntimeError):
        one_sample_forward(x, w, b[:-1].contiguous())                           # one weight row per face
    with pytest.raises(RuntimeError):
        one_sample_forward(x, w, b, torch.zeros(nf, 27, device="cuda"))         # padded copy of the wrong width
    with pytest.raises(RuntimeError):
        one_sample_forward(x.cpu(), w, b)                                       # not CUDA
    with pytest.raises(RuntimeError):
        conv3d.facet2facet_backward(torch.zeros(nf, cout, device="cuda"), x, w, b,
                                    torch.arange(1, nf + 1, dtype=torch.int32, device="cuda"), torch.zeros(nf, 24, device="cuda"))
    with pytest.raises(RuntimeError):
        topology.face_means_sph_harm(4, torch.zeros(10, 2, device="cuda"), torch.arange(1, 11, dtype=torch.int32, device="cuda"))
    # straight at the C ABI: a workspace that is too small, an unknown precision, a degree above 5
    out = torch.empty(nf, cout, device="cuda")
    ws = torch.empty(16, dtype=torch.uint8, device="cuda")
    need = _lib.query("pb200_facet2facet_one_sample_forward_workspace_bytes", nf, cin, cout, F, _lib.PREC_FP32)
    assert need > 16
    with pytest.raises(RuntimeError, match="workspace"):
        _lib.call("pb200_facet2facet_one_sample_forward", nf, cin, cout, F, ptr(x), ptr(w), ptr(b), None, ptr(out), _lib.PREC_FP32,
                  ptr(ws), 16, stream_ptr(x.device))
    big = torch.empty(need, dtype=torch.uint8, device="cuda")
    with pytest.raises(RuntimeError, match="precision"):
        _lib.call("pb200_facet2facet_one_sample_forward", nf, cin, cout, F, ptr(x), ptr(w), ptr(b), None, ptr(out), 99, ptr(big), need,
                  stream_ptr(x.device))
    with pytest.raises(RuntimeError, match="degree"):
        _lib.call("pb200_face_mean_sph_harm", 10, 10, 6, ptr(x), ptr(torch.arange(1, 11, dtype=torch.int32, device="cuda")), ptr(out),
                  stream_ptr(x.device))
    assert _lib.query("pb200_padded_row_floats", 25) == 28 and _lib.query("pb200_padded_row_floats", 16) == 16
    # nothing of the above has left the device in a bad state
    assert torch.isfinite(one_sample_forward(x, w, b)).all()
