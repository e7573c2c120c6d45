"""facet2facet on the tcgen05 tensor-core path (through the C ABI) against the fp64 oracle
and against the library's own fp32 FFMA path.  Gates (max|a-b| / max|b| per tensor): 'fp32'
mode (bf16 hi+lo operands, three products per term) and 'fp32_tf32x3' (tf32 hi+lo) <= 1e-4
like every fp32 feature tensor; 'tf32' mode <= 2e-3; 'bf16' mode <= 2e-2 (the stated
tolerance of bf16-operand variants)."""
import pytest
import torch

from conftest import rel_err
from cases import conv_inputs

pytestmark = pytest.mark.gpu

GATE = {"fp32": 1e-4, "fp32_tf32x3": 1e-4, "tf32": 2e-3, "bf16": 2e-2}
MODES = ["fp32", "fp32_tf32x3", "tf32", "bf16"]

SHAPES = [
    # topology, Cin, K(=F), Cout, max samples per face
    ("ico2x3", 16, 16, 8, 4),          # 960 faces: 4 tiles, one k-group
    ("grid33x2", 32, 16, 64, 4),       # c1-like channels, ~3.7k faces
    ("grid33x2", 128, 25, 128, 4),     # c5-like channels
    ("grid17x2", 64, 9, 128, 9),       # faces with more samples than stay in registers / staged rows
    ("ico1x2", 48, 4, 100, 2),         # Cout not a multiple of 32, Cin = 3 groups
    ("tri", 16, 16, 16, 3),            # a single face
    ("ico2x3", 3, 16, 32, 4),          # the reference networks' texture entry (RGB in, 32 out): channels padded to 16
    ("grid17x2", 40, 25, 200, 4),      # channels padded 40 -> 48, output channels in two chunks (128 + 72)
    ("grid9x1", 256, 16, 384, 3),      # output channels in three chunks; input gradient accumulates over 256 + 128
]


def _dev(d):
    return {k: (v.cuda() if isinstance(v, torch.Tensor) else v) for k, v in d.items()}


@pytest.fixture(scope="module")
def mods():
    from picassoplus_b200.mesh.pi_modules import conv3d
    from oracle import mesh_oracle
    yield conv3d, mesh_oracle
    conv3d.set_f2f_precision("fp32")


@pytest.mark.parametrize("mode", MODES)
@pytest.mark.parametrize("kind,C,K,cout,tmax", SHAPES)
def test_forward_matches_oracle(mods, kind, C, K, cout, tmax, mode):
    conv3d, mo = mods
    d = conv_inputs(kind, C, 1, K, cout, seed=41, max_per_face=tmax)
    c = _dev(d)
    want = mo.facet2facet_forward(d["tex"].double(), d["filt_f2f"].double(), d["bary"].double(), d["cum"])
    conv3d.set_f2f_precision(mode)
    out = conv3d.facet2facet_forward(c["tex"], c["filt_f2f"], c["bary"], c["cum"])
    torch.cuda.synchronize()
    assert out.shape == want.shape
    assert rel_err(out, want) <= GATE[mode], (mode, rel_err(out, want))
    zero_faces = (d["counts"] == 0).nonzero().flatten()
    assert torch.all(out[zero_faces.cuda()] == 0)
    # deterministic
    again = conv3d.facet2facet_forward(c["tex"], c["filt_f2f"], c["bary"], c["cum"])
    assert torch.equal(out, again)


def test_forward_many_tiles_vs_ffma_path(mods):
    """One full 360x360 heightfield mesh at the benchmark's channel widths: ~900 tiles, so
    every CTA walks several tiles and every barrier wraps its phase many times."""
    conv3d, _ = mods
    from picassoplus_b200 import synth
    mb = synth.heightfield_batch(1, 360, seed=9)
    nf = mb.num_faces
    counts, _ = synth.texture_samples(nf, 3)
    g = torch.Generator().manual_seed(5)
    cum = torch.cumsum(torch.from_numpy(counts), 0, dtype=torch.int32).cuda()
    nik = int(counts.sum())
    C, F, cout = 128, 25, 128
    tex = torch.randn(nik, C, generator=g).cuda()
    bary = torch.randn(nik, F, generator=g).cuda()
    W = (torch.randn(cout, C, F, generator=g) / (C * F) ** 0.5).cuda()
    conv3d.set_f2f_precision("fp32_ffma")
    want = conv3d.facet2facet_forward(tex, W, bary, cum)
    for mode in MODES:
        conv3d.set_f2f_precision(mode)
        out = conv3d.facet2facet_forward(tex, W, bary, cum)
        torch.cuda.synchronize()
        assert rel_err(out, want) <= GATE[mode], (mode, rel_err(out, want))


BWD_SHAPES = SHAPES + [
    ("grid17x2", 7, 36, 12, 4),        # odd channel count, F = 36 (7 channels per slice; filter gradient on the FFMA path)
]


@pytest.mark.parametrize("kind,C,K,cout,tmax", [("ico2x3", 3, 16, 32, 4), ("grid17x2", 40, 25, 200, 4),
                                                ("grid9x1", 256, 16, 384, 3), ("grid33x2", 128, 25, 128, 4)])
def test_every_channel_count_runs_on_the_tensor_cores(mods, kind, C, K, cout, tmax):
    """Channel counts that are no multiple of 16 and output widths above 128 / 256 still take the three
    tcgen05 kernels (the library's per-kernel timing table names what was launched), never the FFMA path."""
    conv3d, _ = mods
    from picassoplus_b200 import _lib
    c = _dev(conv_inputs(kind, C, 1, K, cout, seed=47, max_per_face=tmax))
    conv3d.set_f2f_precision("fp32")
    _lib.prof_reset()
    _lib.prof_enable(True)
    try:
        conv3d.facet2facet_forward(c["tex"], c["filt_f2f"], c["bary"], c["cum"])
        conv3d.facet2facet_backward(c["g_f2f"], c["tex"], c["filt_f2f"], c["bary"], c["cum"])
        torch.cuda.synchronize()
    finally:
        _lib.prof_enable(False)
    names = {n for n, _, _ in _lib.prof_read(64)}
    _lib.prof_reset()
    assert {"f2f_fwd_tc", "f2f_bwd_gin_tc", "f2f_bwd_gfilter_tc"} <= names, names
    assert not any("sgemm" in n or n.startswith("f2f_build_A") or n == "f2f_gin_from_gA" for n in names), names



@pytest.mark.parametrize("mode", MODES)
@pytest.mark.parametrize("kind,C,K,cout,tmax", BWD_SHAPES)
def test_backward_matches_oracle(mods, kind, C, K, cout, tmax, mode):
    conv3d, mo = mods
    d = conv_inputs(kind, C, 1, K, cout, seed=43, max_per_face=tmax)
    c = _dev(d)
    wgin, wgf = mo.facet2facet_backward(d["g_f2f"].double(), d["tex"].double(), d["filt_f2f"].double(),
                                        d["bary"].double(), d["cum"])
    conv3d.set_f2f_precision(mode)
    gin, gf = conv3d.facet2facet_backward(c["g_f2f"], c["tex"], c["filt_f2f"], c["bary"], c["cum"])
    torch.cuda.synchronize()
    assert gin.shape == wgin.shape and gf.shape == wgf.shape
    assert rel_err(gin, wgin) <= GATE[mode], (mode, "gin", rel_err(gin, wgin))
    assert rel_err(gf, wgf) <= GATE[mode], (mode, "gf", rel_err(gf, wgf))
    gin2, gf2 = conv3d.facet2facet_backward(c["g_f2f"], c["tex"], c["filt_f2f"], c["bary"], c["cum"])
    assert torch.equal(gin, gin2) and torch.equal(gf, gf2)


def test_backward_many_tiles_vs_ffma_path(mods):
    conv3d, _ = mods
    from picassoplus_b200 import synth
    mb = synth.heightfield_batch(1, 200, seed=9)
    nf = mb.num_faces
    counts, _ = synth.texture_samples(nf, 3)
    g = torch.Generator().manual_seed(5)
    cum = torch.cumsum(torch.from_numpy(counts), 0, dtype=torch.int32).cuda()
    nik = int(counts.sum())
    C, F, cout = 128, 25, 128
    tex = torch.randn(nik, C, generator=g).cuda()
    bary = torch.randn(nik, F, generator=g).cuda()
    W = (torch.randn(cout, C, F, generator=g) / (C * F) ** 0.5).cuda()
    go = torch.randn(nf, cout, generator=g).cuda()
    conv3d.set_f2f_precision("fp32_ffma")
    wgin, wgf = conv3d.facet2facet_backward(go, tex, W, bary, cum)
    for mode in MODES:
        conv3d.set_f2f_precision(mode)
        gin, gf = conv3d.facet2facet_backward(go, tex, W, bary, cum)
        torch.cuda.synchronize()
        assert rel_err(gin, wgin) <= GATE[mode], (mode, rel_err(gin, wgin))
        assert rel_err(gf, wgf) <= GATE[mode], (mode, rel_err(gf, wgf))


def test_tf32x3_mode_is_closer_to_fp64_than_the_default(mods):
    """PB200_PREC_FP32_TF32X3 (tf32 hi+lo operands): within 1e-5 of the fp64 oracle, the
    backward tensors within 2e-6 (bf16 hi+lo, the default fp32 mode, sits near 5e-6 .. 1.3e-5)."""
    conv3d, mo = mods
    d = conv_inputs("grid17x2", 32, 1, 16, 48, seed=5)
    c = _dev(d)
    conv3d.set_f2f_precision("fp32_tf32x3")
    out = conv3d.facet2facet_forward(c["tex"], c["filt_f2f"], c["bary"], c["cum"])
    gin, gf = conv3d.facet2facet_backward(c["g_f2f"], c["tex"], c["filt_f2f"], c["bary"], c["cum"])
    w = mo.facet2facet_forward(d["tex"].double(), d["filt_f2f"].double(), d["bary"].double(), d["cum"])
    wgin, wgf = mo.facet2facet_backward(d["g_f2f"].double(), d["tex"].double(), d["filt_f2f"].double(),
                                        d["bary"].double(), d["cum"])
    errs = [rel_err(out, w), rel_err(gin, wgin), rel_err(gf, wgf)]
    assert max(errs) <= 1e-5, errs
    assert max(errs[1:]) <= 2e-6, errs


def test_wait_timeout_unwinds_and_reports(mods):
    """A wait that runs out must end the kernel by itself: the filter stream of the forward kernel is
    silenced (test switch) with a wait budget of about a millisecond, so the MMA issuer's first wait
    gives up, every role unwinds, tensor memory is freed and the per-device error word is raised.
    The next call reports PB200_ECUDA until the word is cleared; after that the path works again."""
    conv3d, mo = mods
    from picassoplus_b200 import _lib
    d = conv_inputs("ico2x3", 16, 1, 16, 8, seed=41)
    c = _dev(d)
    conv3d.set_f2f_precision("fp32")
    good = conv3d.facet2facet_forward(c["tex"], c["filt_f2f"], c["bary"], c["cum"])     # also allocates the error word
    torch.cuda.synchronize()
    assert _lib.async_error() == 0
    _lib.raw("pb200_set_wait_budget")(2_000_000)
    _lib.raw("pb200_test_silence_filter_stream")(1)
    try:
        conv3d.facet2facet_forward(c["tex"], c["filt_f2f"], c["bary"], c["cum"])        # returns OK, results invalid
        torch.cuda.synchronize()                                                        # the kernel ended by itself
    finally:
        _lib.raw("pb200_test_silence_filter_stream")(0)
        _lib.raw("pb200_set_wait_budget")(0)
    assert _lib.async_error() == 1
    with pytest.raises(RuntimeError, match="gave up"):
        conv3d.facet2facet_forward(c["tex"], c["filt_f2f"], c["bary"], c["cum"])
    _lib.clear_async_error()
    assert _lib.async_error() == 0
    again = conv3d.facet2facet_forward(c["tex"], c["filt_f2f"], c["bary"], c["cum"])
    torch.cuda.synchronize()
    assert torch.equal(again, good)
