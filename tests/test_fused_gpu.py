"""The fused operator + pointwise kernels (vertex2facet / facet2vertex followed by the depth_weights
product, bias and ReLU in one tcgen05 kernel), through the C ABI, against the unfused sequence of
this library (itself checked against the oracle and the reference kernels) and against the fp64
oracle; gates: fp32 mode 1e-4 relative, bf16 mode 2e-2.  The layer modules with fusion on and off
must agree, forward and backward."""
import pytest
import torch

from cases import conv_inputs
from conftest import rel_err

pytestmark = pytest.mark.gpu

SHAPES = [
    # topology, C, K, Cout
    ("ico2x3", 32, 16, 64),
    ("grid17x2+drop", 64, 25, 128),
    ("grid33x2", 128, 25, 128),
    ("grid17x2", 40, 9, 200),       # channels not a multiple of 32, output channels in two chunks
    ("grid9x1", 256, 16, 384),
    ("tri", 8, 4, 5),
]


def _dev(d):
    return {k: (v.cuda() if isinstance(v, torch.Tensor) else v) for k, v in d.items()}


@pytest.mark.parametrize("mode,gate", [("fp32", 1e-4), ("bf16", 2e-2)])
@pytest.mark.parametrize("kind,C,K,cout", SHAPES)
def test_fused_forward_matches_unfused_and_oracle(kind, C, K, cout, mode, gate):
    from oracle import mesh_oracle as mo
    from picassoplus_b200.mesh.pi_modules import conv3d, fused
    d = conv_inputs(kind, C, 1, K, cout, seed=51)
    c = _dev(d)
    g = torch.Generator().manual_seed(3)
    Wd = torch.randn(C, cout, generator=g) / C ** 0.5
    b = torch.randn(1, cout, generator=g) * 0.1
    nfc = mo.count_vertex_adjface(d["face"], d["vt_map"], d["nv_out"])
    fused.set_pointwise_precision(mode)
    try:
        # vertex2facet + pointwise
        out = fused.vertex2facet_pointwise(c["x_v"], c["filt_v2f"], c["face"], Wd.cuda(), b.cuda(), True)
        feats = conv3d.vertex2facet_forward(c["x_v"], c["filt_v2f"], c["face"])
        assert rel_err(out, torch.relu(feats @ Wd.cuda() + b.cuda())) <= gate
        want = torch.relu(mo.vertex2facet_forward(d["x_v"].double(), d["filt_v2f"].double(), d["face"]) @ Wd.double() + b.double())
        assert rel_err(out, want) <= gate
        lin = fused.vertex2facet_pointwise(c["x_v"], c["filt_v2f"], c["face"], Wd.cuda(), None, False)      # no bias, no ReLU
        assert rel_err(lin, feats @ Wd.cuda()) <= gate
        # facet2vertex + pointwise
        out2 = fused.facet2vertex_pointwise(c["x_f"], c["filt_f2v"], c["coeff"], c["face"], nfc.cuda(), c["vt_map"], Wd.cuda(),
                                            b.cuda(), True)
        feats2 = conv3d.facet2vertex_forward(c["x_f"], c["filt_f2v"], c["coeff"], c["face"], nfc.cuda(), c["vt_map"])
        assert rel_err(out2, torch.relu(feats2 @ Wd.cuda() + b.cuda())) <= gate
        want2 = torch.relu(mo.facet2vertex_forward(d["x_f"].double(), d["filt_f2v"].double(), d["coeff"].double(), d["face"], nfc,
                                                   d["vt_map"]) @ Wd.double() + b.double())
        assert rel_err(out2, want2) <= gate
        assert torch.equal(out2, fused.facet2vertex_pointwise(c["x_f"], c["filt_f2v"], c["coeff"], c["face"], nfc.cuda(),
                                                              c["vt_map"], Wd.cuda(), b.cuda(), True))   # run to run identical
    finally:
        fused.set_pointwise_precision("fp32")


def test_modules_with_and_without_fusion_agree():
    from picassoplus_b200.mesh import layers
    from picassoplus_b200.mesh import utils as mesh_utils
    torch.manual_seed(0)
    L, cin, mid, cout = 3, 16, 32, 24
    d = conv_inputs("ico2x3", cin, 1, (L + 1) ** 2, 8, seed=61)
    dev = torch.device("cuda")
    vertex, face, vt = d["vertex"].to(dev), d["face"].to(dev), d["vt_map"].to(dev)
    nfc = mesh_utils.count_vertex_adjface(face, vt, vertex)
    coeff = layers.SphHarmCoeff(L)(mesh_utils.compute_triangle_geometry(vertex, face)[:, :3].contiguous())
    conv = layers.V2VConv3d(cin, [mid, cout], L, [1, 1]).to(dev).train()
    G = torch.randn(d["nv_out"], cout, device=dev)
    results = []
    try:
        for on in (True, False):
            layers.set_fusion(on)
            for p_ in conv.parameters():
                p_.grad = None
            x = d["x_v"].to(dev).requires_grad_()
            out = conv(x, face, nfc, vt, coeff)
            (out * G).sum().backward()
            results.append([out.detach(), x.grad] + [p_.grad.clone() for p_ in conv.parameters()])
    finally:
        layers.set_fusion(True)
    for a, b in zip(*results):
        assert rel_err(a, b) <= 2e-4


@pytest.mark.parametrize("rows,M,N", [(5000, 64, 128), (333, 128, 256), (9000, 256, 384), (70, 8, 12), (4096, 384, 64)])
@pytest.mark.parametrize("mode", ["fp32", "bf16"])
def test_rows_contract_and_masked_rows_matmul(rows, M, N, mode):
    """The two tensor-core kernels of the modules' backward against fp64: a^T b with column sums of b
    (contraction over rows), and (g masked by an activation) @ w."""
    from picassoplus_b200 import _lib
    from picassoplus_b200.mesh.pi_modules import fused
    from picassoplus_b200.topology import ptr, stream_ptr
    gate = 1e-4 if mode == "fp32" else 2e-2
    gen = torch.Generator(device="cuda").manual_seed(rows + M)
    a = torch.randn(rows, M, device="cuda", generator=gen)
    b = torch.randn(rows, N, device="cuda", generator=gen)
    fused.set_pointwise_precision(mode)
    try:
        out, colsum = fused.rows_contract(a, b)
        again, _ = fused.rows_contract(a, b)
        assert torch.equal(out, again)                                  # fixed-order reduction
        want = a.double().t() @ b.double()
        assert rel_err(out, want) <= gate
        assert rel_err(colsum, b.double().sum(0, keepdim=True)) <= 1e-5
        if N % 8 == 0:
            act = torch.randn(rows, N, device="cuda", generator=gen)     # stands for the activated output
            w = torch.randn(N, M, device="cuda", generator=gen) * 0.1    # depth_weights^T
            dev = a.device
            g_feats = torch.empty(rows, M, device=dev)
            g_masked = torch.empty(rows, N, device=dev)
            prec = _lib.PRECISIONS[mode]
            nb = _lib.query("pb200_masked_rows_matmul_workspace_bytes", N, prec)
            ws = torch.empty(max(nb, 1), dtype=torch.uint8, device=dev)
            _lib.call("pb200_masked_rows_matmul", rows, N, M, ptr(b), ptr(act), ptr(w), ptr(g_feats), ptr(g_masked), prec,
                      ptr(ws), nb, stream_ptr(dev))
            gm = b * (act > 0)
            assert torch.equal(g_masked, gm)
            assert rel_err(g_feats, gm.double() @ w.double()) <= gate
    finally:
        fused.set_pointwise_precision("fp32")
