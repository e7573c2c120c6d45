"""GraphedStep: a forward + backward step of the block replayed from a CUDA graph gives
bit-identical outputs and gradients to the eager step, also after the inputs changed in place."""
import pytest
import torch

from cases import conv_inputs

pytestmark = pytest.mark.gpu


def test_graph_replay_matches_eager():
    from picassoplus_b200.block import conv_block
    from picassoplus_b200.graph import GraphedStep
    from picassoplus_b200.math_utils import sph_harm_coeff
    d = conv_inputs("ico2x3", 32, 1, 16, 64, seed=13, zero_sample_faces=False)
    c = {k: (v.cuda() if isinstance(v, torch.Tensor) else v) for k, v in d.items()}
    L = 3
    g = torch.Generator(device="cuda").manual_seed(1)
    Wv = (torch.randn(16, 32, device="cuda", generator=g) * 0.2).requires_grad_()
    Wf = (torch.randn(64, 32, 16, device="cuda", generator=g) * 0.05).requires_grad_()
    Wo = (torch.randn(16, 64, 1, device="cuda", generator=g) * 0.2).requires_grad_()
    x = c["x_v"].clone().requires_grad_()
    nv = x.shape[0]
    vt = torch.arange(nv, dtype=torch.int32, device="cuda")
    from picassoplus_b200.mesh import utils as mesh_utils
    nfc = mesh_utils.count_vertex_adjface(c["face"], vt, c["vertex"])
    sh_eye = sph_harm_coeff(L, torch.eye(3, device="cuda"))
    G = torch.randn(nv, 64, device="cuda", generator=g)
    out_box = {}

    def step():
        for p in (x, Wv, Wf, Wo):
            if p.grad is not None:
                p.grad.zero_()
        o = conv_block(x, Wv, Wf, Wo, c["face"], c["cum"], c["bary"], c["coeff"], nfc, vt, sh_eye)
        o.backward(G)
        out_box["o"] = o.detach()          # no reference to the autograd graph outlives the step

    def snapshot():
        torch.cuda.synchronize()
        return [out_box["o"].detach().clone()] + [p.grad.clone() for p in (x, Wv, Wf, Wo)]

    step()                                    # eager: warms the CSR cache
    want = snapshot()
    gs = GraphedStep(step)
    gs()
    got = snapshot()
    for a, b in zip(got, want):
        assert torch.equal(a, b)
    with torch.no_grad():                     # new data in place: the replay must see it
        x.mul_(0.5)
    step()
    want2 = snapshot()
    gs()
    got2 = snapshot()
    for a, b in zip(got2, want2):
        assert torch.equal(a, b)
    assert not torch.equal(got2[0], got[0])
