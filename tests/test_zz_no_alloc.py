"""The allocation-free entry point pb200_vertex2facet_backward_static, called through the
C ABI, against the regular entry point (caller-provided workspace).

It exists for callers that cannot allocate device memory when they call the library
(a frozen or locked framework allocator, a fixed start-up memory budget, a callback that
must not call cudaMalloc): its scratch is a 4 MiB array inside the library image.  The
file is named so that pytest collects it last: the first call on a device resolves the
array's address, and a failure here cannot hide the result of any other test.
"""
import pytest
import torch

from cases import conv_inputs

pytestmark = pytest.mark.gpu


def _run(lib, name, d, csr, gin, gf, ws=None):
    from picassoplus_b200.topology import ptr, stream_ptr
    Nv, C = d["x_v"].shape
    r = d["filt_v2f"].shape[2]
    Nf = d["face"].shape[0]
    args = [Nf, Nv, C, r, ptr(d["g_v2f"]), ptr(d["x_v"]), ptr(d["filt_v2f"]), ptr(d["face"]), ptr(csr.rowptr),
            ptr(csr.entries), ptr(gin), ptr(gf)]
    if ws is not None:
        args += [ptr(ws), ws.numel()]
    args.append(stream_ptr(d["x_v"].device))
    lib.call(name, *args)


@pytest.mark.parametrize("kind,C,r", [("grid33x2", 128, 1), ("ico2x3", 5, 2)])
def test_static_scratch_variant_matches_regular_entry_point(kind, C, r):
    from picassoplus_b200 import _lib
    from picassoplus_b200.topology import build_vertex_csr
    d = {k: (v.cuda() if isinstance(v, torch.Tensor) else v) for k, v in conv_inputs(kind, C, r, 4, 4, seed=77).items()}
    Nv = d["x_v"].shape[0]
    Nf = d["face"].shape[0]
    csr = build_vertex_csr(d["face"], None, Nv, Nv)
    need = _lib.query("pb200_vertex2facet_backward_workspace_bytes", Nf, Nv, C, r)
    assert need <= _lib.query("pb200_vertex2facet_backward_static_max_bytes")
    ws = torch.empty(need, dtype=torch.uint8, device="cuda")
    gin_ref = torch.empty(Nv, C, device="cuda")
    gf_ref = torch.empty(3, C, r, device="cuda")
    _run(_lib, "pb200_vertex2facet_backward", d, csr, gin_ref, gf_ref, ws)
    for attempt in range(2):                      # two calls in a row share the built-in array
        g2 = d["g_v2f"] * (attempt + 1)           # different data on the second call
        d2 = dict(d, g_v2f=g2.contiguous())
        gin = torch.full((Nv, C), float("nan"), device="cuda")
        gf = torch.full((3, C, r), float("nan"), device="cuda")
        _run(_lib, "pb200_vertex2facet_backward_static", d2, csr, gin, gf)
        torch.cuda.synchronize()
        scale = float(attempt + 1)
        tol = 1e-4                                # the gate of the other fp32 parity tests
        for got, want in ((gin, gin_ref * scale), (gf, gf_ref * scale)):
            err = float((got - want).abs().max() / (want.abs().max() + 1e-30))
            assert err <= tol, (attempt, err)
        if attempt == 0:                          # same inputs, same launch plan: bit-identical
            assert torch.equal(gin, gin_ref) and torch.equal(gf, gf_ref)


def test_static_scratch_variant_rejects_oversized_shapes():
    from picassoplus_b200 import _lib
    limit = _lib.query("pb200_vertex2facet_backward_static_max_bytes")
    C = 4096                                      # needs more partial rows than the array holds
    assert _lib.query("pb200_vertex2facet_backward_workspace_bytes", 10 ** 6, 10 ** 6, C, 1) > limit
    rc = _lib.raw("pb200_vertex2facet_backward_static")(10 ** 6, 10 ** 6, C, 1, None, None, None, None, None, None,
                                                         None, None, None)
    assert rc == _lib.EWORKSPACE
    assert "built-in array" in _lib.last_error()
