"""The C-ABI library loads without a GPU and exports every symbol the header declares;
host-side argument checks answer with status codes (no compute is launched here)."""
import ctypes
import os
import re

from conftest import ROOT


def _declared():
    text = open(os.path.join(ROOT, "include", "picasso_b200.h")).read()
    text = re.sub(r"/\*.*?\*/", "", text, flags=re.S)
    return sorted(set(re.findall(r"\b(pb200_[a-z0-9_]+)\s*\(", text)))


def test_library_exports_every_declared_symbol():
    from picassoplus_b200 import _lib
    names = _declared()
    assert len(names) >= 20
    lib = ctypes.CDLL(_lib.LIB_PATH)
    for n in names:
        assert hasattr(lib, n), n
    assert set(names) == set(_lib.SIGNATURES), set(names) ^ set(_lib.SIGNATURES)


def test_host_side_argument_checks():
    from picassoplus_b200 import _lib
    assert _lib.query("pb200_version") >= 100
    rc = _lib.raw("pb200_sph_harm_coeff")(10, 6, None, None, None)
    assert rc == _lib.EINVAL and "L=6" in _lib.last_error()
    rc = _lib.raw("pb200_vertex2facet_forward")(-1, 0, 4, 1, None, None, None, None, None)
    assert rc == _lib.EINVAL
    rc = _lib.raw("pb200_facet2facet_forward")(4, 8, 3, 3, 51, None, None, None, None, None, 0, None, 0, None)
    assert rc == _lib.EINVAL                       # F <= 50 like the reference
    rc = _lib.raw("pb200_vertex2facet_forward")(4, 8, 3, 1, None, None, None, None, None)
    assert rc == _lib.EINVAL and "null" in _lib.last_error()
    assert _lib.query("pb200_vertex_csr_workspace_bytes", 1000, 600) > 4 * 3000
    assert _lib.query("pb200_facet2facet_backward_workspace_bytes", 1000, 2500, 32, 64, 16, 0) > 0
    assert _lib.launch_count() == 0                # nothing was launched by the checks above
