"""ctypes binding of libpicasso_b200.so (the C ABI in include/picasso_b200.h).

There is no fallback: if the shared library has not been built, importing this module
raises, and every operator call goes through the CUDA kernels or fails with the
library's own error text.
"""
from __future__ import annotations

import ctypes as C
import os

_PKG = os.path.dirname(os.path.abspath(__file__))
LIB_PATH = os.path.join(_PKG, "libpicasso_b200.so")

OK, EINVAL, EWORKSPACE, ECUDA, EINDEX = 0, -1, -2, -3, -4
PREC_FP32, PREC_TF32, PREC_BF16, PREC_FP32_FFMA, PREC_FP32_TF32X3 = 0, 1, 2, 3, 4
PRECISIONS = {"fp32": PREC_FP32, "tf32": PREC_TF32, "bf16": PREC_BF16, "fp32_ffma": PREC_FP32_FFMA,
              "fp32_tf32x3": PREC_FP32_TF32X3}

if not os.path.exists(LIB_PATH):
    raise ImportError(
        f"{LIB_PATH} is missing: build it with `python -m picassoplus_b200.build` "
        "(nvcc, sm_100a). picassoplus_b200 has no CPU or PyTorch fallback.")

_lib = C.CDLL(LIB_PATH)

i64, i32, vp, sz, f32 = C.c_int64, C.c_int, C.c_void_p, C.c_size_t, C.c_float


class ProfRecord(C.Structure):
    _fields_ = [("name", C.c_char * 48), ("launches", C.c_int64), ("total_ms", C.c_double)]


# name -> (restype, argtypes); must list every function the header declares
SIGNATURES = {
    "pb200_version": (i32, []),
    "pb200_last_error": (C.c_char_p, []),
    "pb200_launch_count": (i64, []),
    "pb200_prof_enable": (None, [i32]),
    "pb200_prof_reset": (None, []),
    "pb200_prof_read": (i32, [C.POINTER(ProfRecord), i32]),
    "pb200_async_error": (i32, []),
    "pb200_clear_async_error": (None, []),
    "pb200_set_wait_budget": (None, [i64]),
    "pb200_test_silence_filter_stream": (None, [i32]),
    "pb200_check_num_interior": (i32, [i64, i64, vp, vp, vp]),
    "pb200_count_vertex_adjface": (i32, [i64, i64, i64, vp, vp, vp, vp]),
    "pb200_vertex_csr_workspace_bytes": (sz, [i64, i64]),
    "pb200_build_vertex_csr": (i32, [i64, i64, i64, vp, vp, vp, vp, vp, vp, sz, vp]),
    "pb200_vertex2facet_forward": (i32, [i64, i64, i32, i32, vp, vp, vp, vp, vp]),
    "pb200_vertex2facet_backward_workspace_bytes": (sz, [i64, i64, i32, i32]),
    "pb200_vertex2facet_backward": (i32, [i64, i64, i32, i32, vp, vp, vp, vp, vp, vp, vp, vp, vp, sz, vp]),
    "pb200_vertex2facet_backward_static_max_bytes": (sz, []),
    "pb200_vertex2facet_backward_static": (i32, [i64, i64, i32, i32, vp, vp, vp, vp, vp, vp, vp, vp, vp]),
    "pb200_facet2vertex_forward_workspace_bytes": (sz, [i64, i32, i32, i32]),
    "pb200_facet2vertex_forward": (i32, [i64, i64, i32, i32, i32, vp, vp, vp, vp, vp, vp, vp, vp, sz, vp]),
    "pb200_facet2vertex_backward_workspace_bytes": (sz, [i64, i32, i32, i32]),
    "pb200_facet2vertex_backward": (i32, [i64, i64, i64, i32, i32, i32, vp, vp, vp, vp, vp, vp, vp, vp, vp,
                                          vp, sz, vp]),
    "pb200_vertex2facet_pointwise_workspace_bytes": (sz, [i32, i32]),
    "pb200_vertex2facet_pointwise_forward": (i32, [i64, i64, i32, i32, vp, vp, vp, vp, vp, i32, vp, i32, vp, sz, vp]),
    "pb200_facet2vertex_pointwise_workspace_bytes": (sz, [i64, i32, i32]),
    "pb200_facet2vertex_pointwise_forward": (i32, [i64, i64, i32, i32, i32, vp, vp, vp, vp, vp, vp, vp, vp, i32, vp, i32,
                                                   vp, sz, vp]),
    "pb200_facet2facet_forward_workspace_bytes": (sz, [i64, i64, i32, i32, i32, i32]),
    "pb200_facet2facet_forward": (i32, [i64, i64, i32, i32, i32, vp, vp, vp, vp, vp, i32, vp, sz, vp]),
    "pb200_facet2facet_one_sample_forward_workspace_bytes": (sz, [i64, i32, i32, i32, i32]),
    "pb200_facet2facet_one_sample_forward": (i32, [i64, i32, i32, i32, vp, vp, vp, vp, vp, i32, vp, sz, vp]),
    "pb200_padded_row_floats": (i32, [i32]),
    "pb200_pad_rows": (i32, [i64, i32, vp, vp, vp]),
    "pb200_facet2facet_backward_workspace_bytes": (sz, [i64, i64, i32, i32, i32, i32]),
    "pb200_facet2facet_backward": (i32, [i64, i64, i32, i32, i32, vp, vp, vp, vp, vp, vp, vp, i32, vp, sz, vp]),
    "pb200_facet2facet_backward_padded": (i32, [i64, i64, i32, i32, i32, vp, vp, vp, vp, vp, vp, vp, vp, i32, vp, sz, vp]),
    "pb200_level_prepare": (i32, [i64, i64, i64, i32, vp, vp, vp, i32, i32, vp, vp, vp, vp, vp, vp, vp, vp, sz, vp]),
    "pb200_cluster_csr_workspace_bytes": (sz, [i64, i64]),
    "pb200_build_cluster_csr": (i32, [i64, i64, vp, vp, vp, vp, vp, vp, vp, sz, vp]),
    "pb200_mesh_max_pool_forward": (i32, [i64, i64, i32, vp, vp, vp, vp, vp, vp]),
    "pb200_mesh_max_pool_backward": (i32, [i64, i64, i32, vp, vp, vp, vp]),
    "pb200_mesh_max_pool_backward_clusters": (i32, [i64, i64, i32, vp, vp, vp, vp, vp, vp]),
    "pb200_mesh_avg_pool_forward": (i32, [i64, i64, i32, vp, vp, vp, vp, vp, vp]),
    "pb200_mesh_avg_pool_backward": (i32, [i64, i64, i32, vp, vp, vp, vp, vp]),
    "pb200_mesh_unpool_forward": (i32, [i64, i64, i32, vp, vp, vp, vp]),
    "pb200_mesh_unpool_backward": (i32, [i64, i64, i32, vp, vp, vp, vp, vp]),
    "pb200_build_key_csr": (i32, [i64, i64, vp, i32, vp, vp, vp, vp, sz, vp]),
    "pb200_pcloud_conv3d_forward": (i32, [i64, i64, i64, i32, i32, i32, i32, vp, vp, vp, vp, vp, vp, vp, vp, vp, vp]),
    "pb200_pcloud_conv3d_backward_workspace_bytes": (sz, [i64, i32, i32, i32]),
    "pb200_pcloud_conv3d_backward": (i32, [i64, i64, i64, i32, i32, i32, i32, vp, vp, vp, vp, vp, vp, vp, vp, vp, vp, vp,
                                           vp, sz, vp]),
    "pb200_mesh_simplify_workspace_bytes": (sz, [i64, i64, i64]),
    "pb200_mesh_simplify": (i32, [i32, f32, i64, i64, i64, i64, vp, vp, vp, vp, vp, vp, vp, vp, vp, vp, vp, vp, vp, vp, vp,
                                  vp, sz, vp]),
    "pb200_combine_clusters": (i32, [i64, i64, vp, vp, vp, vp, vp, vp, vp, vp, sz, vp]),
    "pb200_rows_pointwise_forward": (i32, [i64, i32, i32, vp, vp, vp, i32, vp, i32, vp, sz, vp]),
    "pb200_masked_rows_matmul_workspace_bytes": (sz, [i32, i32]),
    "pb200_masked_rows_matmul": (i32, [i64, i32, i32, vp, vp, vp, vp, vp, i32, vp, sz, vp]),
    "pb200_rows_contract_workspace_bytes": (sz, [i64, i32, i32]),
    "pb200_rows_contract": (i32, [i64, i32, i32, vp, vp, vp, vp, i32, vp, sz, vp]),
    "pb200_sph_harm_coeff": (i32, [i64, i32, vp, vp, vp]),
    "pb200_triangle_geometry": (i32, [i64, i64, i32, vp, vp, vp, vp]),
    "pb200_expand_rows_forward": (i32, [i64, i64, i32, vp, vp, vp, vp]),
    "pb200_expand_rows_backward": (i32, [i64, i64, i32, vp, vp, vp, vp]),
    "pb200_face_mean_rows": (i32, [i64, i64, i32, vp, vp, vp, vp]),
    "pb200_face_mean_sph_harm": (i32, [i64, i64, i32, vp, vp, vp, vp]),
}

for _name, (_res, _args) in SIGNATURES.items():
    _fn = getattr(_lib, _name)      # AttributeError here = the library lacks a declared symbol
    _fn.restype = _res
    _fn.argtypes = _args


def raw(name: str):
    return getattr(_lib, name)


def last_error() -> str:
    return _lib.pb200_last_error().decode("utf-8", "replace")


def call(name: str, *args) -> None:
    """Call a status-returning entry point; raise RuntimeError with the library's message."""
    rc = getattr(_lib, name)(*args)
    if rc != OK:
        raise RuntimeError(f"{name} failed ({rc}): {last_error()}")


def query(name: str, *args) -> int:
    return int(getattr(_lib, name)(*args))


def launch_count() -> int:
    return int(_lib.pb200_launch_count())


def prof_enable(on: bool) -> None:
    _lib.pb200_prof_enable(1 if on else 0)


def prof_reset() -> None:
    _lib.pb200_prof_reset()


def prof_read(cap: int = 64):
    """[(kernel name, launches, total ms)] sorted by total time (synchronises the events)."""
    buf = (ProfRecord * cap)()
    n = _lib.pb200_prof_read(buf, cap)
    return [(buf[i].name.decode(), int(buf[i].launches), float(buf[i].total_ms)) for i in range(min(n, cap))]


def async_error() -> int:
    """0, or the code of the tensor-core kernel that gave up on the current device (after a sync)."""
    return int(_lib.pb200_async_error())


def clear_async_error() -> None:
    _lib.pb200_clear_async_error()
