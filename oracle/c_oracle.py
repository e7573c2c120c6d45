"""ctypes doorway to oracle/_build/liboracle.so (the plain-C restatement in mesh_oracle.c).
TEST INFRASTRUCTURE ONLY.  Arguments and results are numpy arrays; `acc64=True` selects the
double-accumulator build of the same loops (the arbiter)."""
from __future__ import annotations

import ctypes as C
import os
import subprocess

import numpy as np

_HERE = os.path.dirname(os.path.abspath(__file__))
_LIB = None


def build() -> str:
    subprocess.run(["make", "-s", "-C", _HERE, "oracle"], check=True)
    return os.path.join(_HERE, "_build", "liboracle.so")


def lib():
    global _LIB
    if _LIB is None:
        path = os.path.join(_HERE, "_build", "liboracle.so")
        if not os.path.exists(path):
            build()
        _LIB = C.CDLL(path)
    return _LIB


C_int = C.c_int


def _p(a):
    return a.ctypes.data_as(C.c_void_p)


def _f32(a):
    return np.ascontiguousarray(a, dtype=np.float32)


def _i32(a):
    return np.ascontiguousarray(a, dtype=np.int32)


def _fn(name, acc64):
    return getattr(lib(), name + ("_f64acc" if acc64 else ""))


def _scratch(n, acc64):
    return np.zeros(max(int(n), 1), dtype=np.float64 if acc64 else np.float32)


def v2f_forward(inp, filt, face, acc64=False):
    inp, filt, face = _f32(inp), _f32(filt), _i32(face)
    _, Cc, r = filt.shape
    out = np.zeros((face.shape[0], Cc * r), np.float32)
    _fn("oracle_v2f_forward", acc64)(C.c_int(face.shape[0]), C.c_int(Cc), C.c_int(r), _p(face), _p(inp),
                                     _p(filt), _p(out))
    return out


def v2f_backward(gout, inp, filt, face, acc64=False):
    gout, inp, filt, face = _f32(gout), _f32(inp), _f32(filt), _i32(face)
    _, Cc, r = filt.shape
    gin, gf = np.zeros_like(inp), np.zeros_like(filt)
    s = _scratch(inp.size + filt.size, acc64)
    _fn("oracle_v2f_backward", acc64)(C.c_int(face.shape[0]), C.c_int(inp.shape[0]), C.c_int(Cc), C.c_int(r),
                                      _p(face), _p(inp), _p(filt), _p(gout), _p(gin), _p(gf), _p(s))
    return gin, gf


def f2v_forward(inp, filt, coeff, face, nf_count, vt_map, acc64=False):
    inp, filt, coeff = _f32(inp), _f32(filt), _f32(coeff)
    face, nf_count, vt_map = _i32(face), _i32(nf_count), _i32(vt_map)
    K, Cc, r = filt.shape
    nvo = nf_count.shape[0]
    out = np.zeros((nvo, Cc * r), np.float32)
    s = _scratch(out.size, acc64)
    _fn("oracle_f2v_forward", acc64)(C.c_int(face.shape[0]), C.c_int(nvo), C.c_int(Cc), C.c_int(r), C.c_int(K),
                                     _p(vt_map), _p(nf_count), _p(face), _p(coeff), _p(inp), _p(filt),
                                     _p(out), _p(s))
    return out


def f2v_backward(gout, inp, filt, coeff, face, nf_count, vt_map, acc64=False):
    gout, inp, filt, coeff = _f32(gout), _f32(inp), _f32(filt), _f32(coeff)
    face, nf_count, vt_map = _i32(face), _i32(nf_count), _i32(vt_map)
    K, Cc, r = filt.shape
    gin, gf = np.zeros_like(inp), np.zeros_like(filt)
    s = _scratch(inp.size + filt.size, acc64)
    _fn("oracle_f2v_backward", acc64)(C.c_int(face.shape[0]), C.c_int(Cc), C.c_int(r), C.c_int(K), _p(vt_map),
                                      _p(nf_count), _p(face), _p(coeff), _p(inp), _p(filt), _p(gout),
                                      _p(gin), _p(gf), _p(s))
    return gin, gf


def f2f_forward(inp, filt, bary, cum, acc64=False):
    inp, filt, bary, cum = _f32(inp), _f32(filt), _f32(bary), _i32(cum)
    Cout, Cin, F = filt.shape
    out = np.zeros((cum.shape[0], Cout), np.float32)
    _fn("oracle_f2f_forward", acc64)(C.c_int(cum.shape[0]), C.c_int(F), C.c_int(Cin), C.c_int(Cout), _p(cum),
                                     _p(bary), _p(inp), _p(filt), _p(out))
    return out


def f2f_backward(gout, inp, filt, bary, cum, acc64=False):
    gout, inp, filt, bary, cum = _f32(gout), _f32(inp), _f32(filt), _f32(bary), _i32(cum)
    Cout, Cin, F = filt.shape
    gin, gf = np.zeros_like(inp), np.zeros_like(filt)
    s = _scratch(inp.size + filt.size, acc64)
    _fn("oracle_f2f_backward", acc64)(C.c_int(cum.shape[0]), C.c_int(inp.shape[0]), C.c_int(F), C.c_int(Cin),
                                      C.c_int(Cout), _p(cum), _p(bary), _p(inp), _p(filt), _p(gout),
                                      _p(gin), _p(gf), _p(s))
    return gin, gf


def count_vertex_adjface(face, vt_map, nv_out):
    face, vt_map = _i32(face), _i32(vt_map)
    out = np.zeros(nv_out, np.int32)
    lib().oracle_count_vertex_adjface(C.c_int(face.shape[0]), _p(face), _p(vt_map), _p(out))
    return out


def sph_harm_coeff(L, xyz, consts):
    xyz, consts = _f32(xyz), _f32(consts)
    out = np.zeros((xyz.shape[0], (L + 1) ** 2), np.float32)
    lib().oracle_sph_harm_coeff(C.c_int(xyz.shape[0]), C.c_int(L), _p(xyz), _p(consts), _p(out))
    return out


def triangle_geometry(vertex, face):
    vertex, face = _f32(vertex), _i32(face)
    out = np.zeros((face.shape[0], 5), np.float32)
    lib().oracle_triangle_geometry(C.c_int(face.shape[0]), C.c_int(vertex.shape[1]), _p(vertex), _p(face), _p(out))
    return out


def max_pool_forward(inp, vt_replace, vt_map, nv_out):
    inp, vt_replace, vt_map = _f32(inp), _i32(vt_replace), _i32(vt_map)
    C = inp.shape[1]
    out, idx = np.zeros((nv_out, C), np.float32), np.zeros((nv_out, C), np.int32)
    lib().oracle_max_pool_forward(C_int(inp.shape[0]), C_int(nv_out), C_int(C), _p(vt_replace), _p(vt_map), _p(inp),
                                  _p(out), _p(idx))
    return out, idx


def max_pool_backward(gout, nv_in, max_index):
    gout, max_index = _f32(gout), _i32(max_index)
    gin = np.zeros((nv_in, gout.shape[1]), np.float32)
    lib().oracle_max_pool_backward(C_int(nv_in), C_int(gout.shape[0]), C_int(gout.shape[1]), _p(max_index), _p(gout),
                                   _p(gin))
    return gin


def avg_pool_forward(inp, vt_replace, vt_map, nv_out):
    inp, vt_replace, vt_map = _f32(inp), _i32(vt_replace), _i32(vt_map)
    out = np.zeros((nv_out, inp.shape[1]), np.float32)
    lib().oracle_avg_pool_forward(C_int(inp.shape[0]), C_int(nv_out), C_int(inp.shape[1]), _p(vt_replace), _p(vt_map),
                                  _p(inp), _p(out))
    return out


def avg_pool_backward(gout, vt_replace, vt_map):
    gout, vt_replace, vt_map = _f32(gout), _i32(vt_replace), _i32(vt_map)
    gin = np.zeros((vt_replace.shape[0], gout.shape[1]), np.float32)
    lib().oracle_avg_pool_backward(C_int(vt_replace.shape[0]), C_int(gout.shape[1]), _p(vt_replace), _p(vt_map),
                                   _p(gout), _p(gin))
    return gin


def unpool_forward(inp, vt_replace, vt_map):
    inp, vt_replace, vt_map = _f32(inp), _i32(vt_replace), _i32(vt_map)
    out = np.zeros((vt_map.shape[0], inp.shape[1]), np.float32)
    lib().oracle_unpool_forward(C_int(vt_map.shape[0]), C_int(inp.shape[1]), _p(vt_replace), _p(vt_map), _p(inp), _p(out))
    return out


def unpool_backward(gout, nv_coarse, vt_replace, vt_map):
    gout, vt_replace, vt_map = _f32(gout), _i32(vt_replace), _i32(vt_map)
    gin = np.zeros((nv_coarse, gout.shape[1]), np.float32)
    lib().oracle_unpool_backward(C_int(vt_map.shape[0]), C_int(nv_coarse), C_int(gout.shape[1]), _p(vt_replace),
                                 _p(vt_map), _p(gout), _p(gin))
    return gin


def pcloud_forward(inp, filt, nn_count, nn_index, bin_index, bin_coeff=None):
    inp, filt, nn_count, nn_index, bin_index = _f32(inp), _f32(filt), _i32(nn_count), _i32(nn_index), _i32(bin_index)
    F, Cc, r = filt.shape
    T = 1 if bin_coeff is None else bin_index.shape[1]
    coeff = None if bin_coeff is None else _f32(bin_coeff)
    out = np.zeros((nn_count.shape[0], Cc * r), np.float32)
    lib().oracle_pcloud_forward(C_int(nn_count.shape[0]), C_int(nn_index.shape[0]), C_int(Cc), C_int(r), C_int(T),
                                _p(nn_count), _p(nn_index), _p(bin_index), None if coeff is None else _p(coeff), _p(inp),
                                _p(filt), _p(out))
    return out


def pcloud_backward(gout, inp, filt, nn_count, nn_index, bin_index, bin_coeff=None):
    gout, inp, filt = _f32(gout), _f32(inp), _f32(filt)
    nn_count, nn_index, bin_index = _i32(nn_count), _i32(nn_index), _i32(bin_index)
    F, Cc, r = filt.shape
    T = 1 if bin_coeff is None else bin_index.shape[1]
    coeff = None if bin_coeff is None else _f32(bin_coeff)
    gin, gf = np.zeros_like(inp), np.zeros_like(filt)
    lib().oracle_pcloud_backward(C_int(inp.shape[0]), C_int(nn_index.shape[0]), C_int(F), C_int(Cc), C_int(r), C_int(T),
                                 _p(nn_count), _p(nn_index), _p(bin_index), None if coeff is None else _p(coeff), _p(inp),
                                 _p(filt), _p(gout), _p(gin), _p(gf))
    return gin, gf


def mesh_simplify(vertex, face, geometry, nv_cum, mf_cum, nv2remove, use_area=True, wgt_bnd=5.0):
    """One decimation pass (decimate_oracle.c).  nv_cum / mf_cum are the running totals per sample.
    Returns a dict with the reference's seven outputs plus the candidate costs in edge order."""
    vertex, face, geometry = _f32(vertex), _i32(face), _f32(geometry)
    nv_cum, mf_cum, nv2remove = _i32(nv_cum), _i32(mf_cum), _i32(nv2remove)
    Nv, D = vertex.shape
    Nf, B = face.shape[0], nv_cum.shape[0]
    out = dict(vertexOut=np.zeros((Nv, D), np.float32), faceOut=np.zeros((Nf, 3), np.int32),
               isDegenerate=np.zeros(Nf, np.uint8), vtReplace=np.zeros(Nv, np.int32), vtMap=np.zeros(Nv, np.int32),
               nvOut=np.zeros(B, np.int32), mfOut=np.zeros(B, np.int32))
    cost = np.zeros(max(3 * Nf, 1), np.float32)
    fn = lib().oracle_mesh_simplify
    fn.restype = C.c_int
    nu = fn(C.c_int(int(bool(use_area))), C.c_float(float(wgt_bnd)), C.c_int(B), C.c_int(D), C.c_int(Nv), C.c_int(Nf),
            _p(nv_cum), _p(mf_cum), _p(nv2remove), _p(vertex), _p(face), _p(geometry), _p(out["nvOut"]), _p(out["mfOut"]),
            _p(out["vertexOut"]), _p(out["faceOut"]), _p(out["vtReplace"]), _p(out["vtMap"]), _p(out["isDegenerate"]),
            _p(cost))
    if nu < 0:
        raise MemoryError("oracle_mesh_simplify")
    out["isDegenerate"] = out["isDegenerate"].astype(bool)
    out["edgeCost"] = cost[:nu]
    return out


def combine_clusters(rep_a, map_a, rep_b, map_b):
    rep_a, map_a, rep_b, map_b = _i32(rep_a), _i32(map_a), _i32(rep_b), _i32(map_b)
    rep_out, map_out = np.zeros_like(rep_a), np.zeros_like(map_a)
    fn = lib().oracle_combine_clusters
    fn.restype = None
    fn(C.c_int(rep_a.shape[0]), C.c_int(rep_b.shape[0]), _p(rep_a), _p(map_a), _p(rep_b), _p(map_b), _p(rep_out),
       _p(map_out))
    return rep_out, map_out
