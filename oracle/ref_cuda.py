"""ctypes doorway to oracle/_ref/libref_mesh_conv3d.so: the reference's own, unmodified
CUDA kernels (compiled for sm_100a by oracle/Makefile, target `ref`), called on CUDA torch
tensors.  TEST INFRASTRUCTURE ONLY; used as the live parity checker on a GPU and to make
the fixtures under tests/golden/.  Output allocation follows the reference binding
(picasso/mesh/pi_modules/source/mesh_conv3d.cpp:67,112-113,147,180-181,222,261-262):
zero-initialised, dtype and device of `input`.

The reference kernels read nfCount[vtMap[v]] before testing vtMap[v] >= 0
(mesh_conv3d_gpu.cu:324-325), an out-of-bounds read when vtMap holds -1; callers here must
pass a vtMap without negative entries."""
from __future__ import annotations

import ctypes as C
import os

import torch

_HERE = os.path.dirname(os.path.abspath(__file__))
_PATH = os.path.join(_HERE, "_ref", "libref_mesh_conv3d.so")
_LIB = None


def available() -> bool:
    return os.path.exists(_PATH) and torch.cuda.is_available()


def lib():
    global _LIB
    if _LIB is None:
        _LIB = C.CDLL(_PATH)
    return _LIB


def _p(t):
    assert t.is_cuda and t.is_contiguous()
    return C.c_void_p(t.data_ptr())


def _chk(code):
    if code != 0:
        raise RuntimeError(f"reference CUDA op failed with cudaError {code}")


def _sync_in():
    torch.cuda.synchronize()   # the reference uses the legacy default stream


def v2f_forward(inp, filt, face):
    _sync_in()
    _, Cc, r = filt.shape
    out = torch.zeros(face.shape[0], Cc * r, dtype=inp.dtype, device=inp.device)
    _chk(lib().ref_v2f_forward(face.shape[0], Cc, r, _p(face), _p(inp), _p(filt), _p(out)))
    return out


def v2f_backward(gout, inp, filt, face):
    _sync_in()
    _, Cc, r = filt.shape
    gin, gf = torch.zeros_like(inp), torch.zeros_like(filt)
    _chk(lib().ref_v2f_backward(face.shape[0], Cc, r, _p(face), _p(inp), _p(filt), _p(gout), _p(gin), _p(gf)))
    return gin, gf


def f2v_forward(inp, filt, coeff, face, nf_count, vt_map):
    assert int(vt_map.min()) >= 0, "reference kernel reads out of bounds for negative vtMap"
    _sync_in()
    K, Cc, r = filt.shape
    out = torch.zeros(nf_count.shape[0], Cc * r, dtype=inp.dtype, device=inp.device)
    _chk(lib().ref_f2v_forward(face.shape[0], Cc, r, K, _p(vt_map), _p(nf_count), _p(face), _p(coeff),
                               _p(inp), _p(filt), _p(out)))
    return out


def f2v_backward(gout, inp, filt, coeff, face, nf_count, vt_map):
    assert int(vt_map.min()) >= 0, "reference kernel reads out of bounds for negative vtMap"
    _sync_in()
    K, Cc, r = filt.shape
    gin, gf = torch.zeros_like(inp), torch.zeros_like(filt)
    _chk(lib().ref_f2v_backward(face.shape[0], Cc, r, K, _p(vt_map), _p(nf_count), _p(face), _p(coeff),
                                _p(inp), _p(filt), _p(gout), _p(gin), _p(gf)))
    return gin, gf


def f2f_forward(inp, filt, bary, cum):
    _sync_in()
    Cout, Cin, F = filt.shape
    out = torch.zeros(cum.shape[0], Cout, dtype=inp.dtype, device=inp.device)
    _chk(lib().ref_f2f_forward(cum.shape[0], F, Cin, Cout, _p(cum), _p(bary), _p(inp), _p(filt), _p(out)))
    return out


def f2f_backward(gout, inp, filt, bary, cum):
    _sync_in()
    Cout, Cin, F = filt.shape
    gin, gf = torch.zeros_like(inp), torch.zeros_like(filt)
    _chk(lib().ref_f2f_backward(cum.shape[0], F, Cin, Cout, _p(cum), _p(bary), _p(inp), _p(filt), _p(gout),
                                _p(gin), _p(gf)))
    return gin, gf


def count_vertex_adjface(face, vt_map, nv_out):
    _sync_in()
    out = torch.zeros(nv_out, dtype=torch.int32, device=face.device)
    _chk(lib().ref_count_vertex_adjface(face.shape[0], _p(face), _p(vt_map), _p(out)))
    return out


# ---- mesh pool / unpool (mesh_pool3d_gpu.cu, mesh_unpool3d_gpu.cu); output allocation as the
# bindings do it (mesh_pool3d.cpp, mesh_unpool3d.cpp: zero-initialised)
def max_pool_forward(inp, vt_replace, vt_map, nv_out):
    _sync_in()
    C = inp.shape[1]
    out = torch.zeros(nv_out, C, dtype=inp.dtype, device=inp.device)
    idx = torch.zeros(nv_out, C, dtype=torch.int32, device=inp.device)
    _chk(lib().ref_max_pool_forward(inp.shape[0], C, _p(vt_replace), _p(vt_map), _p(inp), _p(out), _p(idx)))
    return out, idx


def max_pool_backward(gout, nv_in, max_index):
    _sync_in()
    C = gout.shape[1]
    gin = torch.zeros(nv_in, C, dtype=gout.dtype, device=gout.device)
    _chk(lib().ref_max_pool_backward(gout.shape[0], C, _p(max_index), _p(gout), _p(gin)))
    return gin


def avg_pool_forward(inp, vt_replace, vt_map, nv_out):
    _sync_in()
    C = inp.shape[1]
    out = torch.zeros(nv_out, C, dtype=inp.dtype, device=inp.device)
    _chk(lib().ref_avg_pool_forward(inp.shape[0], C, _p(vt_replace), _p(vt_map), _p(inp), _p(out)))
    return out


def avg_pool_backward(gout, vt_replace, vt_map):
    _sync_in()
    C = gout.shape[1]
    gin = torch.zeros(vt_replace.shape[0], C, dtype=gout.dtype, device=gout.device)
    _chk(lib().ref_avg_pool_backward(vt_replace.shape[0], C, _p(vt_replace), _p(vt_map), _p(gout), _p(gin)))
    return gin


def unpool_forward(inp, vt_replace, vt_map):
    _sync_in()
    C = inp.shape[1]
    out = torch.zeros(vt_map.shape[0], C, dtype=inp.dtype, device=inp.device)
    _chk(lib().ref_unpool_forward(inp.shape[0], C, vt_map.shape[0], _p(vt_replace), _p(vt_map), _p(inp), _p(out)))
    return out


def unpool_backward(gout, nv_coarse, vt_replace, vt_map):
    _sync_in()
    C = gout.shape[1]
    gin = torch.zeros(nv_coarse, C, dtype=gout.dtype, device=gout.device)
    _chk(lib().ref_unpool_backward(nv_coarse, C, vt_map.shape[0], _p(vt_replace), _p(vt_map), _p(gout), _p(gin)))
    return gin


# ---- point-cloud depthwise convolution (pcloud_conv3d_gpu.cu); bin_coeff None = hard assignment
def pcloud_forward(inp, filt, nn_count, nn_index, bin_index, bin_coeff=None):
    _sync_in()
    F, Cc, r = filt.shape
    T = 1 if bin_coeff is None else bin_index.shape[1]
    out = torch.zeros(nn_count.shape[0], Cc * r, dtype=inp.dtype, device=inp.device)
    _chk(lib().ref_pcloud_forward(inp.shape[0], nn_count.shape[0], nn_index.shape[0], F, Cc, r, T, _p(nn_count), _p(nn_index),
                                  _p(bin_index), None if bin_coeff is None else _p(bin_coeff), _p(inp), _p(filt), _p(out)))
    return out


def pcloud_backward(gout, inp, filt, nn_count, nn_index, bin_index, bin_coeff=None):
    _sync_in()
    F, Cc, r = filt.shape
    T = 1 if bin_coeff is None else bin_index.shape[1]
    gin, gf = torch.zeros_like(inp), torch.zeros_like(filt)
    _chk(lib().ref_pcloud_backward(inp.shape[0], nn_count.shape[0], nn_index.shape[0], F, Cc, r, T, _p(nn_count),
                                   _p(nn_index), _p(bin_index), None if bin_coeff is None else _p(bin_coeff), _p(inp),
                                   _p(filt), _p(gout), _p(gin), _p(gf)))
    return gin, gf


def mesh_simplify(vertex, face, geometry, nv_cum, mf_cum, nv2remove, use_area=True, wgt_bnd=5.0):
    """One pass of the reference's decimation (decimate_gpu.cu:618-747; outputs allocated as
    decimate.cpp:57-63 does).  The reference keeps a per-vertex array on the host stack: small meshes only."""
    assert vertex.shape[0] <= 200_000
    _sync_in()
    Nv, D = vertex.shape
    Nf, B = face.shape[0], nv_cum.shape[0]
    dev = vertex.device
    out = dict(vertexOut=torch.zeros(Nv, D, dtype=torch.float32, device=dev),
               faceOut=torch.zeros(Nf, 3, dtype=torch.int32, device=dev),
               isDegenerate=torch.zeros(Nf, dtype=torch.bool, device=dev),
               vtReplace=torch.zeros(Nv, dtype=torch.int32, device=dev), vtMap=torch.zeros(Nv, dtype=torch.int32, device=dev),
               nvOut=torch.zeros(B, dtype=torch.int32, device=dev), mfOut=torch.zeros(B, dtype=torch.int32, device=dev))
    _chk(lib().ref_mesh_simplify(int(bool(use_area)), C.c_float(float(wgt_bnd)), B, D, Nv, Nf, _p(nv_cum), _p(mf_cum),
                                 _p(nv2remove), _p(vertex), _p(face), _p(geometry), _p(out["nvOut"]), _p(out["mfOut"]),
                                 _p(out["vertexOut"]), _p(out["faceOut"]), _p(out["vtReplace"]), _p(out["vtMap"]),
                                 _p(out["isDegenerate"])))
    return out


def combine_clusters(rep_a, map_a, rep_b, map_b):
    _sync_in()
    rep_out, map_out = torch.zeros_like(rep_a), torch.zeros_like(map_a)
    _chk(lib().ref_combine_clusters(rep_a.shape[0], rep_b.shape[0], _p(rep_a), _p(map_a), _p(rep_b), _p(map_b),
                                    _p(rep_out), _p(map_out)))
    return rep_out, map_out
