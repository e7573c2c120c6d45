"""The two per-level helpers of the reference's picasso/mesh/pi_modules/decimate.py that
the convolutions depend on: triangle geometry (decimate.py:70-85) and the adjacent-face
count (decimate.py:88-93).  Mesh decimation itself is not part of this package."""
from __future__ import annotations

import torch

from ... import _lib
from ...topology import ptr, stream_ptr


def compute_triangle_geometry_(vertex, face):
    '''(Nf, 5) float32: unit normal, plane intercept d, area of every facet.'''
    if not (vertex.is_cuda and face.is_cuda):
        raise RuntimeError("vertex and face must be CUDA tensors")
    if vertex.dtype != torch.float32 or vertex.dim() != 2 or vertex.shape[1] < 3:
        raise RuntimeError("vertex must be a float32 (Nv, >=3) tensor")
    if face.dtype != torch.int32 or face.dim() != 2 or face.shape[1] != 3:
        raise RuntimeError("face must be an int32 (Nf, 3) tensor")
    vertex = vertex.contiguous()
    face = face.contiguous()
    dev = vertex.device
    with torch.cuda.device(dev):
        geom = torch.empty(face.shape[0], 5, dtype=torch.float32, device=dev)
        _lib.call("pb200_triangle_geometry", face.shape[0], vertex.shape[0], vertex.shape[1], ptr(vertex), ptr(face),
                  ptr(geom), stream_ptr(dev))
    return geom


def count_vertex_adjface_(face, vtMap, vertexOut):
    '''(NvOut,) int32: number of adjacent faces of every output vertex {vtMap[i] | vtMap[i] >= 0}.'''
    for t, name in ((face, "faceIn"), (vtMap, "vtMap"), (vertexOut, "vtOut")):
        if not t.is_cuda:
            raise RuntimeError(f"{name} must be a CUDA tensor")
        if not t.is_contiguous():
            raise RuntimeError(f"{name} must be contiguous")
    if face.dim() != 2 or face.shape[1] != 3:
        raise RuntimeError("The shape of input face should be (NfIn, 3)).")
    if vertexOut.dim() != 2:
        raise RuntimeError("The shape of vertexOut should be (NvOut,3).")
    if face.dtype != torch.int32 or vtMap.dtype != torch.int32 or vtMap.dim() != 1:
        raise RuntimeError("face and vtMap must be int32")
    dev = face.device
    nv_out = vertexOut.shape[0]
    with torch.cuda.device(dev):
        nf_count = torch.empty(nv_out, dtype=torch.int32, device=dev)
        _lib.call("pb200_count_vertex_adjface", face.shape[0], vtMap.shape[0], nv_out, ptr(face), ptr(vtMap),
                  ptr(nf_count), stream_ptr(dev))
    return nf_count
