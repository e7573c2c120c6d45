"""Mirror of the reference's picasso/mesh/pi_modules/decimate.py: quadric-error mesh decimation
(`mesh_decimation_`, decimate.py:5-48), cluster merge (`combine_clusters_`, decimate.py:51-64),
triangle geometry (decimate.py:70-85) and the adjacent-face count (decimate.py:88-93).  `simplify`
and `combine_clusters` stand where the reference's extension module `mesh_decimation` exports them
(decimate.cpp:165-169)."""
from __future__ import annotations

import ctypes

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


def _check(t, name, dims, dtype):
    if not t.is_cuda:
        raise RuntimeError(f"{name} must be a CUDA tensor")
    if not t.is_contiguous():
        raise RuntimeError(f"{name} must be contiguous")
    if t.dim() != dims:
        raise RuntimeError(f"{name} must have dimension of {dims}")
    if t.dtype != dtype:
        raise RuntimeError(f"{name} must be {dtype}")


def simplify(vertexIn, faceIn, planeIn, nvIn, mfIn, nv2Remove, useArea, wgtBnd, return_info=False):
    '''One decimation pass; arguments, checks and the seven results as the reference binding
    (decimate.cpp:22-99): nvIn / mfIn are the running totals per sample.
    Returns vertexOut, faceOut, isDegenerate, vtReplace, vtMap, nvOut, mfOut; with return_info=True also
    (the library's counters, the cost of every distinct edge in (lower vertex, higher vertex) order).'''
    _check(vertexIn, "vertexIn", 2, torch.float32)
    _check(faceIn, "faceIn", 2, torch.int32)
    _check(planeIn, "planeIn", 2, torch.float32)
    _check(nvIn, "nvIn", 1, torch.int32)
    _check(mfIn, "mfIn", 1, torch.int32)
    _check(nv2Remove, "nv2Remove", 1, torch.int32)
    if vertexIn.shape[1] < 3:
        raise RuntimeError("The shape of input vertex should be (Nv, 3+)).")
    if faceIn.shape[1] != 3:
        raise RuntimeError("The shape of input face should be (Nf, 3)).")
    Nv, D = vertexIn.shape
    Nf, B = faceIn.shape[0], nvIn.shape[0]
    if planeIn.shape[0] != Nf or planeIn.shape[1] != 5:
        raise RuntimeError("The shape of input face normals should be (Nf, 5)).")
    if mfIn.shape[0] != B or nv2Remove.shape[0] != B:
        raise RuntimeError("nvIn, mfIn and nv2Remove must have one entry per sample")
    dev = vertexIn.device
    with torch.cuda.device(dev):
        i32 = dict(dtype=torch.int32, device=dev)
        vertexOut = torch.empty(Nv, D, dtype=torch.float32, device=dev)
        faceOut = torch.empty(Nf, 3, **i32)
        isDegenerate = torch.empty(Nf, dtype=torch.bool, device=dev)
        vtReplace = torch.empty(Nv, **i32)
        vtMap = torch.empty(Nv, **i32)
        nvOut = torch.empty(B, **i32)
        mfOut = torch.empty(B, **i32)
        ws_bytes = _lib.query("pb200_mesh_simplify_workspace_bytes", B, Nv, Nf)
        ws = torch.empty(ws_bytes, dtype=torch.uint8, device=dev)
        info = (ctypes.c_int64 * 4)()
        cost = torch.empty(max(3 * Nf, 1), dtype=torch.float32, device=dev) if return_info else None
        _lib.call("pb200_mesh_simplify", int(bool(useArea)), float(wgtBnd), B, D, Nv, Nf, ptr(nvIn), ptr(mfIn),
                  ptr(nv2Remove), ptr(vertexIn), ptr(faceIn), ptr(planeIn), ptr(nvOut), ptr(mfOut), ptr(vertexOut),
                  ptr(faceOut), ptr(vtReplace), ptr(vtMap), ptr(isDegenerate), ptr(cost) if return_info else None, info, ptr(ws),
                  ws_bytes,
                  stream_ptr(dev))
    if return_info:
        return (vertexOut, faceOut, isDegenerate, vtReplace, vtMap, nvOut, mfOut), list(info), cost[:info[0]]
    return vertexOut, faceOut, isDegenerate, vtReplace, vtMap, nvOut, mfOut


def combine_clusters(repA, mapA, repB, mapB):
    '''decimate.cpp:102-137: returns (repOut, mapOut) over the vertices of A.'''
    for t, name in ((repA, "repA"), (mapA, "mapA"), (repB, "repB"), (mapB, "mapB")):
        _check(t, name, 1, torch.int32)
    if repA.shape[0] != mapA.shape[0]:
        raise RuntimeError("The shape of repA and mapA should be identical.")
    if repB.shape[0] != mapB.shape[0]:
        raise RuntimeError("The shape of repB and mapB should be identical.")
    dev = repA.device
    nvA, nvB = repA.shape[0], repB.shape[0]
    with torch.cuda.device(dev):
        repOut, mapOut = torch.empty_like(repA), torch.empty_like(mapA)
        status = torch.empty(1, dtype=torch.int32, device=dev)
        ws = torch.empty(nvB + 1, dtype=torch.int32, device=dev)
        _lib.call("pb200_combine_clusters", nvA, nvB, ptr(repA), ptr(mapA), ptr(repB), ptr(mapB), ptr(repOut),
                  ptr(mapOut), ptr(status), ptr(ws), ws.numel() * 4, stream_ptr(dev))
    return repOut, mapOut


def combine_clusters_(repA, mapA, repB, mapB):
    '''decimate.py:51-64'''
    return combine_clusters(repA, mapA, repB, mapB)


def mesh_decimation_(vertexIn, faceIn, geometryIn, nvIn, mfIn, nvOut, useArea=True, wgtBnd=5):
    '''Decimates every sample of the batch to nvOut vertices (decimate.py:5-48): passes of `simplify`
    until every sample has shed its vertices, clusters merged across the passes.
    Returns vertexOut, faceOut, geometryOut, nvOut, mfOut, vtReplace, vtMap.'''
    nv2Remove = nvIn - nvOut
    repIn = torch.zeros(vertexIn.shape[0], dtype=torch.int32, device=vertexIn.device)
    mapIn = torch.arange(vertexIn.shape[0], dtype=torch.int32, device=vertexIn.device)
    while bool(torch.any(nv2Remove > 0)):
        nvIn_cumsum = torch.cumsum(nvIn, dim=-1, dtype=torch.int32)
        mfIn_cumsum = torch.cumsum(mfIn, dim=-1, dtype=torch.int32)
        vertexOut, faceOut, isDegenerate, repOut, mapOut, nvOut, mfOut = simplify(
            vertexIn.contiguous(), faceIn.contiguous(), geometryIn.contiguous(), nvIn_cumsum, mfIn_cumsum,
            nv2Remove.to(torch.int32).contiguous(), useArea, wgtBnd)
        removed = nvIn - nvOut
        if not bool(torch.any(removed > 0)):
            break          # nothing left to contract (no candidate edges): the reference would loop forever
        faceIn = faceOut[~isDegenerate, :]
        vertexIn = vertexOut[mapOut >= 0, :]
        geometryIn = compute_triangle_geometry_(vertexIn, faceIn)
        nv2Remove = nv2Remove - removed
        repIn, mapIn = combine_clusters_(repIn, mapIn, repOut, mapOut)
        nvIn, mfIn = nvOut, mfOut
    return vertexIn, faceIn, geometryIn, nvIn, mfIn, repIn, mapIn
