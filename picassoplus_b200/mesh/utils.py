"""Per-level helpers with the reference's names (picasso/mesh/utils.py:8-58): decimation, triangle
geometry, adjacent-face count, cluster merge and the mesh hierarchy builder."""
import torch

from .pi_modules.decimate import (combine_clusters_, compute_triangle_geometry_, count_vertex_adjface_,
                                  mesh_decimation_)


def mesh_decimation(vertexIn, faceIn, geometryIn, nvIn, mfIn, nvSample, useArea=True, wgtBnd=1.):
    return mesh_decimation_(vertexIn, faceIn, geometryIn, nvIn, mfIn, nvSample, useArea=useArea, wgtBnd=wgtBnd)


def compute_triangle_geometry(vertex, face):
    return compute_triangle_geometry_(vertex, face)


def count_vertex_adjface(face, vtMap, vertexOut):
    return count_vertex_adjface_(face, vtMap, vertexOut[:, :3].contiguous())


def combine_clusters(rep_highRes, map_highRes, rep_lowRes, map_lowRes):
    return combine_clusters_(rep_highRes, map_highRes, rep_lowRes, map_lowRes)


class MeshHierarchy:
    """Levels of a batch of meshes by repeated decimation; same constructor forms and result as the
    reference's helper (picasso/mesh/utils.py:32-58):
      MeshHierarchy(nv_samples, useArea, wgtBnd)          level l keeps nv_samples[l] (a (B,) tensor) vertices per sample
      MeshHierarchy(stride, min_nvOut, useArea, wgtBnd)   level l keeps 1/stride[l] of the level before, at least min_nvOut[l]
    Calling it on (vertex, face, nv, mf) returns one tuple (vertex, face, geometry, nv, mf, vtReplace, vtMap)
    per level; the cluster arrays of a level are indexed by the vertices of the level before (None at level 0)."""

    def __init__(self, *params):
        if len(params) == 3:
            self.nv_samples, self.useArea, self.wgtBnd = params
            self.stride = self.min_nvOut = None
            self.Iters = len(self.nv_samples)
        elif len(params) == 4:
            self.stride, self.min_nvOut, self.useArea, self.wgtBnd = params
            self.nv_samples = None
            self.Iters = len(self.stride)
        else:
            raise ValueError("MeshHierarchy takes (nv_samples, useArea, wgtBnd) or (stride, min_nvOut, useArea, wgtBnd)")
        self.num_params = len(params)

    def _target(self, level, nv):
        """vertices per sample that level `level` + 1 keeps"""
        if self.nv_samples is not None:
            return self.nv_samples[level].to(nv.device)
        shrunk = (nv.to(torch.float) / float(self.stride[level])).to(torch.int)
        return torch.clip(shrunk, min=self.min_nvOut[level])

    def __call__(self, vertex_in, face_in, nv_in, mf_in):
        levels = [(vertex_in, face_in, compute_triangle_geometry(vertex_in, face_in), nv_in, mf_in, None, None)]
        for level in range(self.Iters):
            vertex, face, geometry, nv, mf = levels[-1][:5]
            levels.append(mesh_decimation(vertex, face, geometry, nv, mf, self._target(level, nv), self.useArea, self.wgtBnd))
        return levels
