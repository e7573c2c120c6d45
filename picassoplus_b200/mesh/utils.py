"""Per-level helpers with the reference's names (picasso/mesh/utils.py:15-24)."""
from .pi_modules.decimate import compute_triangle_geometry_, count_vertex_adjface_


def compute_triangle_geometry(vertex, face):
    return compute_triangle_geometry_(vertex, face)


def count_vertex_adjface(face, vtMap, vertexOut):
    return count_vertex_adjface_(face, vtMap, vertexOut[:, :3].contiguous())
