"""Seeded synthetic meshes that stand in for the datasets the reference trains on.

Every generator is deterministic in its seed and runs on the CPU (numpy); batches follow
the reference's ragged-concatenation convention: vertices of all meshes stacked, faces
stacked with vertex ids offset so they are global in the batch, plus per-mesh counts
(reference: picasso/mesh/dataset_shape.py:43-58).
"""
from __future__ import annotations

import math
from dataclasses import dataclass
from typing import List, Sequence, Tuple

import numpy as np


# --------------------------------------------------------------------------- icosphere
def icosahedron() -> Tuple[np.ndarray, np.ndarray]:
    """The 12-vertex / 20-face regular icosahedron on the unit sphere."""
    t = (1.0 + math.sqrt(5.0)) / 2.0
    v = np.array(
        [[-1, t, 0], [1, t, 0], [-1, -t, 0], [1, -t, 0],
         [0, -1, t], [0, 1, t], [0, -1, -t], [0, 1, -t],
         [t, 0, -1], [t, 0, 1], [-t, 0, -1], [-t, 0, 1]], dtype=np.float64)
    v /= np.linalg.norm(v, axis=1, keepdims=True)
    f = np.array(
        [[0, 11, 5], [0, 5, 1], [0, 1, 7], [0, 7, 10], [0, 10, 11],
         [1, 5, 9], [5, 11, 4], [11, 10, 2], [10, 7, 6], [7, 1, 8],
         [3, 9, 4], [3, 4, 2], [3, 2, 6], [3, 6, 8], [3, 8, 9],
         [4, 9, 5], [2, 4, 11], [6, 2, 10], [8, 6, 7], [9, 8, 1]], dtype=np.int64)
    return v, f


def icosphere(level: int) -> Tuple[np.ndarray, np.ndarray]:
    """Subdivide the icosahedron `level` times (midpoint split, shared midpoints
    de-duplicated) and project to the unit sphere: V = 10*4^level + 2, F = 20*4^level."""
    v, f = icosahedron()
    for _ in range(level):
        nv = v.shape[0]
        e = np.concatenate([f[:, [0, 1]], f[:, [1, 2]], f[:, [2, 0]]], axis=0)
        e = np.sort(e, axis=1)
        key = e[:, 0] * nv + e[:, 1]
        uniq, inv = np.unique(key, return_inverse=True)
        mid = (v[uniq // nv] + v[uniq % nv]) * 0.5
        mid /= np.linalg.norm(mid, axis=1, keepdims=True)
        v = np.concatenate([v, mid], axis=0)
        nf = f.shape[0]
        m01 = nv + inv[:nf]
        m12 = nv + inv[nf:2 * nf]
        m20 = nv + inv[2 * nf:]
        f = np.concatenate([
            np.stack([f[:, 0], m01, m20], 1),
            np.stack([f[:, 1], m12, m01], 1),
            np.stack([f[:, 2], m20, m12], 1),
            np.stack([m01, m12, m20], 1)], axis=0)
    return v.astype(np.float32), f.astype(np.int32)


def random_rotation(rng: np.random.Generator) -> np.ndarray:
    """Uniform-ish rotation: QR of a 3x3 normal matrix with the determinant fixed to +1."""
    q, r = np.linalg.qr(rng.standard_normal((3, 3)))
    q = q * np.sign(np.diag(r))
    if np.linalg.det(q) < 0:
        q[:, 0] = -q[:, 0]
    return q


# ------------------------------------------------------------------------- heightfield
def _value_noise(n: int, rng: np.random.Generator, octaves: int = 4, amplitude: float = 0.5,
                 base_cells: int = 4) -> np.ndarray:
    """Fractal value noise on an n x n grid over [0,1]^2: per octave a random lattice,
    smoothstep-interpolated; amplitude halves and frequency doubles per octave."""
    xs = np.linspace(0.0, 1.0, n, dtype=np.float64)
    z = np.zeros((n, n), dtype=np.float64)
    amp = amplitude
    cells = base_cells
    for _ in range(octaves):
        lat = rng.uniform(-1.0, 1.0, size=(cells + 1, cells + 1))
        g = xs * cells
        i0 = np.minimum(g.astype(np.int64), cells - 1)
        t = g - i0
        s = t * t * (3.0 - 2.0 * t)
        a = lat[i0][:, i0]
        b = lat[i0 + 1][:, i0]
        c = lat[i0][:, i0 + 1]
        d = lat[i0 + 1][:, i0 + 1]
        sy = s[:, None]
        sx = s[None, :]
        z += amp * ((a * (1 - sy) + b * sy) * (1 - sx) + (c * (1 - sy) + d * sy) * sx)
        amp *= 0.5
        cells *= 2
    return z


def heightfield(n: int, seed: int, delete_frac: float = 0.10) -> Tuple[np.ndarray, np.ndarray]:
    """n x n vertex grid on [0,1]^2 with fractal-noise heights, two triangles per cell
    with a fixed diagonal, then each face deleted with probability `delete_frac`
    (vertices stay, so isolated / boundary vertices appear)."""
    rng = np.random.default_rng(seed)
    z = _value_noise(n, rng)
    ys, xs = np.meshgrid(np.linspace(0, 1, n), np.linspace(0, 1, n), indexing="ij")
    v = np.stack([xs, ys, z], axis=-1).reshape(-1, 3).astype(np.float32)
    idx = np.arange(n * n, dtype=np.int64).reshape(n, n)
    a = idx[:-1, :-1].ravel()
    b = idx[:-1, 1:].ravel()
    c = idx[1:, :-1].ravel()
    d = idx[1:, 1:].ravel()
    f = np.stack([np.stack([a, b, c], 1), np.stack([b, d, c], 1)], axis=1).reshape(-1, 3)
    keep = rng.random(f.shape[0]) >= delete_frac
    return v, f[keep].astype(np.int32)


def heightfield_hierarchy(n: int, seed: int, levels: int = 4, delete_frac: float = 0.10):
    """A heightfield mesh and `levels - 1` coarser versions of it, with the cluster encoding that
    mesh decimation produces (picasso/mesh/pi_modules/decimate.py:23-28), standing in for the
    reference's GPU decimation: level l+1 keeps every second grid vertex in both directions (face
    ratio about 0.25 per level: 1, 0.25, 0.0625, 0.016 over four levels); the up to four fine
    vertices of a 2x2 cell form one cluster whose representative is the kept vertex.  Returns
    [(vertex, face)] per level and [(vt_replace, vt_map)] per transition (arrays over the finer
    level's vertices).  Cells whose representative is vertex 0 stay singletons (a representative is
    named by its negated id, which vertex 0 does not have); their other vertices belong to no
    cluster, like the vertices decimation drops."""
    rng = np.random.default_rng(seed)
    z = _value_noise(n, rng)
    meshes, maps = [], []
    step, m = 1, n
    for lvl in range(levels):
        zi = z[::step, ::step]
        m = zi.shape[0]
        ys, xs = np.meshgrid(np.linspace(0, 1, n)[::step], np.linspace(0, 1, n)[::step], indexing="ij")
        v = np.stack([xs, ys, zi], axis=-1).reshape(-1, 3).astype(np.float32)
        idx = np.arange(m * m, dtype=np.int64).reshape(m, m)
        a, b, c, d = idx[:-1, :-1].ravel(), idx[:-1, 1:].ravel(), idx[1:, :-1].ravel(), idx[1:, 1:].ravel()
        f = np.stack([np.stack([a, b, c], 1), np.stack([b, d, c], 1)], axis=1).reshape(-1, 3)
        keep = rng.random(f.shape[0]) >= delete_frac
        meshes.append((v, f[keep].astype(np.int32)))
        if lvl + 1 < levels:
            mc = (m + 1) // 2                                   # coarse grid size
            ii, jj = np.meshgrid(np.arange(m), np.arange(m), indexing="ij")
            rep = ((ii // 2) * 2 * m + (jj // 2) * 2).ravel()   # fine id of the cell's kept vertex
            me = np.arange(m * m)
            is_rep = rep == me
            vt_map = np.full(m * m, -1, np.int32)
            vt_map[is_rep] = ((ii // 2) * mc + (jj // 2)).ravel()[is_rep]
            vt_replace = np.zeros(m * m, np.int32)
            member = (~is_rep) & (rep > 0)
            vt_replace[member] = -rep[member]
            np.add.at(vt_replace, rep[member], 1)
            maps.append((vt_replace, vt_map))
        step *= 2
    return meshes, maps


# ------------------------------------------------------------------------------ batches
@dataclass
class MeshBatch:
    vertex: np.ndarray   # (sum Nv, 3) float32
    face: np.ndarray     # (sum Nf, 3) int32, vertex ids global in the batch
    nv: np.ndarray       # (B,) int32 vertices per mesh
    mf: np.ndarray       # (B,) int32 faces per mesh

    @property
    def num_vertices(self) -> int:
        return int(self.vertex.shape[0])

    @property
    def num_faces(self) -> int:
        return int(self.face.shape[0])


def concat_meshes(meshes: Sequence[Tuple[np.ndarray, np.ndarray]]) -> MeshBatch:
    vs: List[np.ndarray] = []
    fs: List[np.ndarray] = []
    off = 0
    for v, f in meshes:
        vs.append(v.astype(np.float32))
        fs.append(f.astype(np.int64) + off)
        off += v.shape[0]
    assert off < 2 ** 31
    return MeshBatch(np.concatenate(vs, 0), np.concatenate(fs, 0).astype(np.int32),
                     np.array([v.shape[0] for v, _ in meshes], np.int32),
                     np.array([f.shape[0] for _, f in meshes], np.int32))


def icosphere_batch(batch: int, level: int, seed: int, mode: str) -> MeshBatch:
    """mode 'jitter': radius * (1 + N(0, 0.02)); mode 'noise_rot': radial U(-0.1, 0.1)
    plus a random rotation per mesh."""
    rng = np.random.default_rng(seed)
    v0, f0 = icosphere(level)
    meshes = []
    for _ in range(batch):
        if mode == "jitter":
            rad = 1.0 + rng.normal(0.0, 0.02, size=(v0.shape[0], 1))
            v = v0 * rad
        elif mode == "noise_rot":
            rad = 1.0 + rng.uniform(-0.1, 0.1, size=(v0.shape[0], 1))
            v = (v0 * rad) @ random_rotation(rng).T
        else:
            raise ValueError(mode)
        meshes.append((v.astype(np.float32), f0))
    return concat_meshes(meshes)


def heightfield_batch(batch: int, n: int, seed: int) -> MeshBatch:
    return concat_meshes([heightfield(n, seed * 1000 + i) for i in range(batch)])


def texture_samples(num_faces: int, seed: int, max_per_face: int = 4
                    ) -> Tuple[np.ndarray, np.ndarray]:
    """Per-face sample counts T_f ~ U{1..max_per_face} and Dirichlet(1,1,1) barycentric
    coordinates for every sample (grouped by face, as the reference's texture input is)."""
    rng = np.random.default_rng(seed)
    counts = rng.integers(1, max_per_face + 1, size=num_faces).astype(np.int32)
    bary = rng.dirichlet(np.ones(3), size=int(counts.sum())).astype(np.float32)
    return counts, bary


def xavier_normal(shape: Sequence[int], rng: np.random.Generator) -> np.ndarray:
    """torch.nn.init.xavier_normal_ statistics for a tensor of this shape
    (fan_in = shape[1] * receptive field, fan_out = shape[0] * receptive field)."""
    shape = tuple(int(s) for s in shape)
    rf = int(np.prod(shape[2:])) if len(shape) > 2 else 1
    fan_in, fan_out = shape[1] * rf, shape[0] * rf
    std = math.sqrt(2.0 / float(fan_in + fan_out))
    return (rng.standard_normal(shape) * std).astype(np.float32)


# name -> (generator description); sizes follow the five benchmark configurations
CONFIGS = {
    "c1": dict(kind="icosphere", batch=4, level=4, mode="jitter", cin=32, cout=64, L=3, seed=1),
    "c2": dict(kind="icosphere", batch=64, level=3, mode="noise_rot", cin=32, cout=64, L=3, seed=2),
    "c2b": dict(kind="icosphere", batch=64, level=3, mode="noise_rot", cin=64, cout=128, L=3, seed=2),
    "c3": dict(kind="heightfield", batch=2, n=700, cin=64, cout=64, L=3, seed=3),
    "c5": dict(kind="heightfield", batch=32, n=360, cin=128, cout=128, L=4, seed=5),
}


def make_batch(cfg: dict, batch: int | None = None, first_mesh: int = 0) -> MeshBatch:
    """Meshes [first_mesh, first_mesh + batch) of a configuration (a rank's shard when the
    batch is split across GPUs; meshes are generated independently so shards agree with
    the whole batch)."""
    total = cfg["batch"]
    batch = total - first_mesh if batch is None else batch
    if cfg["kind"] == "icosphere":
        full = icosphere_batch(total, cfg["level"], cfg["seed"], cfg["mode"])
        return slice_batch(full, first_mesh, batch)
    return concat_meshes([heightfield(cfg["n"], cfg["seed"] * 1000 + i)
                          for i in range(first_mesh, first_mesh + batch)])


def slice_batch(mb: MeshBatch, first: int, count: int) -> MeshBatch:
    """Sub-batch of whole meshes with vertex ids re-based to the slice."""
    voff = np.concatenate([[0], np.cumsum(mb.nv)]).astype(np.int64)
    foff = np.concatenate([[0], np.cumsum(mb.mf)]).astype(np.int64)
    v0, v1 = voff[first], voff[first + count]
    f0, f1 = foff[first], foff[first + count]
    return MeshBatch(mb.vertex[v0:v1].copy(), (mb.face[f0:f1].astype(np.int64) - v0).astype(np.int32),
                     mb.nv[first:first + count].copy(), mb.mf[first:first + count].copy())
