"""Seeded operator inputs shared by the parity tests and the golden-fixture generator."""
from __future__ import annotations

import numpy as np
import torch

from picassoplus_b200 import synth


def topology(kind: str, seed: int):
    """(vertex, face, vtMap, NvOut) as numpy; kinds: ico<level>x<batch>, grid<n>x<batch>,
    and the suffix '+drop' that maps every 5th vertex to -1 and compacts the rest."""
    drop = kind.endswith("+drop")
    base = kind[:-5] if drop else kind
    if base.startswith("ico"):
        level, batch = base[3:].split("x")
        mb = synth.icosphere_batch(int(batch), int(level), seed, "noise_rot")
    elif base.startswith("grid"):
        n, batch = base[4:].split("x")
        mb = synth.heightfield_batch(int(batch), int(n), seed)
    elif base == "tri":
        mb = synth.concat_meshes([(np.eye(3, dtype=np.float32), np.array([[0, 1, 2]], np.int32))])
    elif base == "tet+iso":   # a tetrahedron plus a vertex no face touches
        v = np.array([[0, 0, 0], [1, 0, 0], [0, 1, 0], [0, 0, 1], [2, 2, 2]], np.float32)
        f = np.array([[0, 2, 1], [0, 1, 3], [1, 2, 3], [0, 3, 2]], np.int32)
        mb = synth.concat_meshes([(v, f)])
    else:
        raise ValueError(kind)
    nv = mb.num_vertices
    vt = np.arange(nv, dtype=np.int32)
    nv_out = nv
    if drop:
        keep = (np.arange(nv) % 5) != 0
        vt = np.where(keep, np.cumsum(keep) - 1, -1).astype(np.int32)
        nv_out = int(keep.sum())
    return mb.vertex, mb.face, vt, nv_out


def conv_inputs(kind: str, C: int, r: int, K: int, cout: int, seed: int, zero_sample_faces: bool = True,
                max_per_face: int = 4):
    """All operator inputs for one case, as a dict of CPU torch tensors."""
    g = torch.Generator().manual_seed(seed)
    vertex, face, vt, nv_out = topology(kind, seed)
    nv, nf = vertex.shape[0], face.shape[0]
    counts, bary = synth.texture_samples(nf, seed + 7, max_per_face)
    if zero_sample_faces and nf > 4:
        counts[1] = 0
        counts[nf - 1] = 0
        bary = bary[: int(counts.sum())]
    d = dict(
        vertex=torch.from_numpy(vertex), face=torch.from_numpy(face), vt_map=torch.from_numpy(vt),
        nv_out=nv_out,
        x_v=torch.randn(nv, C, generator=g), filt_v2f=torch.randn(3, C, r, generator=g),
        g_v2f=torch.randn(nf, C * r, generator=g),
        x_f=torch.randn(nf, C, generator=g), filt_f2v=torch.randn(K, C, r, generator=g) / K ** 0.5,
        coeff=torch.randn(nf, K, generator=g), g_f2v=torch.randn(nv_out, C * r, generator=g),
        counts=torch.from_numpy(counts), cum=torch.cumsum(torch.from_numpy(counts), 0, dtype=torch.int32),
        tex=torch.randn(int(counts.sum()), C, generator=g),
        bary=torch.randn(int(counts.sum()), K, generator=g),
        filt_f2f=torch.randn(cout, C, K, generator=g) / (C * K) ** 0.5,
        g_f2f=torch.randn(nf, cout, generator=g),
        bary_xyz=torch.from_numpy(bary),
    )
    return d


GOLDEN_CASES = {
    # name: (topology, C, r, K, Cout, seed)
    "ico1x2_c8_r1_k16": ("ico1x2", 8, 1, 16, 12, 11),
    "ico1x2_c5_r2_k9": ("ico1x2", 5, 2, 9, 7, 12),
    "grid9x1_c4_r1_k25": ("grid9x1", 4, 1, 25, 4, 13),
}


def cluster_inputs(nv_in: int, nv_out: int, C: int, seed: int, drop_frac: float = 0.1, ties: bool = False):
    """A random decimation clustering in the reference's encoding (picasso/mesh/pi_modules/
    decimate.py:23-28) plus features and upstream gradients, as CPU torch tensors.
    nv_out representatives keep their order (vtMap counts them from 0); every other vertex is
    contracted into a random representative (vtReplace = -representative, vtMap = -1) or, with
    probability drop_frac, belongs to no cluster (vtReplace = 0, vtMap = -1).  Vertex 0 is never a
    contraction target (-0 cannot be told from 0).  ties=True quantises the features so that equal
    maxima occur inside clusters."""
    rng = np.random.default_rng(seed)
    reps = np.sort(rng.choice(nv_in, size=nv_out, replace=False))
    is_rep = np.zeros(nv_in, bool)
    is_rep[reps] = True
    vt_map = np.full(nv_in, -1, np.int32)
    vt_map[reps] = np.arange(nv_out, dtype=np.int32)
    vt_replace = np.zeros(nv_in, np.int32)
    targets = reps[reps > 0]
    for v in np.nonzero(~is_rep)[0]:
        if targets.size and rng.random() >= drop_frac:
            r = int(targets[rng.integers(targets.size)])
            vt_replace[v] = -r
            vt_replace[r] += 1
    g = torch.Generator().manual_seed(seed)
    x = torch.randn(nv_in, C, generator=g)
    if ties:
        x = torch.round(x * 2) / 2
    return dict(vt_replace=torch.from_numpy(vt_replace), vt_map=torch.from_numpy(vt_map), nv_in=nv_in, nv_out=nv_out,
                x=x, g_coarse=torch.randn(nv_out, C, generator=g), x_coarse=torch.randn(nv_out, C, generator=g),
                g_fine=torch.randn(nv_in, C, generator=g))


POOL_GOLDEN_CASES = {
    # name: (NvIn, NvOut, C, seed)
    "pool_n300_m90_c8": (300, 90, 8, 31),
    "pool_n257_m64_c5": (257, 64, 5, 32),
}


def pcloud_inputs(Np: int, Mp: int, knn: int, F: int, C: int, r: int, T: int, seed: int, shuffle: bool = False):
    """Neighbour pairs of a point-cloud convolution as a neighbour search would emit them (grouped by
    output point unless shuffle=True), filter bins (T = 0: hard assignment; T > 0: T fuzzy bins with
    weights that sum to 1), features, filter and upstream gradient, as CPU torch tensors.  Some output
    points have no neighbour at all."""
    rng = np.random.default_rng(seed)
    counts = rng.integers(0, knn + 1, size=Mp)
    counts[rng.integers(0, Mp)] = knn
    out_idx = np.repeat(np.arange(Mp), counts)
    in_idx = rng.integers(0, Np, size=out_idx.shape[0])
    if shuffle:
        perm = rng.permutation(out_idx.shape[0])
        out_idx, in_idx = out_idx[perm], in_idx[perm]
    nn_index = np.stack([out_idx, in_idx], 1).astype(np.int32)
    nn_count = np.maximum(counts, 1).astype(np.int32)            # the reference divides by it: never 0
    npairs = nn_index.shape[0]
    g = torch.Generator().manual_seed(seed)
    d = dict(nn_index=torch.from_numpy(nn_index), nn_count=torch.from_numpy(nn_count),
             x=torch.randn(Np, C, generator=g), filt=torch.randn(F, C, r, generator=g) / F ** 0.5,
             g_out=torch.randn(Mp, C * r, generator=g))
    if T == 0:
        d["bin_index"] = torch.from_numpy(rng.integers(0, F, size=npairs).astype(np.int32))
        d["bin_coeff"] = None
    else:
        d["bin_index"] = torch.from_numpy(rng.integers(0, F, size=(npairs, T)).astype(np.int32))
        w = rng.random((npairs, T)).astype(np.float32) + 0.05
        d["bin_coeff"] = torch.from_numpy(w / w.sum(1, keepdims=True))
    return d


PCLOUD_GOLDEN_CASES = {
    # name: (Np, Mp, knn, F, C, r, T, seed)
    "pcloud_hard_n200_m60_c6_r2": (200, 60, 12, 9, 6, 2, 0, 41),
    "pcloud_fuzzy_n150_m80_c8_r1": (150, 80, 10, 17, 8, 1, 3, 42),
}


def decimate_inputs(meshes, remove_frac: float, D: int, seed: int, noise: float = 0.0):
    """A batch for one decimation pass, as CPU torch tensors: `meshes` is a list of ("heightfield", n, seed)
    / ("icosphere", level) descriptions, remove_frac the share of every sample's vertices to remove,
    D >= 3 the vertex row width (columns past xyz are random features), noise the standard deviation of
    a random displacement of every vertex.  Height fields have boundary edges and holes, spheres are
    closed.  Without noise the meshes are regular and many candidate edges have exactly equal costs;
    with noise the costs are well separated."""
    import numpy as _np
    from picassoplus_b200 import synth
    from oracle import c_oracle
    rng = _np.random.default_rng(seed)
    vs, fs, nv, mf, off = [], [], [], [], 0
    for m in meshes:
        v, f = synth.heightfield(m[1], seed=m[2]) if m[0] == "heightfield" else synth.icosphere(m[1])
        v = v.astype(_np.float32)
        if noise > 0:
            v = v + (noise * rng.standard_normal(v.shape)).astype(_np.float32)
        vs.append(v)
        fs.append(f.astype(_np.int32) + off)
        off += v.shape[0]
        nv.append(v.shape[0])
        mf.append(f.shape[0])
    V = _np.concatenate(vs)
    if D > 3:
        V = _np.concatenate([V, rng.standard_normal((V.shape[0], D - 3)).astype(_np.float32)], axis=1)
    F = _np.concatenate(fs)
    geo = c_oracle.triangle_geometry(V[:, :3].copy(), F)
    nv, mf = _np.array(nv, _np.int32), _np.array(mf, _np.int32)
    remove = _np.floor(nv * remove_frac).astype(_np.int32)
    t = torch.from_numpy
    return dict(vertex=t(_np.ascontiguousarray(V)), face=t(F), geometry=t(geo), nv=t(nv), mf=t(mf),
                nv_cum=t(_np.cumsum(nv).astype(_np.int32)), mf_cum=t(_np.cumsum(mf).astype(_np.int32)),
                remove=t(remove))


# one decimation pass, library against the sequential restatement (bit for bit):
# name: (meshes, remove_frac, D, seed, noise, useArea, wgtBnd)
DECIMATE_CASES = {
    "two_sweeps": ([("heightfield", 24, 1), ("icosphere", 2), ("heightfield", 17, 3)], 0.75, 3, 51, 0.0, True, 5.0),
    "early_stop": ([("icosphere", 3), ("heightfield", 20, 7)], 0.15, 6, 52, 0.0, False, 0.0),
    "plain_weight": ([("heightfield", 30, 9)], 0.5, 4, 53, 0.0, False, 3.0),
    "one_sample_skipped": ([("heightfield", 16, 2), ("icosphere", 2), ("heightfield", 12, 4)], 0.6, 3, 54, 0.02, True, 5.0),
    "larger": ([("heightfield", 90, 11), ("heightfield", 70, 12), ("icosphere", 4)], 0.7, 3, 55, 0.01, True, 5.0),
}

# fixtures recorded from the reference's own kernels: small meshes with displaced vertices, where the
# candidate costs are far enough apart that neither the order of the reference's float atomics nor its
# fused multiply-adds change the clustering:
# name: (meshes, remove_frac, D, seed, noise, useArea, wgtBnd)
DECIMATE_GOLDEN_CASES = {
    "decim_two_sweeps": ([("heightfield", 8, 1), ("icosphere", 1), ("heightfield", 10, 2)], 0.75, 3, 5, 0.05, True, 5.0),
    "decim_early_stop": ([("heightfield", 8, 1), ("icosphere", 1), ("heightfield", 10, 2)], 0.2, 5, 5, 0.05, True, 5.0),
    "decim_medium": ([("heightfield", 12, 3), ("icosphere", 2)], 0.6, 3, 6, 0.03, True, 5.0),
    "decim_closed_plain": ([("icosphere", 2), ("icosphere", 1)], 0.5, 3, 7, 0.05, False, 0.0),
}
