"""CPU restatement (PyTorch, fp32 or fp64 by input dtype) of the reference's mesh
convolution path.  TEST INFRASTRUCTURE ONLY: nothing in the product package imports this
file; it exists to check the CUDA kernels and to serve as the timed CPU baseline.

Parity status: the reference ships no tests, golden vectors or fixtures for this path, so
the restatement is pinned against outputs of the reference's own CUDA operators run on a
B200 (fixtures under tests/golden/, made by tests/golden/make_golden.py) and against the
independent plain-C restatement in oracle/mesh_oracle.c.

Each function cites the reference code it follows (paths relative to the reference root).
"""
from __future__ import annotations

import math

import numpy as np
import torch


# ------------------------------------------------------------------ spherical harmonics
def _sph_constants(dtype: torch.dtype):
    """Normalisation constants exactly as picasso/math_utils.py:6,17-59 evaluates them: a
    python scalar combined with the fp32 CPU tensor TPI = tensor(pi), i.e. computed in fp32
    (fp64 here when the fp64 arbiter is requested)."""
    TPI = torch.tensor(math.pi, dtype=dtype)
    s = torch.sqrt
    c = {}
    c[0] = 1 / 2. * s(1 / TPI)
    c[1] = 1 / 2. * s(3 / 2 / TPI)
    c[2] = 1 / 2. * s(3 / TPI)
    c[3] = c[1]
    c[4] = 1 / 4. * s(15 / 2 / TPI)
    c[5] = 1 / 2. * s(15 / 2 / TPI)
    c[6] = 1 / 4. * s(5 / TPI)
    c[7] = c[4]
    c[8] = c[5]
    c[9] = 1 / 8. * s(35 / TPI)
    c[10] = 1 / 4. * s(105 / 2 / TPI)
    c[11] = 1 / 8. * s(21 / TPI)
    c[12] = 1 / 4. * s(7 / TPI)
    c[13], c[14], c[15] = c[9], c[10], c[11]
    c[16] = 3 / 16. * s(35 / 2 / TPI)
    c[17] = 3 / 8. * s(35 / TPI)
    c[18] = 3 / 8. * s(5 / 2 / TPI)
    c[19] = 3 / 8. * s(5 / TPI)
    c[20] = 3 / 16. * s(1 / TPI)
    c[21], c[22], c[23], c[24] = c[16], c[17], c[18], c[19]
    c[25] = 3 / 32. * s(77 / TPI)
    c[26] = 3 / 16. * s(385 / 2 / TPI)
    c[27] = 1 / 32. * s(385 / TPI)
    c[28] = 1 / 8. * s(1155 / 2 / TPI)
    c[29] = 1 / 16. * s(165 / 2 / TPI)
    c[30] = 1 / 16. * s(11 / TPI)
    c[31], c[32], c[33], c[34], c[35] = c[25], c[26], c[27], c[28], c[29]
    return c


def sph_constants_f32() -> np.ndarray:
    """The 36 fp32 normalisation constants (for handing to a kernel or a C routine)."""
    c = _sph_constants(torch.float32)
    return np.array([float(c[i]) for i in range(36)], dtype=np.float32)


def sph_harm_reorder(L: int, phi: torch.Tensor, theta: torch.Tensor) -> torch.Tensor:
    """picasso/math_utils.py:10-62 (torch_sph_harm_reorder): per degree l the columns are the
    cos(m phi) terms for m = l..1, the m = 0 term, then the sin(m phi) terms for m = l..1."""
    if L >= 6:
        raise NotImplementedError
    dt = phi.dtype
    c = _sph_constants(dt)
    st, ct = torch.sin(theta), torch.cos(theta)
    out = torch.zeros(phi.shape[0], (L + 1) ** 2, dtype=dt)
    cos, sin = torch.cos, torch.sin
    if L >= 0:
        out[:, 0] = c[0]
    if L >= 1:
        out[:, 1] = c[1] * st * cos(phi)
        out[:, 2] = c[2] * ct
        out[:, 3] = c[3] * st * sin(phi)
    if L >= 2:
        out[:, 4] = c[4] * (st ** 2) * cos(2 * phi)
        out[:, 5] = c[5] * st * ct * cos(phi)
        out[:, 6] = c[6] * (3 * (ct ** 2) - 1)
        out[:, 7] = c[7] * (st ** 2) * sin(2 * phi)
        out[:, 8] = c[8] * st * ct * sin(phi)
    if L >= 3:
        out[:, 9] = c[9] * (st ** 3) * cos(3 * phi)
        out[:, 10] = c[10] * (st ** 2) * ct * cos(2 * phi)
        out[:, 11] = c[11] * st * (5 * (ct ** 2) - 1) * cos(phi)
        out[:, 12] = c[12] * (5 * (ct ** 3) - 3 * ct)
        out[:, 13] = c[13] * (st ** 3) * sin(3 * phi)
        out[:, 14] = c[14] * (st ** 2) * ct * sin(2 * phi)
        out[:, 15] = c[15] * st * (5 * (ct ** 2) - 1) * sin(phi)
    if L >= 4:
        out[:, 16] = c[16] * (st ** 4) * cos(4 * phi)
        out[:, 17] = c[17] * (st ** 3) * ct * cos(3 * phi)
        out[:, 18] = c[18] * (st ** 2) * (7 * (ct ** 2) - 1) * cos(2 * phi)
        out[:, 19] = c[19] * st * (7 * (ct ** 3) - 3 * ct) * cos(phi)
        out[:, 20] = c[20] * (35 * ct ** 4 - 30 * (ct ** 2) + 3)
        out[:, 21] = c[21] * (st ** 4) * sin(4 * phi)
        out[:, 22] = c[22] * (st ** 3) * ct * sin(3 * phi)
        out[:, 23] = c[23] * (st ** 2) * (7 * (ct ** 2) - 1) * sin(2 * phi)
        out[:, 24] = c[24] * st * (7 * (ct ** 3) - 3 * ct) * sin(phi)
    if L >= 5:
        out[:, 25] = c[25] * (st ** 5) * cos(5 * phi)
        out[:, 26] = c[26] * (st ** 4) * ct * cos(4 * phi)
        out[:, 27] = c[27] * (st ** 3) * (9 * (ct ** 2) - 1) * cos(3 * phi)
        out[:, 28] = c[28] * (st ** 2) * (3 * (ct ** 3) - ct) * cos(2 * phi)
        out[:, 29] = c[29] * st * (21 * ct ** 4 - 14 * ct ** 2 + 1) * cos(phi)
        out[:, 30] = c[30] * (63 * ct ** 5 - 70 * ct ** 3 + 15 * ct)
        out[:, 31] = c[31] * (st ** 5) * sin(5 * phi)
        out[:, 32] = c[32] * (st ** 4) * ct * sin(4 * phi)
        out[:, 33] = c[33] * (st ** 3) * (9 * (ct ** 2) - 1) * sin(3 * phi)
        out[:, 34] = c[34] * (st ** 2) * (3 * (ct ** 3) - ct) * sin(2 * phi)
        out[:, 35] = c[35] * st * (21 * ct ** 4 - 14 * ct ** 2 + 1) * sin(phi)
    return out


def sph_harm_coeff(L: int, cart: torch.Tensor) -> torch.Tensor:
    """picasso/mesh/layers.py:341-356 (SphHarmCoeff): project to the unit sphere with
    +1e-10 in the denominator, azimuth phi in [0, 2pi), polar theta measured from +z."""
    l2 = torch.sqrt(torch.sum(cart ** 2, dim=-1, keepdim=True))
    p = cart / (l2 + 1e-10)
    phi = torch.atan2(p[:, 1], p[:, 0])
    theta = torch.atan2(p[:, 2], torch.linalg.norm(p[:, :2], dim=-1))
    phi = torch.where(phi < 0, phi + 2 * np.pi, phi)
    theta = np.pi / 2 - theta
    return sph_harm_reorder(L, phi, theta)


# ----------------------------------------------------------------- geometry / adjacency
def triangle_geometry(vertex: torch.Tensor, face: torch.Tensor) -> torch.Tensor:
    """picasso/mesh/pi_modules/decimate.py:70-85: [unit normal, plane intercept, area]."""
    vertex = vertex[:, :3]
    face = face.to(torch.long)
    vec10 = vertex[face[:, 1]] - vertex[face[:, 0]]
    vec20 = vertex[face[:, 2]] - vertex[face[:, 0]]
    raw = torch.cross(vec10, vec20, dim=-1)
    l2 = torch.sqrt(torch.sum(raw ** 2, dim=-1, keepdim=True))
    area = l2 / 2
    normal = raw / (l2 + 1e-10)
    d = -torch.sum(normal * vertex[face[:, 0]], dim=-1, keepdim=True)
    return torch.cat([normal, d, area], dim=-1)


def oriented_normals(geometry: torch.Tensor, vertex: torch.Tensor, face: torch.Tensor) -> torch.Tensor:
    """picasso/networks/scene_seg.py:117-124 (get_oriented_normals): flip a face normal when it points
    away from the origin taken as viewpoint; sign = sign(sum(-center*normal)) with every sign above -1
    set to +1, so only a strictly negative dot product flips."""
    face = face.to(torch.long)
    normals = geometry[:, :3]
    center = (vertex[face[:, 0], :3] + vertex[face[:, 1], :3] + vertex[face[:, 2], :3]) / 3
    sign = torch.sign(torch.sum(-center * normals, dim=-1, keepdim=True))
    sign = torch.where(sign > -1, torch.ones_like(sign), sign)
    return normals * sign


def count_vertex_adjface(face: torch.Tensor, vt_map: torch.Tensor, nv_out: int) -> torch.Tensor:
    """picasso/mesh/pi_modules/source/decimate_gpu.cu:813-831: one count per face corner
    whose mapped vertex id is non-negative."""
    vo = vt_map.to(torch.long)[face.to(torch.long).reshape(-1)]
    vo = vo[vo >= 0]
    return torch.bincount(vo, minlength=nv_out).to(torch.int32)


# ------------------------------------------------------------------------------ V2F
def vertex2facet_forward(inp, filt, face):
    """mesh_conv3d_gpu.cu:176-195: out[f, c*r+m] = sum_k filter[k,c,m] * in[face[f,k], c]."""
    face = face.to(torch.long)
    _, C, r = filt.shape
    out = torch.zeros(face.shape[0], C, r, dtype=inp.dtype, device=inp.device)
    for k in range(3):
        out += filt[k].unsqueeze(0) * inp[face[:, k]].unsqueeze(-1)
    return out.reshape(face.shape[0], C * r)


def vertex2facet_backward(gout, inp, filt, face):
    """mesh_conv3d_gpu.cu:201-260: gIn[face[f,k], c] += sum_m gOut[f,c*r+m]*filter[k,c,m];
    gF[k,c,m] = sum_f gOut[f,c*r+m] * in[face[f,k], c]."""
    face = face.to(torch.long)
    _, C, r = filt.shape
    g = gout.reshape(-1, C, r)
    gin = torch.zeros_like(inp)
    gf = torch.zeros_like(filt)
    for k in range(3):
        gin.index_add_(0, face[:, k], (g * filt[k].unsqueeze(0)).sum(-1))
        gf[k] = (g * inp[face[:, k]].unsqueeze(-1)).sum(0)
    return gin, gf


# ------------------------------------------------------------------------------ F2V
def _f2v_terms(coeff, filt):
    K, C, r = filt.shape
    return (coeff @ filt.reshape(K, C * r)).reshape(-1, C, r)   # w[f, c, m]


def facet2vertex_forward(inp, filt, coeff, face, nf_count, vt_map):
    """mesh_conv3d_gpu.cu:299-329: w[f,co] = sum_k coeff[f,k]*filter[k,co];
    out[vo,co] += w*in[f,c]/nfCount[vo] for the three corners with vo = vtMap[v] >= 0."""
    face = face.to(torch.long)
    K, C, r = filt.shape
    nv_out = nf_count.shape[0]
    wx = _f2v_terms(coeff, filt) * inp.unsqueeze(-1)          # (Nf, C, r)
    out = torch.zeros(nv_out, C, r, dtype=inp.dtype, device=inp.device)
    vmap = vt_map.to(torch.long)
    nf = nf_count.to(inp.dtype)
    for j in range(3):
        vo = vmap[face[:, j]]
        ok = vo >= 0
        vo_ok = vo[ok]
        out.index_add_(0, vo_ok, wx[ok] / nf[vo_ok].reshape(-1, 1, 1))
    return out.reshape(nv_out, C * r)


def facet2vertex_backward(gout, inp, filt, coeff, face, nf_count, vt_map):
    """mesh_conv3d_gpu.cu:338-426: gt[f,co] = sum_{corners, vo>=0} gOut[vo,co]/nfCount[vo];
    gIn[f,c] = sum_m gt*w;  gF[k,c,m] = sum_f coeff[f,k]*in[f,c]*gt[f,c,m]."""
    face = face.to(torch.long)
    K, C, r = filt.shape
    vmap = vt_map.to(torch.long)
    nf = nf_count.to(inp.dtype)
    g = gout.reshape(-1, C, r)
    gt = torch.zeros(face.shape[0], C, r, dtype=inp.dtype, device=inp.device)
    for j in range(3):
        vo = vmap[face[:, j]]
        ok = vo >= 0
        vo_c = vo.clamp(min=0)
        term = g[vo_c] / nf[vo_c].clamp(min=1).reshape(-1, 1, 1)
        gt += torch.where(ok.reshape(-1, 1, 1), term, torch.zeros_like(term))
    w = _f2v_terms(coeff, filt)
    gin = (gt * w).sum(-1)
    gf = (coeff.t() @ (inp.unsqueeze(-1) * gt).reshape(-1, C * r)).reshape(K, C, r)
    return gin, gf


# ------------------------------------------------------------------------------ F2F
def _f2f_segments(cum, n_samples):
    cum = cum.to(torch.long)
    counts = torch.diff(cum, prepend=torch.zeros(1, dtype=torch.long, device=cum.device))
    fid = torch.repeat_interleave(torch.arange(cum.shape[0], device=cum.device), counts, output_size=n_samples)
    return counts, fid


def _f2f_A(inp, bary, counts, fid, f0, f1, k0, k1):
    """A[f,d,ci] = (1/T_f) sum_{k in f} bary[k,d]*in[k,ci] for faces [f0,f1)."""
    F = bary.shape[1]
    A = torch.zeros(f1 - f0, F, inp.shape[1], dtype=inp.dtype, device=inp.device)
    if k1 > k0:
        A.index_add_(0, fid[k0:k1] - f0, bary[k0:k1].unsqueeze(-1) * inp[k0:k1].unsqueeze(1))
    T = counts[f0:f1].to(inp.dtype).clamp(min=1).reshape(-1, 1, 1)
    return A / T


def _face_chunks(cum, chunk):
    nf = cum.shape[0]
    cl = cum.to(torch.long)
    for f0 in range(0, nf, chunk):
        f1 = min(nf, f0 + chunk)
        k0 = int(cl[f0 - 1]) if f0 > 0 else 0
        k1 = int(cl[f1 - 1])
        yield f0, f1, k0, k1


def facet2facet_forward(inp, filt, bary, cum, chunk=8192):
    """mesh_conv3d_gpu.cu:6-37: out[f,co] = (1/T_f) sum_ci sum_{k in f} in[k,ci] *
    sum_d bary[k,d]*filter[co,ci,d]; the samples of face f are rows cum[f-1]..cum[f]-1
    (cum = inclusive cumulative sample count); a face with no samples gives 0."""
    Cout = filt.shape[0]
    counts, fid = _f2f_segments(cum, inp.shape[0])
    out = torch.zeros(cum.shape[0], Cout, dtype=inp.dtype, device=inp.device)
    Wt = filt.permute(2, 1, 0).reshape(-1, Cout)             # [(d,ci), co]
    for f0, f1, k0, k1 in _face_chunks(cum, chunk):
        A = _f2f_A(inp, bary, counts, fid, f0, f1, k0, k1)
        out[f0:f1] = A.reshape(f1 - f0, -1) @ Wt
    return out


def facet2facet_backward(gout, inp, filt, bary, cum, chunk=8192):
    """mesh_conv3d_gpu.cu:45-135: gIn[k,ci] = (1/T_f) sum_co gOut[f,co] sum_d bary[k,d] *
    filter[co,ci,d];  gF[co,ci,d] = sum_f gOut[f,co] * A[f,d,ci]."""
    Cout, Cin, F = filt.shape
    counts, fid = _f2f_segments(cum, inp.shape[0])
    gin = torch.zeros_like(inp)
    gfl = torch.zeros(F * Cin, Cout, dtype=inp.dtype, device=inp.device)
    Wt = filt.permute(2, 1, 0).reshape(-1, Cout)
    for f0, f1, k0, k1 in _face_chunks(cum, chunk):
        A = _f2f_A(inp, bary, counts, fid, f0, f1, k0, k1)
        gfl += A.reshape(f1 - f0, -1).t() @ gout[f0:f1]
        if k1 > k0:
            gA = (gout[f0:f1] @ Wt.t()).reshape(f1 - f0, F, Cin)
            gA = gA / counts[f0:f1].to(inp.dtype).clamp(min=1).reshape(-1, 1, 1)
            gin[k0:k1] = (bary[k0:k1].unsqueeze(-1) * gA[fid[k0:k1] - f0]).sum(1)
    gf = gfl.reshape(F, Cin, Cout).permute(2, 1, 0).contiguous()
    return gin, gf


# ----------------------------------------------------------------- mesh pool / unpool
def _cluster_key(vt_replace, vt_map):
    """Coarse id of every fine vertex, -1 outside every cluster (the index arithmetic shared by all
    kernels of mesh_pool3d_gpu.cu and mesh_unpool3d_gpu.cu: mapid = -vtReplace[v] for a contracted
    vertex, else v; the cluster's coarse id is vtMap[mapid])."""
    v = torch.arange(vt_replace.shape[0], device=vt_replace.device)
    rep = vt_replace.to(torch.long)
    mapid = torch.where(rep < 0, -rep, v)
    return vt_map.to(torch.long)[mapid], mapid


def mesh_max_pool_forward(inp, vt_replace, vt_map, nv_out):
    """mesh_pool3d_gpu.cu:20-88: output[vo] = max over the cluster's members; maxIndex = a member that
    attains it (the smallest id here; the reference takes whichever thread wrote last)."""
    key, _ = _cluster_key(vt_replace, vt_map)
    C = inp.shape[1]
    out = torch.zeros(nv_out, C, dtype=inp.dtype, device=inp.device)
    idx = torch.zeros(nv_out, C, dtype=torch.int32, device=inp.device)
    ok = key >= 0
    members = torch.nonzero(ok).flatten()
    if members.numel():
        k = key[members]
        out_m = torch.full((nv_out, C), -float("inf"), dtype=inp.dtype, device=inp.device)
        out_m.scatter_reduce_(0, k.unsqueeze(1).expand(-1, C), inp[members], reduce="amax")
        hit = inp[members] == out_m[k]
        cand = torch.where(hit, members.unsqueeze(1).expand(-1, C), torch.full_like(hit, 2 ** 31 - 1, dtype=torch.long))
        first = torch.full((nv_out, C), 2 ** 31 - 1, dtype=torch.long, device=inp.device)
        first.scatter_reduce_(0, k.unsqueeze(1).expand(-1, C), cand, reduce="amin")
        has = torch.zeros(nv_out, dtype=torch.bool, device=inp.device)
        has[k] = True
        out[has] = out_m[has]
        idx[has] = first[has].to(torch.int32)
    return out, idx


def mesh_max_pool_backward(gout, nv_in, max_index):
    """mesh_pool3d_gpu.cu:93-105: gradInput[maxIndex[vo,c], c] = gradOutput[vo,c], zero elsewhere."""
    C = gout.shape[1]
    gin = torch.zeros(nv_in, C, dtype=gout.dtype, device=gout.device)
    gin.scatter_(0, max_index.to(torch.long), gout)
    return gin


def mesh_avg_pool_forward(inp, vt_replace, vt_map, nv_out):
    """mesh_pool3d_gpu.cu:112-132: output[vo] += input[v] / (vtReplace[mapid] + 1)."""
    key, mapid = _cluster_key(vt_replace, vt_map)
    count = (vt_replace.to(torch.long)[mapid] + 1).to(inp.dtype)
    out = torch.zeros(nv_out, inp.shape[1], dtype=inp.dtype, device=inp.device)
    ok = key >= 0
    out.index_add_(0, key[ok], inp[ok] / count[ok].unsqueeze(1))
    return out


def mesh_avg_pool_backward(gout, vt_replace, vt_map):
    """mesh_pool3d_gpu.cu:138-158: gradInput[v] = gradOutput[vo] / count for cluster members."""
    key, mapid = _cluster_key(vt_replace, vt_map)
    count = (vt_replace.to(torch.long)[mapid] + 1).to(gout.dtype)
    gin = torch.zeros(vt_replace.shape[0], gout.shape[1], dtype=gout.dtype, device=gout.device)
    ok = key >= 0
    gin[ok] = gout[key[ok]] / count[ok].unsqueeze(1)
    return gin


def mesh_unpool_forward(inp, vt_replace, vt_map):
    """mesh_unpool3d_gpu.cu:5-26: output[v] = input[vtMap[mapid]] for every fine vertex of a cluster."""
    key, _ = _cluster_key(vt_replace, vt_map)
    out = torch.zeros(vt_map.shape[0], inp.shape[1], dtype=inp.dtype, device=inp.device)
    ok = key >= 0
    out[ok] = inp[key[ok]]
    return out


def mesh_unpool_backward(gout, nv_coarse, vt_replace, vt_map):
    """mesh_unpool3d_gpu.cu:29-46: gradInput[vtMap[mapid]] += gradOutput[v]."""
    key, _ = _cluster_key(vt_replace, vt_map)
    gin = torch.zeros(nv_coarse, gout.shape[1], dtype=gout.dtype, device=gout.device)
    ok = key >= 0
    gin.index_add_(0, key[ok], gout[ok])
    return gin


# ------------------------------------------------------- point-cloud depthwise convolution
def _pair_weights(filt, bin_index, bin_coeff):
    """w[p, c, m]: filter[bin[p]] (hard assignment) or sum_t coeff[p,t]*filter[bin[p,t]] (fuzzy);
    picasso/point/pi_modules/source/pcloud_conv3d_gpu.cu:24,108-116."""
    if bin_coeff is None:
        return filt[bin_index.to(torch.long)]
    return (bin_coeff.unsqueeze(-1).unsqueeze(-1) * filt[bin_index.to(torch.long)]).sum(1)


def pcloud_conv3d_forward(inp, filt, nn_count, nn_index, bin_index, bin_coeff=None):
    """pcloud_conv3d_gpu.cu:8-27 (hard) / 94-118 (fuzzy): output[out_p, c*r+m] += input[in_p, c] *
    w_p[c, m] / nnCount[out_p] over the neighbour pairs p = (out_p, in_p)."""
    F, C, r = filt.shape
    o, i = nn_index[:, 0].to(torch.long), nn_index[:, 1].to(torch.long)
    w = _pair_weights(filt, bin_index, bin_coeff)
    term = inp[i].unsqueeze(-1) * w / nn_count.to(inp.dtype)[o].reshape(-1, 1, 1)
    out = torch.zeros(nn_count.shape[0], C, r, dtype=inp.dtype, device=inp.device)
    out.index_add_(0, o, term)
    return out.reshape(-1, C * r)


def pcloud_conv3d_backward(gout, inp, filt, nn_count, nn_index, bin_index, bin_coeff=None):
    """pcloud_conv3d_gpu.cu:30-88 (hard) / 121-193 (fuzzy): gIn[in_p, c] += sum_m gOut[out_p, c*r+m] *
    w_p[c,m] / nnCount[out_p];  gF[f, c, m] += coeff * gOut[out_p, c*r+m] * input[in_p, c] / nnCount[out_p]."""
    F, C, r = filt.shape
    o, i = nn_index[:, 0].to(torch.long), nn_index[:, 1].to(torch.long)
    w = _pair_weights(filt, bin_index, bin_coeff)
    g = gout.reshape(-1, C, r)[o] / nn_count.to(inp.dtype)[o].reshape(-1, 1, 1)
    gin = torch.zeros_like(inp)
    gin.index_add_(0, i, (g * w).sum(-1))
    d = g * inp[i].unsqueeze(-1)
    gf = torch.zeros_like(filt)
    if bin_coeff is None:
        gf.index_add_(0, bin_index.to(torch.long), d)
    else:
        for t in range(bin_index.shape[1]):
            gf.index_add_(0, bin_index[:, t].to(torch.long), bin_coeff[:, t].reshape(-1, 1, 1) * d)
    return gin, gf


# ------------------------------------------------------------- autograd wrappers (CPU)
class _V2F(torch.autograd.Function):
    @staticmethod
    def forward(ctx, inp, filt, face):
        ctx.save_for_backward(inp, filt, face)
        return vertex2facet_forward(inp, filt, face)

    @staticmethod
    def backward(ctx, g):
        gi, gf = vertex2facet_backward(g.contiguous(), *ctx.saved_tensors)
        return gi, gf, None


class _F2V(torch.autograd.Function):
    @staticmethod
    def forward(ctx, inp, filt, coeff, face, nf_count, vt_map):
        ctx.save_for_backward(inp, filt, coeff, face, nf_count, vt_map)
        return facet2vertex_forward(inp, filt, coeff, face, nf_count, vt_map)

    @staticmethod
    def backward(ctx, g):
        gi, gf = facet2vertex_backward(g.contiguous(), *ctx.saved_tensors)
        return gi, gf, None, None, None, None


class _F2F(torch.autograd.Function):
    @staticmethod
    def forward(ctx, inp, filt, bary, cum):
        ctx.save_for_backward(inp, filt, bary, cum)
        return facet2facet_forward(inp, filt, bary, cum)

    @staticmethod
    def backward(ctx, g):
        gi, gf = facet2facet_backward(g.contiguous(), *ctx.saved_tensors)
        return gi, gf, None, None


vertex2facet = _V2F.apply
facet2vertex = _F2V.apply
facet2facet = _F2F.apply


def conv_block(x, Wv, Wf, Wo, face, counts, cum, bary_sh, coeff, nf_count, vt_map, sh_eye):
    """The benchmark's V2F -> F2F -> F2V block: y = V2F(x, (SH(eye3) @ Wv) as (3,Cin,1));
    texture rows repeat y[f] once per sample of f; z = F2F(tex, Wf, SH(bary), cum);
    o = F2V(z, Wo, SH(normals), face, nfCount, vtMap)."""
    cin = x.shape[1]
    y = vertex2facet(x, (sh_eye @ Wv).reshape(3, cin, 1), face)
    tex = torch.repeat_interleave(y, counts.to(torch.long), dim=0)
    z = facet2facet(tex, Wf, bary_sh, cum)
    return facet2vertex(z, Wo, coeff, face, nf_count, vt_map)
