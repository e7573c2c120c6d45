"""Per-topology device structures shared by the operators: the vertex -> (face, corner)
CSR, its cache, and the validation of index arrays.

A level's `face` / `vtMap` tensors are reused by every convolution of that level (4 to 16
operator calls per step in the reference's encoder blocks,
picasso/networks/pi2_blocks.py:88-92), so the CSR is built once per (face, vtMap) pair
and looked up afterwards.

Cache policy.  A slot is named by the storage of the index tensors (device, data pointer,
length); the slot remembers the tensors' version counters.  A lookup whose versions differ
(the tensors were overwritten in place, as a streaming loader does with its device buffers)
rebuilds the CSR and REPLACES the slot, so stale entries never pile up.  Slots hold a
reference to their index tensors, so the memory behind a key cannot be recycled while the
slot lives.  The cache is bounded by bytes (`set_cache_budget`, default 2 GiB of CSR arrays
per process) and evicts least-recently-used slots; `set_cache_budget(0)` turns it off.
Callers that manage topologies themselves can pass a prebuilt `VertexCSR` to the operator
wrappers (`csr=`) and skip the cache altogether.

Validation.  Building a CSR validates every index of `face` / `vtMap` on the device.  In the
default mode the status word is read back right after the build (ONE device synchronisation
per cache miss, which also answers whether `vtMap` is the identity) and a bad index raises
RuntimeError.  `set_validation("deferred")` removes that synchronisation: status words are
kept and `check_deferred()` reads them all at a point where the caller synchronises anyway
(the end of a step).  Bad indices are never dereferenced in either mode.
"""
from __future__ import annotations

import threading
from collections import OrderedDict
from typing import List, Optional

import torch

from . import _lib

_budget_bytes = 2 << 30
_cache: "OrderedDict[tuple, VertexCSR]" = OrderedDict()
_cache_bytes = 0
_lock = threading.Lock()
_validation = "sync"
_deferred: List[tuple] = []          # (status tensor, message)


def stream_ptr(device) -> int:
    return torch.cuda.current_stream(device).cuda_stream


def ptr(t: Optional[torch.Tensor]):
    return None if t is None else t.data_ptr()


def set_cache_budget(nbytes: int) -> None:
    """Upper bound on the bytes of CSR arrays the cache keeps (0 = no caching)."""
    global _budget_bytes
    with _lock:
        _budget_bytes = int(nbytes)
        _evict_locked()


def set_validation(mode: str) -> None:
    """'sync' (default): raise on a bad index at build time, one device sync per cache miss.
    'deferred': no sync; call check_deferred() after the step's own synchronisation."""
    global _validation
    if mode not in ("sync", "deferred"):
        raise ValueError(mode)
    _validation = mode


def check_deferred() -> None:
    """Reads every status word collected in deferred mode (synchronises); raises RuntimeError
    for the first bad one."""
    with _lock:
        items = list(_deferred)
        _deferred.clear()
    if not items:
        return
    codes = torch.stack([s.reshape(-1)[0] for s, _ in items]).tolist()
    for code, (_, msg) in zip(codes, items):
        if code != 0:
            raise RuntimeError(msg)


class VertexCSR:
    """rowptr (NvOut+1,), entries (3*Nf,) int32: row v lists (f << 2 | corner) ascending."""

    def __init__(self, rowptr, entries, keep, versions=None, shared=False):
        self.rowptr = rowptr
        self.entries = entries
        self._keep = keep
        self._versions = versions
        self.nbytes = 0 if shared else rowptr.numel() * 4 + entries.numel() * 4


def _slot(face, vt_map, nv_in, nv_out):
    vk = None if vt_map is None else (vt_map.data_ptr(), vt_map.shape[0])
    return (face.device.index, face.data_ptr(), face.shape[0], vk, int(nv_in), int(nv_out))


def _versions(face, vt_map):
    return (face._version, None if vt_map is None else vt_map._version)


def _evict_locked():
    global _cache_bytes
    while _cache and _cache_bytes > _budget_bytes:
        _, old = _cache.popitem(last=False)
        _cache_bytes -= old.nbytes


def _launch_build(face, vt_map, nv_in, nv_out):
    dev = face.device
    nf = face.shape[0]
    rowptr = torch.empty(nv_out + 1, dtype=torch.int32, device=dev)
    entries = torch.empty(max(3 * nf, 1), dtype=torch.int32, device=dev)
    status = torch.empty(1, dtype=torch.int32, device=dev)
    wbytes = _lib.query("pb200_vertex_csr_workspace_bytes", nf, nv_out)
    ws = torch.empty(wbytes, dtype=torch.uint8, device=dev)
    _lib.call("pb200_build_vertex_csr", nf, nv_in, nv_out, ptr(face), ptr(vt_map), ptr(rowptr),
              ptr(entries), ptr(status), ptr(ws), wbytes, stream_ptr(dev))
    return rowptr, entries, status


def _bad_index_message(nv_in, nv_out):
    return f"face / vtMap hold an index outside the vertex range (NvIn={nv_in}, NvOut={nv_out})"


def build_vertex_csr(face: torch.Tensor, vt_map: Optional[torch.Tensor], nv_in: int, nv_out: int) -> VertexCSR:
    """Uncached build.  Validates every index: in 'sync' mode a bad one raises RuntimeError here
    (one device synchronisation), in 'deferred' mode at the next check_deferred()."""
    with torch.cuda.device(face.device):
        rowptr, entries, status = _launch_build(face, vt_map, nv_in, nv_out)
        if _validation == "deferred":
            with _lock:
                _deferred.append((status, _bad_index_message(nv_in, nv_out)))
        elif int(status.item()) != 0:
            raise RuntimeError(_bad_index_message(nv_in, nv_out))
    return VertexCSR(rowptr, entries, (face, vt_map), _versions(face, vt_map))


def _lookup(slot, versions):
    with _lock:
        hit = _cache.get(slot)
        if hit is not None and hit._versions == versions:
            _cache.move_to_end(slot)
            return hit
    return None


def _store(slot, csr):
    global _cache_bytes
    with _lock:
        old = _cache.pop(slot, None)
        if old is not None:
            _cache_bytes -= old.nbytes
        if _budget_bytes > 0:
            _cache[slot] = csr
            _cache_bytes += csr.nbytes
            _evict_locked()


def vertex_csr(face: torch.Tensor, vt_map: Optional[torch.Tensor], nv_in: int, nv_out: int) -> VertexCSR:
    """Cached CSR keyed by output vertex vo = vtMap[face[f][j]] (identity when vt_map is None).
    In 'sync' mode an identity vtMap over nv_in == nv_out vertices shares the arrays of
    vt_map=None (the identity test rides on the build's one synchronisation); in 'deferred'
    mode nothing is read back and the CSR is built from vtMap as given."""
    slot = _slot(face, vt_map, nv_in, nv_out)
    versions = _versions(face, vt_map)
    hit = _lookup(slot, versions)
    if hit is not None:
        return hit
    csr = None
    may_be_identity = vt_map is not None and nv_in == nv_out and vt_map.shape[0] == nv_in
    if may_be_identity and _validation == "sync":
        base_slot = _slot(face, None, nv_in, nv_out)
        base = _lookup(base_slot, _versions(face, None))
        with torch.cuda.device(face.device):
            ident = (vt_map == torch.arange(nv_in, dtype=vt_map.dtype, device=vt_map.device)).all().to(torch.int32)
            if base is None:
                # build the identity CSR and test vtMap in the same synchronisation
                rowptr, entries, status = _launch_build(face, None, nv_in, nv_out)
                code, is_ident = torch.stack([status[0], ident]).tolist()
                if code != 0:
                    raise RuntimeError(_bad_index_message(nv_in, nv_out))
                base = VertexCSR(rowptr, entries, (face, None), _versions(face, None))
                _store(base_slot, base)
            else:
                is_ident = int(ident.item())
        if is_ident:
            csr = VertexCSR(base.rowptr, base.entries, (face, vt_map), versions, shared=True)
    if csr is None:
        csr = build_vertex_csr(face, vt_map, nv_in, nv_out)
    _store(slot, csr)
    return csr


def prepare_level(vertex: torch.Tensor, face: torch.Tensor, vt_map: Optional[torch.Tensor], nv_out: int, L: int,
                  orient: bool = False, want_geometry: bool = True, want_normals: bool = False):
    """Everything a mesh level's convolutions need, in one library call: triangle geometry
    (picasso/mesh/pi_modules/decimate.py:70-85), the (optionally origin-oriented,
    picasso/networks/scene_seg.py:117-124) face normals, their spherical-harmonic filter coefficients
    (picasso/mesh/layers.py:341-356), nfCount (decimate_gpu.cu:813-836) and the vertex CSR, which is
    put into the cache for the operator calls that follow.  Returns a dict with keys geometry (Nf,5)
    or None, normals (Nf,3) or None, coeff (Nf,(L+1)^2), nf_count (NvOut,), csr."""
    if L >= 6 or L < 0:
        raise NotImplementedError
    if not (vertex.is_cuda and face.is_cuda) or vertex.dtype != torch.float32 or face.dtype != torch.int32:
        raise RuntimeError("vertex must be a float32 and face an int32 CUDA tensor")
    if vertex.dim() != 2 or vertex.shape[1] < 3 or face.dim() != 2 or face.shape[1] != 3:
        raise RuntimeError("vertex must have shape (Nv, >=3) and face (Nf, 3)")
    vertex, face = vertex.contiguous(), face.contiguous()
    nv_in, nf = vertex.shape[0], face.shape[0]
    dev = face.device
    K = (L + 1) ** 2
    with torch.cuda.device(dev):
        geometry = torch.empty(nf, 5, dtype=torch.float32, device=dev) if want_geometry else None
        normals = torch.empty(nf, 3, dtype=torch.float32, device=dev) if want_normals else None
        coeff = torch.empty(nf, K, dtype=torch.float32, device=dev)
        nf_count = torch.empty(nv_out, dtype=torch.int32, device=dev)
        rowptr = torch.empty(nv_out + 1, dtype=torch.int32, device=dev)
        entries = torch.empty(max(3 * nf, 1), dtype=torch.int32, device=dev)
        status = torch.empty(1, dtype=torch.int32, device=dev)
        wbytes = _lib.query("pb200_vertex_csr_workspace_bytes", nf, nv_out)
        ws = torch.empty(wbytes, dtype=torch.uint8, device=dev)
        _lib.call("pb200_level_prepare", nf, nv_in, nv_out, vertex.shape[1], ptr(vertex), ptr(face), ptr(vt_map), L,
                  1 if orient else 0, ptr(geometry), ptr(normals), ptr(coeff), ptr(nf_count), ptr(rowptr), ptr(entries),
                  ptr(status), ptr(ws), wbytes, stream_ptr(dev))
        if _validation == "deferred":
            with _lock:
                _deferred.append((status, _bad_index_message(nv_in, nv_out)))
        elif int(status.item()) != 0:
            raise RuntimeError(_bad_index_message(nv_in, nv_out))
    csr = VertexCSR(rowptr, entries, (face, vt_map), _versions(face, vt_map))
    _store(_slot(face, vt_map, nv_in, nv_out), csr)
    return dict(geometry=geometry, normals=normals, coeff=coeff, nf_count=nf_count, csr=csr)


class ClusterCSR:
    """Decimation clusters of a fine level: key (NvIn,) = coarse id of each fine vertex or -1;
    rowptr (NvOut+1,), members (NvIn,) = member fine vertices of every coarse vertex, ascending."""

    def __init__(self, key, rowptr, members, keep, versions):
        self.key = key
        self.rowptr = rowptr
        self.members = members
        self._keep = keep
        self._versions = versions
        self.nbytes = 4 * (key.numel() + rowptr.numel() + members.numel())


def cluster_csr(vt_replace: torch.Tensor, vt_map: torch.Tensor, nv_out: int) -> ClusterCSR:
    """Cached cluster structures of (vtReplace, vtMap) (same cache, budget and validation modes as
    vertex_csr).  One pooling level is used by a pool in the encoder and an unpool in the decoder,
    forward and backward: four lookups per step, one build."""
    nv_in = vt_replace.shape[0]
    slot = ("cluster", vt_replace.device.index, vt_replace.data_ptr(), vt_map.data_ptr(), nv_in, int(nv_out))
    versions = (vt_replace._version, vt_map._version)
    hit = _lookup(slot, versions)
    if hit is not None:
        return hit
    dev = vt_replace.device
    with torch.cuda.device(dev):
        key = torch.empty(max(nv_in, 1), dtype=torch.int32, device=dev)
        rowptr = torch.empty(nv_out + 1, dtype=torch.int32, device=dev)
        members = torch.empty(max(nv_in, 1), dtype=torch.int32, device=dev)
        status = torch.empty(1, dtype=torch.int32, device=dev)
        wbytes = _lib.query("pb200_cluster_csr_workspace_bytes", nv_in, nv_out)
        ws = torch.empty(wbytes, dtype=torch.uint8, device=dev)
        _lib.call("pb200_build_cluster_csr", nv_in, nv_out, ptr(vt_replace), ptr(vt_map), ptr(key), ptr(rowptr),
                  ptr(members), ptr(status), ptr(ws), wbytes, stream_ptr(dev))
        msg = f"vtReplace / vtMap hold an index outside the vertex range (NvIn={nv_in}, NvOut={nv_out})"
        if _validation == "deferred":
            with _lock:
                _deferred.append((status, msg))
        elif int(status.item()) != 0:
            raise RuntimeError(msg)
    csr = ClusterCSR(key, rowptr, members, (vt_replace, vt_map), versions)
    _store(slot, csr)
    return csr


class PairCSR:
    """Neighbour pairs grouped by one column of nnIndex: rowptr (rows+1,), members (pairs,) = pair ids
    of every row, ascending."""

    def __init__(self, rowptr, members, keep, versions):
        self.rowptr = rowptr
        self.members = members
        self._keep = keep
        self._versions = versions
        self.nbytes = 4 * (rowptr.numel() + members.numel())


def pair_csr(nn_index: torch.Tensor, column: int, n_rows: int) -> PairCSR:
    """Cached grouping of the neighbour pairs of a point-cloud convolution by their output point
    (column 0) or input point (column 1); same cache, budget and validation modes as vertex_csr."""
    npairs = nn_index.shape[0]
    slot = ("pairs", nn_index.device.index, nn_index.data_ptr(), npairs, int(column), int(n_rows))
    versions = (nn_index._version,)
    hit = _lookup(slot, versions)
    if hit is not None:
        return hit
    dev = nn_index.device
    with torch.cuda.device(dev):
        rowptr = torch.empty(n_rows + 1, dtype=torch.int32, device=dev)
        members = torch.empty(max(npairs, 1), dtype=torch.int32, device=dev)
        status = torch.empty(1, dtype=torch.int32, device=dev)
        wbytes = _lib.query("pb200_cluster_csr_workspace_bytes", npairs, n_rows)
        ws = torch.empty(wbytes, dtype=torch.uint8, device=dev)
        key_ptr = None if npairs == 0 else nn_index.data_ptr() + 4 * column
        _lib.call("pb200_build_key_csr", npairs, n_rows, key_ptr, 2, ptr(rowptr), ptr(members), ptr(status), ptr(ws), wbytes,
                  stream_ptr(dev))
        msg = f"nn_index column {column} holds an index outside [0, {n_rows})"
        if _validation == "deferred":
            with _lock:
                _deferred.append((status, msg))
        elif int(status.item()) != 0:
            raise RuntimeError(msg)
    csr = PairCSR(rowptr, members, (nn_index,), versions)
    _store(slot, csr)
    return csr


class FaceMeans:
    """Per-face mean of the sample rows of a batch (Nf, F) and the running count 1, 2, ..., Nf that says
    'one sample per face'."""

    def __init__(self, rows, one_each, keep, versions):
        self.rows = rows
        self.one_each = one_each
        # the copy with rows padded to a multiple of four floats that the tensor-core kernels read (None when the row
        # length is such a multiple already): made once here instead of in every forward and backward call
        self.rows_padded = pad_rows(rows)
        self._keep = keep
        self._versions = versions
        self.nbytes = 4 * (rows.numel() + one_each.numel() + (0 if self.rows_padded is None else self.rows_padded.numel()))


def pad_rows(rows: torch.Tensor):
    """(N, F) float32 rows -> (N, F rounded up to 4) with zero pad columns, or None when F % 4 == 0."""
    n, F = rows.shape
    if F % 4 == 0 or n == 0:
        return None
    Fp = _lib.query("pb200_padded_row_floats", F)
    dev = rows.device
    with torch.cuda.device(dev):
        out = torch.empty(n, Fp, dtype=torch.float32, device=dev)
        _lib.call("pb200_pad_rows", n, F, ptr(rows), ptr(out), stream_ptr(dev))
    return out


def face_means(sample_rows: torch.Tensor, num_interior: torch.Tensor) -> FaceMeans:
    """Cached mean over every face's samples of sample_rows (NiK, F) (num_interior = inclusive running sample
    count, as facet2facet takes it); same cache and budget as vertex_csr.  Forward and backward of a step share it."""
    nf, nik = num_interior.shape[0], sample_rows.shape[0]
    slot = ("face_means", sample_rows.device.index, sample_rows.data_ptr(), num_interior.data_ptr(), nik, nf,
            sample_rows.shape[1])
    versions = (sample_rows._version, num_interior._version)
    hit = _lookup(slot, versions)
    if hit is not None:
        return hit
    dev = sample_rows.device
    with torch.cuda.device(dev):
        check_num_interior(num_interior, nik)
        rows = torch.empty(nf, sample_rows.shape[1], dtype=torch.float32, device=dev)
        _lib.call("pb200_face_mean_rows", nf, nik, sample_rows.shape[1], ptr(sample_rows), ptr(num_interior), ptr(rows),
                  stream_ptr(dev))
        one_each = torch.arange(1, nf + 1, dtype=torch.int32, device=dev)
    fm = FaceMeans(rows, one_each, (sample_rows, num_interior), versions)
    _store(slot, fm)
    return fm


def face_means_sph_harm(L: int, sample_xyz: torch.Tensor, num_interior: torch.Tensor) -> FaceMeans:
    """face_means(sph_harm_coeff(L, sample_xyz), num_interior) in one kernel (identical bits), without the
    (NiK, (L+1)^2) array; cached the same way."""
    nf, nik = num_interior.shape[0], sample_xyz.shape[0]
    slot = ("face_means_sh", sample_xyz.device.index, sample_xyz.data_ptr(), num_interior.data_ptr(), nik, nf, int(L))
    versions = (sample_xyz._version, num_interior._version)
    hit = _lookup(slot, versions)
    if hit is not None:
        return hit
    if sample_xyz.dim() != 2 or sample_xyz.shape[1] != 3 or sample_xyz.dtype != torch.float32 or not sample_xyz.is_contiguous():
        raise RuntimeError("sample_xyz must be a contiguous float32 tensor of shape (NiK, 3)")
    dev = sample_xyz.device
    with torch.cuda.device(dev):
        check_num_interior(num_interior, nik)
        rows = torch.empty(nf, (L + 1) ** 2, dtype=torch.float32, device=dev)
        _lib.call("pb200_face_mean_sph_harm", nf, nik, int(L), ptr(sample_xyz), ptr(num_interior), ptr(rows), stream_ptr(dev))
        one_each = torch.arange(1, nf + 1, dtype=torch.int32, device=dev)
    fm = FaceMeans(rows, one_each, (sample_xyz, num_interior), versions)
    _store(slot, fm)
    return fm


def check_num_interior(num_interior: torch.Tensor, nik: int) -> None:
    """Validates a running sample count (non-decreasing, inside [0, nik], ends at nik) on the
    device: raises in 'sync' mode, queues the status word in 'deferred' mode.  The facet2facet
    kernels trust numInterior as the reference does; run this once per array."""
    dev = num_interior.device
    with torch.cuda.device(dev):
        status = torch.empty(1, dtype=torch.int32, device=dev)
        _lib.call("pb200_check_num_interior", num_interior.shape[0], int(nik), ptr(num_interior), ptr(status),
                  stream_ptr(dev))
        msg = f"numInterior is not a running count that ends at NiK={nik}"
        if _validation == "deferred":
            with _lock:
                _deferred.append((status, msg))
        elif int(status.item()) != 0:
            raise RuntimeError(msg)


def cache_stats():
    with _lock:
        return {"slots": len(_cache), "bytes": _cache_bytes, "budget": _budget_bytes}


def clear_cache() -> None:
    global _cache_bytes
    with _lock:
        _cache.clear()
        _cache_bytes = 0
