"""Per-topology device structures shared by the operators: the vertex -> (face, corner)
CSR and its cache.

A level's `face` / `vtMap` tensors are reused by every convolution of that level (4 to 16
operator calls per step in the reference's encoder blocks,
picasso/networks/pi2_blocks.py:88-92), so the CSR is built once per (face, vtMap) pair
and looked up afterwards.  Cache entries hold a reference to the index tensors they were
built from, so the memory behind a cached key cannot be recycled while the entry lives;
an in-place edit of an index tensor bumps its version counter and misses the cache.
"""
from __future__ import annotations

import threading
from collections import OrderedDict
from typing import Optional

import torch

from . import _lib

_CACHE_CAPACITY = 32
_cache: "OrderedDict[tuple, VertexCSR]" = OrderedDict()
_lock = threading.Lock()


def stream_ptr(device) -> int:
    return torch.cuda.current_stream(device).cuda_stream


def ptr(t: Optional[torch.Tensor]):
    return None if t is None else t.data_ptr()


class VertexCSR:
    """rowptr (NvOut+1,), entries (3*Nf,) int32: row v lists (f << 2 | corner) ascending."""

    def __init__(self, rowptr, entries, keep):
        self.rowptr = rowptr
        self.entries = entries
        self._keep = keep


def _key(face, vt_map, nv_in, nv_out):
    vk = None if vt_map is None else (vt_map.data_ptr(), vt_map._version, vt_map.shape[0])
    return (face.device.index, face.data_ptr(), face._version, face.shape[0], vk, int(nv_in), int(nv_out))


def build_vertex_csr(face: torch.Tensor, vt_map: Optional[torch.Tensor], nv_in: int, nv_out: int) -> VertexCSR:
    """Uncached build; validates every index and raises RuntimeError on an out-of-range one
    (one device synchronisation per topology)."""
    dev = face.device
    nf = face.shape[0]
    with torch.cuda.device(dev):
        rowptr = torch.empty(nv_out + 1, dtype=torch.int32, device=dev)
        entries = torch.empty(max(3 * nf, 1), dtype=torch.int32, device=dev)
        status = torch.empty(1, dtype=torch.int32, device=dev)
        wbytes = _lib.query("pb200_vertex_csr_workspace_bytes", nf, nv_out)
        ws = torch.empty(wbytes, dtype=torch.uint8, device=dev)
        _lib.call("pb200_build_vertex_csr", nf, nv_in, nv_out, ptr(face), ptr(vt_map), ptr(rowptr),
                  ptr(entries), ptr(status), ptr(ws), wbytes, stream_ptr(dev))
        code = int(status.item())
    if code != 0:
        raise RuntimeError("face / vtMap hold an index outside the vertex range "
                           f"(NvIn={nv_in}, NvOut={nv_out})")
    return VertexCSR(rowptr, entries, (face, vt_map))


def vertex_csr(face: torch.Tensor, vt_map: Optional[torch.Tensor], nv_in: int, nv_out: int) -> VertexCSR:
    """Cached CSR keyed by output vertex vo = vtMap[face[f][j]] (identity when vt_map is None).
    An identity vtMap over nv_in == nv_out vertices shares the entry of vt_map=None."""
    key = _key(face, vt_map, nv_in, nv_out)
    with _lock:
        hit = _cache.get(key)
        if hit is not None:
            _cache.move_to_end(key)
            return hit
    csr = None
    if vt_map is not None and nv_in == nv_out and vt_map.shape[0] == nv_in:
        ident = torch.arange(nv_in, dtype=vt_map.dtype, device=vt_map.device)
        if bool(torch.equal(vt_map, ident)):
            base = vertex_csr(face, None, nv_in, nv_out)
            csr = VertexCSR(base.rowptr, base.entries, (face, vt_map))
    if csr is None:
        csr = build_vertex_csr(face, vt_map, nv_in, nv_out)
    with _lock:
        _cache[key] = csr
        while len(_cache) > _CACHE_CAPACITY:
            _cache.popitem(last=False)
    return csr


def clear_cache() -> None:
    with _lock:
        _cache.clear()
