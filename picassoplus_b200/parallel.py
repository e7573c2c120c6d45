"""Mesh-level data parallelism: whole meshes per rank, one all-reduce of filter gradients.

A batch is a concatenation of disjoint meshes (reference: picasso/mesh/dataset_shape.py:
43-58); no operator couples faces or vertices of different meshes, so ranks take
contiguous mesh ranges, re-base the vertex ids of their faces, and run the operators
unchanged.  The only exchange is the sum of the filter gradients, sent as one flat buffer
(NCCL on GPUs, gloo in the CPU tests).  For a fixed world size the result is
deterministic; across world sizes it differs by fp32 re-association.
"""
from __future__ import annotations

from typing import List, Sequence, Tuple

import torch
import torch.distributed as dist


def partition_meshes(face_counts: Sequence[int], world_size: int) -> List[Tuple[int, int]]:
    """Contiguous mesh ranges [(first, count)] per rank, balanced by face count: rank r ends
    at the first mesh boundary whose cumulative face count reaches (r+1)/world of the total.
    Every rank gets at least one mesh when there are enough meshes."""
    n = len(face_counts)
    total = float(sum(face_counts))
    bounds = [0]
    run = 0.0
    i = 0
    for r in range(1, world_size):
        target = total * r / world_size
        while i < n and run + face_counts[i] / 2.0 <= target:
            run += face_counts[i]
            i += 1
        lo = bounds[-1] + (1 if n - bounds[-1] > world_size - r else 0)   # leave meshes for the ranks after
        i = max(i, min(lo, n))
        i = min(i, n - (world_size - r)) if n >= world_size else min(i, n)
        i = max(i, bounds[-1])
        run = float(sum(face_counts[:i]))
        bounds.append(i)
    bounds.append(n)
    return [(bounds[r], bounds[r + 1] - bounds[r]) for r in range(world_size)]


def shard_batch(vertex: torch.Tensor, face: torch.Tensor, nv: torch.Tensor, mf: torch.Tensor,
                first: int, count: int):
    """The sub-batch of meshes [first, first+count): vertex rows, faces with vertex ids
    re-based to the shard, and the per-mesh counts."""
    voff = torch.cat([torch.zeros(1, dtype=torch.long), torch.cumsum(nv.long().cpu(), 0)])
    foff = torch.cat([torch.zeros(1, dtype=torch.long), torch.cumsum(mf.long().cpu(), 0)])
    v0, v1 = int(voff[first]), int(voff[first + count])
    f0, f1 = int(foff[first]), int(foff[first + count])
    return vertex[v0:v1], (face[f0:f1] - v0).to(face.dtype), nv[first:first + count], mf[first:first + count], (v0, v1, f0, f1)


def bind_to_gpu_cpus(device_index: int) -> int:
    """Restricts the calling process to the CPU cores that NVML reports as near GPU `device_index`, so that host
    buffers allocated afterwards (pinned staging memory above all) come from that socket's memory and a rank's
    host-to-device copies do not cross the socket link.  Read-only towards the GPU (no setting is changed); returns the
    number of cores bound to, or 0 when NVML or the affinity call is not available (the process then keeps its
    affinity)."""
    import os
    try:
        import pynvml
        pynvml.nvmlInit()
        try:
            visible = os.environ.get("CUDA_VISIBLE_DEVICES")
            index = device_index
            if visible:
                entry = visible.split(",")[device_index].strip()
                if entry.isdigit():
                    index = int(entry)
                    handle = pynvml.nvmlDeviceGetHandleByIndex(index)
                else:
                    handle = pynvml.nvmlDeviceGetHandleByUUID(entry.encode() if isinstance(entry, str) else entry)
            else:
                handle = pynvml.nvmlDeviceGetHandleByIndex(index)
            words = (os.cpu_count() + 63) // 64
            mask = pynvml.nvmlDeviceGetCpuAffinity(handle, words)
        finally:
            pynvml.nvmlShutdown()
        cpus = {64 * w + b for w, word in enumerate(mask) for b in range(64) if (int(word) >> b) & 1}
        cpus &= set(os.sched_getaffinity(0))
        if not cpus:
            return 0
        os.sched_setaffinity(0, cpus)
        return len(cpus)
    except Exception:
        return 0


class FilterGradAllReduce:
    """Sums the gradients of a fixed list of (filter) parameters over the process group in
    one collective on a flat buffer that is allocated once."""

    def __init__(self, params: Sequence[torch.Tensor], group=None):
        self.params = list(params)
        self.group = group
        self.sizes = [p.numel() for p in self.params]
        p0 = self.params[0]
        self.flat = torch.zeros(sum(self.sizes), dtype=p0.dtype, device=p0.device)
        self.views = []
        off = 0
        for p, n in zip(self.params, self.sizes):
            self.views.append(self.flat[off:off + n].view(p.shape))
            off += n

    @property
    def nbytes(self) -> int:
        return self.flat.numel() * self.flat.element_size()

    def __call__(self) -> None:
        """Replace every .grad by the sum over ranks (no-op for a single process)."""
        if not dist.is_available() or not dist.is_initialized() or dist.get_world_size(self.group) == 1:
            return
        for p, v in zip(self.params, self.views):
            if p.grad is None:
                v.zero_()
            else:
                v.copy_(p.grad)
        dist.all_reduce(self.flat, op=dist.ReduceOp.SUM, group=self.group)
        for p, v in zip(self.params, self.views):
            if p.grad is None:
                p.grad = v.clone()
            else:
                p.grad.copy_(v)


class HostBatchFeed:
    """Double-buffered host-to-device feed for a sequence of mesh batches that live in pinned
    host memory: while the caller's stream computes batch g, batch g+1 is copied on a side
    stream into the other device buffer.  Iterating yields, per batch, a dict of device
    tensors (views of the buffers, valid until the next batch is requested).

    The batches of one step are independent under the mesh convolutions (filter gradients
    accumulate over them), so a step over all of them equals a step over their concatenation.
    """

    def __init__(self, pinned_batches: Sequence[dict], device: torch.device, depth: int = 2):
        assert depth >= 1 and len(pinned_batches) > 0
        self.batches = list(pinned_batches)
        self.device = device
        self.depth = depth
        self.copy_stream = torch.cuda.Stream(device=device)
        keys = list(self.batches[0].keys())
        self.bufs = []
        for _ in range(depth):                 # also for a single batch: cycle() copies pass p+1 during pass p
            buf = {}
            for k in keys:
                rows = max(b[k].shape[0] for b in self.batches)
                t0 = self.batches[0][k]
                buf[k] = torch.empty((rows,) + tuple(t0.shape[1:]), dtype=t0.dtype, device=device)
            self.bufs.append(buf)
        self.free = [None] * len(self.bufs)
        self.bytes_per_pass = sum(t.numel() * t.element_size() for b in self.batches for t in b.values())

    def _issue(self, i: int) -> torch.cuda.Event:
        """Copies batch i % len(batches) into buffer i % len(bufs) on the copy stream."""
        g, slot = i % len(self.batches), i % len(self.bufs)
        with torch.cuda.stream(self.copy_stream):
            if self.free[slot] is not None:
                self.copy_stream.wait_event(self.free[slot])
            for k, t in self.batches[g].items():
                self.bufs[slot][k][: t.shape[0]].copy_(t, non_blocking=True)
            ev = torch.cuda.Event()
            ev.record(self.copy_stream)
        return ev

    def _run(self, total):
        """Yields batches with running index 0, 1, ... (batch = index modulo the number of batches);
        `total` = how many to yield, None = without end."""
        n, nb = len(self.batches), len(self.bufs)
        cur = torch.cuda.current_stream(self.device)
        ahead = nb if total is None else min(nb, total)
        copied = {i: self._issue(i) for i in range(ahead)}
        i = 0
        while total is None or i < total:
            cur.wait_event(copied.pop(i))
            slot, g = i % nb, i % n
            yield {k: self.bufs[slot][k][: t.shape[0]] for k, t in self.batches[g].items()}
            done = torch.cuda.Event()
            done.record(cur)
            self.free[slot] = done
            if total is None or i + nb < total:
                copied[i + nb] = self._issue(i + nb)
            i += 1

    def __iter__(self):
        """One pass over the batches."""
        return self._run(len(self.batches))

    def cycle(self):
        """Endless iterator over pass after pass (a training loop over the same pinned batches):
        the copy of the first batch of the next pass overlaps the last batch of the current one,
        so no pass starts with an exposed copy."""
        return self._run(None)
