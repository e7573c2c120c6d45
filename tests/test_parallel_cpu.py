"""Mesh-level data parallelism on CPU ranks (gloo, world_size 2): shards of whole meshes,
re-based faces, and the flat all-reduce of filter gradients reproduce the whole-batch
result.  The per-rank operator math is done by the oracle (the checker), the sharding and
the collective by the product code."""
import os
import socket

import numpy as np
import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

from conftest import rel_err
from picassoplus_b200 import synth
from picassoplus_b200.parallel import FilterGradAllReduce, partition_meshes, shard_batch


def test_partition_covers_all_meshes():
    for counts, world in [([10] * 32, 8), ([10] * 32, 3), ([5, 50, 5, 5, 5, 30], 3), ([7] * 5, 2), ([3], 1)]:
        parts = partition_meshes(counts, world)
        assert len(parts) == world
        assert parts[0][0] == 0 and sum(c for _, c in parts) == len(counts)
        for (a, n), (b, _) in zip(parts, parts[1:]):
            assert a + n == b
    assert partition_meshes([10] * 32, 8) == [(4 * r, 4) for r in range(8)]


def _free_port():
    s = socket.socket()
    s.bind(("127.0.0.1", 0))
    p = s.getsockname()[1]
    s.close()
    return p


def _worker(rank, world, port, q):
    from oracle import mesh_oracle as mo
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
    dist.init_process_group("gloo", rank=rank, world_size=world)
    torch.set_num_threads(1)
    mb = synth.icosphere_batch(5, 1, seed=3, mode="noise_rot")
    g = torch.Generator().manual_seed(0)
    C, K = 6, 4
    x = torch.randn(mb.num_vertices, C, generator=g, dtype=torch.double)
    Wv = torch.randn(3, C, 1, generator=g, dtype=torch.double)
    Wo = torch.randn(K, C, 1, generator=g, dtype=torch.double)
    coeff = torch.randn(mb.num_faces, K, generator=g, dtype=torch.double)
    G = torch.randn(mb.num_vertices, C, generator=g, dtype=torch.double)
    vertex, face = torch.from_numpy(mb.vertex), torch.from_numpy(mb.face)
    nv, mf = torch.from_numpy(mb.nv), torch.from_numpy(mb.mf)

    def run(vx, fc, xs, cs, Gs):
        wv, wo = Wv.clone().requires_grad_(), Wo.clone().requires_grad_()
        vt = torch.arange(vx.shape[0], dtype=torch.int32)
        nfc = mo.count_vertex_adjface(fc, vt, vx.shape[0])
        y = mo.vertex2facet(xs, wv, fc)
        o = mo.facet2vertex(y, wo, cs, fc, nfc, vt)
        (o * Gs).sum().backward()
        return o.detach(), wv, wo

    first, count = partition_meshes(mb.mf.tolist(), world)[rank]
    vx, fc, _, _, (v0, v1, f0, f1) = shard_batch(vertex, face, nv, mf, first, count)
    o, wv, wo = run(vx, fc, x[v0:v1], coeff[f0:f1], G[v0:v1])
    FilterGradAllReduce([wv, wo])()
    o_full, wv_full, wo_full = run(vertex, face, x, coeff, G)
    ok = (rel_err(o, o_full[v0:v1]) < 1e-12 and rel_err(wv.grad, wv_full.grad) < 1e-12
          and rel_err(wo.grad, wo_full.grad) < 1e-12)
    q.put((rank, bool(ok), int(fc.min()), int(fc.max()), vx.shape[0]))
    dist.destroy_process_group()


def test_two_rank_gloo_matches_whole_batch():
    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    port = _free_port()
    procs = [ctx.Process(target=_worker, args=(r, 2, port, q)) for r in range(2)]
    for p in procs:
        p.start()
    res = [q.get(timeout=120) for _ in procs]
    for p in procs:
        p.join(timeout=60)
        assert p.exitcode == 0
    for rank, ok, fmin, fmax, nvs in res:
        assert ok, f"rank {rank} disagrees with the whole-batch result"
        assert fmin == 0 and fmax == nvs - 1      # faces were re-based to the shard
