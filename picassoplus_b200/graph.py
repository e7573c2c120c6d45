"""CUDA-graph replay of a mesh-convolution step.

Small batches are launch-bound: the V2F -> F2F -> F2V block is 15 kernel launches plus the
autograd bookkeeping around them, about half a millisecond of host time whatever the mesh
size.  The operators of this package launch on the current stream, allocate their outputs
and workspaces through the torch caching allocator and never synchronise once the vertex
CSR of a topology is cached, so a whole forward + backward step can be captured into one
CUDA graph and replayed with a single launch.

    step = GraphedStep(fn)      # fn() reads its inputs from fixed tensors and leaves its
    step()                      # results (outputs, .grad of leaf tensors) in fixed tensors

The caller keeps inputs in place (copy new data INTO the captured tensors), must run the
step eagerly once per topology before capturing, so that every cache is warm, and must not
keep a tensor that references the autograd graph of an earlier step alive (detach what is
kept): autograd ties its gradient-accumulation nodes to the stream they were created on.
"""
from __future__ import annotations

from typing import Callable

import torch


class GraphedStep:
    def __init__(self, fn: Callable[[], None], warmup: int = 3):
        self.fn = fn
        dev = torch.cuda.current_device()
        side = torch.cuda.Stream(device=dev)
        side.wait_stream(torch.cuda.current_stream(dev))
        with torch.cuda.stream(side):                # warm-up off the capturing stream
            for _ in range(max(warmup, 1)):
                fn()
        torch.cuda.current_stream(dev).wait_stream(side)
        torch.cuda.synchronize(dev)
        self.graph = torch.cuda.CUDAGraph()
        with torch.cuda.graph(self.graph):
            fn()

    def __call__(self) -> None:
        self.graph.replay()
