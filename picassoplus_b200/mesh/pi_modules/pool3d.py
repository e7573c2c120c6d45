"""Mesh pooling over decimation clusters: same classes, functions, argument order and
return conventions as the reference's picasso/mesh/pi_modules/pool3d.py, with the CUDA
work done by libpicasso_b200.so through its C ABI.

Checks mirror the reference binding (picasso/mesh/pi_modules/source/mesh_pool3d.cpp:
CHECK_INPUT = CUDA / contiguous / rank for input (2), vt_replace (1), vt_map (1), vt_out (2));
a violated check raises RuntimeError.  vt_out is used for its row count only, as there.
"""
from __future__ import annotations

import torch

from ... import _lib
from ...topology import cluster_csr, ptr, stream_ptr
from .conv3d import _check


def _pool_checks(input, vt_replace, vt_map, vt_out):
    _check(input, "input", 2, torch.float32)
    _check(vt_replace, "vt_replace", 1, torch.int32)
    _check(vt_map, "vt_map", 1, torch.int32)
    if not isinstance(vt_out, torch.Tensor) or not vt_out.is_cuda or vt_out.dim() != 2 or not vt_out.is_contiguous():
        raise RuntimeError("vt_out must be a contiguous CUDA tensor of dimension 2")
    if vt_replace.shape[0] != input.shape[0] or vt_map.shape[0] != input.shape[0]:
        raise RuntimeError("vt_replace and vt_map must have one entry per input vertex")


def max_forward(input, vt_replace, vt_map, vt_out, return_clusters=False):
    _pool_checks(input, vt_replace, vt_map, vt_out)
    nv_in, C = input.shape
    nv_out = vt_out.shape[0]
    dev = input.device
    with torch.cuda.device(dev):
        cl = cluster_csr(vt_replace, vt_map, nv_out)
        out = torch.empty(nv_out, C, dtype=input.dtype, device=dev)
        max_index = torch.empty(nv_out, C, dtype=torch.int32, device=dev)
        _lib.call("pb200_mesh_max_pool_forward", nv_in, nv_out, C, ptr(input), ptr(cl.rowptr), ptr(cl.members),
                  ptr(out), ptr(max_index), stream_ptr(dev))
    if return_clusters:
        return out, max_index, cl
    return out, max_index


def max_backward(grad_output, input, max_index, clusters=None):
    """clusters: the ClusterCSR the forward pooled over (the autograd function keeps it); with it the gradient is a
    gather over the fine vertices instead of a zero fill and a scatter. Same result."""
    _check(grad_output, "grad_output", 2, torch.float32)
    _check(input, "input", 2, torch.float32)
    _check(max_index, "max_index", 2, torch.int32)
    nv_in, C = input.shape
    nv_out = grad_output.shape[0]
    if tuple(max_index.shape) != (nv_out, C) or grad_output.shape[1] != C:
        raise RuntimeError("grad_output and max_index must have shape (NvOut, channels)")
    dev = input.device
    with torch.cuda.device(dev):
        gin = torch.empty(nv_in, C, dtype=input.dtype, device=dev)
        if clusters is not None and clusters.rowptr.shape[0] == nv_out + 1 and clusters.key.shape[0] >= nv_in:
            _lib.call("pb200_mesh_max_pool_backward_clusters", nv_in, nv_out, C, ptr(max_index), ptr(grad_output),
                      ptr(clusters.key), ptr(clusters.rowptr), ptr(gin), stream_ptr(dev))
        else:
            _lib.call("pb200_mesh_max_pool_backward", nv_in, nv_out, C, ptr(max_index), ptr(grad_output), ptr(gin),
                      stream_ptr(dev))
    return gin


def avg_forward(input, vt_replace, vt_map, vt_out):
    _pool_checks(input, vt_replace, vt_map, vt_out)
    nv_in, C = input.shape
    nv_out = vt_out.shape[0]
    dev = input.device
    with torch.cuda.device(dev):
        cl = cluster_csr(vt_replace, vt_map, nv_out)
        out = torch.empty(nv_out, C, dtype=input.dtype, device=dev)
        _lib.call("pb200_mesh_avg_pool_forward", nv_in, nv_out, C, ptr(input), ptr(vt_replace), ptr(cl.rowptr),
                  ptr(cl.members), ptr(out), stream_ptr(dev))
    return out


def avg_backward(grad_output, input, vt_replace, vt_map):
    _check(grad_output, "grad_output", 2, torch.float32)
    _check(input, "input", 2, torch.float32)
    _check(vt_replace, "vt_replace", 1, torch.int32)
    _check(vt_map, "vt_map", 1, torch.int32)
    nv_in, C = input.shape
    nv_out = grad_output.shape[0]
    dev = input.device
    with torch.cuda.device(dev):
        cl = cluster_csr(vt_replace, vt_map, nv_out)
        gin = torch.empty(nv_in, C, dtype=input.dtype, device=dev)
        _lib.call("pb200_mesh_avg_pool_backward", nv_in, nv_out, C, ptr(grad_output), ptr(vt_replace), ptr(cl.key),
                  ptr(gin), stream_ptr(dev))
    return gin


class MaxPoolFunction(torch.autograd.Function):
    @staticmethod
    def forward(ctx, input, vt_replace, vt_map, vt_out):
        vt_replace.requires_grad = False
        vt_map.requires_grad = False
        vt_out.requires_grad = False
        output, max_index, ctx.clusters = max_forward(input, vt_replace, vt_map, vt_out, return_clusters=True)
        variables = [input, max_index]
        ctx.save_for_backward(*variables)
        return output

    @staticmethod
    def backward(ctx, grad_output):
        input, max_index = ctx.saved_tensors
        grad_input = max_backward(grad_output.contiguous(), input, max_index, ctx.clusters)
        return grad_input, None, None, None


def maxPool(input, vt_replace, vt_map, vt_out):
    return MaxPoolFunction.apply(input, vt_replace, vt_map, vt_out)


class AvgPoolFunction(torch.autograd.Function):
    @staticmethod
    def forward(ctx, input, vt_replace, vt_map, vt_out):
        vt_replace.requires_grad = False
        vt_map.requires_grad = False
        vt_out.requires_grad = False
        output = avg_forward(input, vt_replace, vt_map, vt_out)
        variables = [input, vt_replace, vt_map]
        ctx.save_for_backward(*variables)
        return output

    @staticmethod
    def backward(ctx, grad_output):
        grad_input = avg_backward(grad_output.contiguous(), *ctx.saved_tensors)
        return grad_input, None, None, None


def avgPool(input, vt_replace, vt_map, vt_out):
    return AvgPoolFunction.apply(input, vt_replace, vt_map, vt_out)
