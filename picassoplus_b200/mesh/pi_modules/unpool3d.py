"""Mesh unpooling (interpolation from the coarse level back to the fine level): same class,
function, argument order and return conventions as the reference's
picasso/mesh/pi_modules/unpool3d.py, with the CUDA work done by libpicasso_b200.so.

Checks mirror the reference binding (picasso/mesh/pi_modules/source/mesh_unpool3d.cpp:
CUDA / contiguous / rank for input (2), vt_replace (1), vt_map (1)); the fine level has
vt_map.shape[0] vertices, the coarse level input.shape[0].
"""
from __future__ import annotations

import torch

from ... import _lib
from ...topology import cluster_csr, ptr, stream_ptr
from .conv3d import _check


def forward(input, vt_replace, vt_map):
    _check(input, "input", 2, torch.float32)
    _check(vt_replace, "vt_replace", 1, torch.int32)
    _check(vt_map, "vt_map", 1, torch.int32)
    nv_coarse, C = input.shape
    nv_fine = vt_map.shape[0]
    if vt_replace.shape[0] != nv_fine:
        raise RuntimeError("vt_replace and vt_map must have one entry per fine vertex")
    dev = input.device
    with torch.cuda.device(dev):
        cl = cluster_csr(vt_replace, vt_map, nv_coarse)
        out = torch.empty(nv_fine, C, dtype=input.dtype, device=dev)
        _lib.call("pb200_mesh_unpool_forward", nv_coarse, nv_fine, C, ptr(input), ptr(cl.key), ptr(out), stream_ptr(dev))
    return out


def backward(grad_output, input, vt_replace, vt_map):
    _check(grad_output, "grad_output", 2, torch.float32)
    _check(input, "input", 2, torch.float32)
    _check(vt_replace, "vt_replace", 1, torch.int32)
    _check(vt_map, "vt_map", 1, torch.int32)
    nv_coarse, C = input.shape
    nv_fine = vt_map.shape[0]
    if tuple(grad_output.shape) != (nv_fine, C):
        raise RuntimeError("grad_output must have shape (fine vertices, channels)")
    dev = input.device
    with torch.cuda.device(dev):
        cl = cluster_csr(vt_replace, vt_map, nv_coarse)
        gin = torch.empty(nv_coarse, C, dtype=input.dtype, device=dev)
        _lib.call("pb200_mesh_unpool_backward", nv_coarse, nv_fine, C, ptr(grad_output), ptr(cl.rowptr), ptr(cl.members),
                  ptr(gin), stream_ptr(dev))
    return gin


class InterpolateFunction(torch.autograd.Function):
    @staticmethod
    def forward(ctx, input, vt_replace, vt_map):
        vt_replace.requires_grad = False
        vt_map.requires_grad = False
        output = forward(input, vt_replace, vt_map)
        variables = [input, vt_replace, vt_map]
        ctx.save_for_backward(*variables)
        return output

    @staticmethod
    def backward(ctx, grad_output):
        grad_input = backward(grad_output.contiguous(), *ctx.saved_tensors)
        return grad_input, None, None


def interpolate(input, vt_replace, vt_map):
    return InterpolateFunction.apply(input, vt_replace, vt_map)
