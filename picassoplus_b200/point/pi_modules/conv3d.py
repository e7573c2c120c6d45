"""Point-cloud depthwise convolution (hard and fuzzy filter-bin assignment): same classes, functions,
argument order and return conventions as the reference's picasso/point/pi_modules/conv3d.py, with
the CUDA work done by libpicasso_b200.so through its C ABI.

Checks mirror the reference binding (picasso/point/pi_modules/source/pcloud_conv3d.cpp:37-53,
175-195: CUDA / contiguous / rank of input (2), filter (3), nn_count (1), nn_index (2), bin_index
(1, fuzzy: 2), bin_coeff (2); filter.size(1) == channels); a violated check raises RuntimeError.
"""
from __future__ import annotations

import torch

from ... import _lib
from ...mesh.pi_modules.conv3d import _check
from ...topology import pair_csr, ptr, stream_ptr


def _checks(input, filter, nn_count, nn_index, bin_index, bin_coeff):
    _check(input, "input", 2, torch.float32)
    _check(filter, "filter", 3, torch.float32)
    _check(nn_count, "nn_count", 1, torch.int32)
    _check(nn_index, "nn_index", 2, torch.int32)
    if bin_coeff is None:
        _check(bin_index, "bin_index", 1, torch.int32)
    else:
        _check(bin_index, "bin_index", 2, torch.int32)
        _check(bin_coeff, "bin_coeff", 2, torch.float32)
        if tuple(bin_coeff.shape) != tuple(bin_index.shape):
            raise RuntimeError("bin_coeff and bin_index must have the same shape")
    if filter.shape[1] != input.shape[1]:
        raise RuntimeError("Input Channel size error of the filter")
    if nn_index.shape[0] > 0 and nn_index.shape[1] != 2:
        raise RuntimeError("nn_index must have shape (pairs, 2)")
    if bin_index.shape[0] != nn_index.shape[0]:
        raise RuntimeError("bin_index must have one row per neighbor pair")


def _forward(input, filter, nn_count, nn_index, bin_index, bin_coeff):
    _checks(input, filter, nn_count, nn_index, bin_index, bin_coeff)
    Np, C = input.shape
    F, _, r = filter.shape
    Mp, Nout = nn_count.shape[0], nn_index.shape[0]
    T = 1 if bin_coeff is None else bin_index.shape[1]
    dev = input.device
    with torch.cuda.device(dev):
        by_out = pair_csr(nn_index, 0, Mp)
        out = torch.empty(Mp, C * r, dtype=input.dtype, device=dev)
        _lib.call("pb200_pcloud_conv3d_forward", Np, Mp, Nout, F, C, r, T, ptr(input), ptr(filter), ptr(nn_count),
                  ptr(nn_index), ptr(bin_index), ptr(bin_coeff), ptr(by_out.rowptr), ptr(by_out.members), ptr(out),
                  stream_ptr(dev))
    return out


def _backward(grad_output, input, filter, nn_count, nn_index, bin_index, bin_coeff):
    _checks(input, filter, nn_count, nn_index, bin_index, bin_coeff)
    _check(grad_output, "grad_output", 2, torch.float32)
    Np, C = input.shape
    F, _, r = filter.shape
    Mp, Nout = nn_count.shape[0], nn_index.shape[0]
    T = 1 if bin_coeff is None else bin_index.shape[1]
    if tuple(grad_output.shape) != (Mp, C * r):
        raise RuntimeError("grad_output must have shape (output points, out_channels)")
    dev = input.device
    with torch.cuda.device(dev):
        by_in = pair_csr(nn_index, 1, Np)
        gin = torch.empty(Np, C, dtype=input.dtype, device=dev)
        gf = torch.empty(F, C, r, dtype=input.dtype, device=dev)
        nb = _lib.query("pb200_pcloud_conv3d_backward_workspace_bytes", Nout, F, C, r)
        ws = torch.empty(max(nb, 1), dtype=torch.uint8, device=dev)
        _lib.call("pb200_pcloud_conv3d_backward", Np, Mp, Nout, F, C, r, T, ptr(grad_output), ptr(input), ptr(filter),
                  ptr(nn_count), ptr(nn_index), ptr(bin_index), ptr(bin_coeff), ptr(by_in.rowptr), ptr(by_in.members),
                  ptr(gin), ptr(gf), ptr(ws), nb, stream_ptr(dev))
    return gin, gf


def SPH3D_forward(input, filter, nn_count, nn_index, bin_index):
    return _forward(input, filter, nn_count, nn_index, bin_index, None)


def SPH3D_backward(grad_output, input, filter, nn_count, nn_index, bin_index):
    return _backward(grad_output, input, filter, nn_count, nn_index, bin_index, None)


def fuzzySPH3D_forward(input, filter, nn_count, nn_index, bin_index, bin_coeff):
    return _forward(input, filter, nn_count, nn_index, bin_index, bin_coeff)


def fuzzySPH3D_backward(grad_output, input, filter, nn_count, nn_index, bin_index, bin_coeff):
    return _backward(grad_output, input, filter, nn_count, nn_index, bin_index, bin_coeff)


class ConvFunction(torch.autograd.Function):
    @staticmethod
    def forward(ctx, input, filter, nn_count, nn_index, bin_index):
        nn_count.requires_grad = False
        nn_index.requires_grad = False
        bin_index.requires_grad = False
        output = SPH3D_forward(input, filter, nn_count, nn_index, bin_index)
        variables = [input, filter, nn_count, nn_index, bin_index]
        ctx.save_for_backward(*variables)
        return output

    @staticmethod
    def backward(ctx, grad_output):
        grad_input, grad_filter = SPH3D_backward(grad_output.contiguous(), *ctx.saved_tensors)
        return grad_input, grad_filter, None, None, None


def conv3d(input, filter, nn_count, nn_index, bin_index):
    return ConvFunction.apply(input, filter, nn_count, nn_index, bin_index)


class FuzzyConv3dFunction(torch.autograd.Function):
    @staticmethod
    def forward(ctx, input, filter, nn_count, nn_index, bin_index, bin_coeff):
        nn_count.requires_grad = False
        nn_index.requires_grad = False
        bin_index.requires_grad = False
        bin_coeff.requires_grad = False
        output = fuzzySPH3D_forward(input, filter, nn_count, nn_index, bin_index, bin_coeff)
        variables = [input, filter, nn_count, nn_index, bin_index, bin_coeff]
        ctx.save_for_backward(*variables)
        return output

    @staticmethod
    def backward(ctx, grad_output):
        grad_input, grad_filter = fuzzySPH3D_backward(grad_output.contiguous(), *ctx.saved_tensors)
        return grad_input, grad_filter, None, None, None, None


def fuzzyconv3d(input, filter, nn_count, nn_index, bin_index, bin_coeff):
    return FuzzyConv3dFunction.apply(input, filter, nn_count, nn_index, bin_index, bin_coeff)
