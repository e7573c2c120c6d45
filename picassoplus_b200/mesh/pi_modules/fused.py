"""Operator + pointwise stage as one autograd Function each (no counterpart in the reference, whose
modules run operator -> torch.matmul -> + bias -> ReLU as separate kernels,
picasso/mesh/layers.py:109-120,166-175).  Forward: one fused tensor-core kernel; the operator's
(rows, C) output never exists in memory.  Backward: the operator's output is recomputed with the
stand-alone forward kernel (cheaper than having stored it); the gradient of the operator output is one
tensor-core kernel that applies the activation mask on the fly (pb200_masked_rows_matmul) and hands back the
masked gradient, from which the weight and bias gradients are reduced; the operator gradient is the
stand-alone backward kernel.
"""
from __future__ import annotations

import torch

from ... import _lib
from ...topology import ptr, stream_ptr, vertex_csr
from . import conv3d

_precision = _lib.PREC_FP32


def set_pointwise_precision(name: str) -> None:
    """'fp32' (default: bf16 hi+lo operands, about 1e-5 relative) or 'bf16'."""
    global _precision
    if name not in ("fp32", "bf16"):
        raise ValueError(name)
    _precision = _lib.PRECISIONS[name]


def eligible(x: torch.Tensor, channels: int, multiplier: int, activation_fn) -> bool:
    """The fused kernels take depth multiplier 1, channels that are a multiple of 8, and ReLU or no
    activation."""
    return (x.is_cuda and x.dtype == torch.float32 and multiplier == 1 and channels % 8 == 0 and
            (activation_fn is None or isinstance(activation_fn, torch.nn.ReLU)))


def _pointwise_backward(grad_out, out, feats, depth_weights, relu):
    """Gradients of out = act(feats @ depth_weights + bias): (d feats, d depth_weights, d bias).  The product
    with depth_weights^T runs on the tensor cores with the activation mask applied on the fly
    (pb200_masked_rows_matmul), which also hands back the masked gradient for the two reductions."""
    Nrows, Cout = grad_out.shape
    C = depth_weights.shape[0]
    if Cout % 8 != 0 or Nrows == 0:
        g = grad_out * (out > 0) if relu else grad_out
        return g @ depth_weights.t(), feats.t() @ g, g.sum(0, keepdim=True)
    dev = grad_out.device
    grad_out = conv3d._aligned16(grad_out)
    with torch.cuda.device(dev):
        g_feats = torch.empty(Nrows, C, dtype=grad_out.dtype, device=dev)
        g = torch.empty_like(grad_out) if relu else None
        wt = depth_weights.t().contiguous()
        nb = _lib.query("pb200_masked_rows_matmul_workspace_bytes", Cout, _precision)
        ws = torch.empty(max(nb, 1), dtype=torch.uint8, device=dev)
        _lib.call("pb200_masked_rows_matmul", Nrows, Cout, C, ptr(grad_out), ptr(out) if relu else None, ptr(wt),
                  ptr(g_feats), ptr(g), _precision, ptr(ws), nb, stream_ptr(dev))
    if g is None:
        g = grad_out
    g_w, g_b = rows_contract(feats, g)
    return g_feats, g_w, g_b


def rows_contract(a, b):
    """(a^T @ b, column sums of b as a (1, N) row) with the contraction over rows on the tensor cores
    (pb200_rows_contract); torch for widths that are no multiple of 4."""
    Nrows, M = a.shape
    N = b.shape[1]
    if M % 4 != 0 or N % 4 != 0 or Nrows == 0:
        return a.t() @ b, b.sum(0, keepdim=True)
    dev = a.device
    a, b = conv3d._aligned16(a), conv3d._aligned16(b)
    with torch.cuda.device(dev):
        out = torch.empty(M, N, dtype=a.dtype, device=dev)
        colsum = torch.empty(1, N, dtype=a.dtype, device=dev)
        nb = _lib.query("pb200_rows_contract_workspace_bytes", Nrows, M, N)
        ws = torch.empty(max(nb, 1), dtype=torch.uint8, device=dev)
        _lib.call("pb200_rows_contract", Nrows, M, N, ptr(a), ptr(b), ptr(out), ptr(colsum), _precision, ptr(ws), nb,
                  stream_ptr(dev))
    return out, colsum


class V2FPointwiseFunction(torch.autograd.Function):
    @staticmethod
    def forward(ctx, input, filter, face, depth_weights, biases, relu):
        face.requires_grad = False
        conv3d._check(input, "input", 2, torch.float32)
        conv3d._check(filter, "filter", 3, torch.float32)
        conv3d._check(face, "face", 2, torch.int32)
        conv3d._check(depth_weights, "depth_weights", 2, torch.float32)
        Nv, C = input.shape
        Nf, Cout = face.shape[0], depth_weights.shape[1]
        if tuple(filter.shape) != (3, C, 1) or depth_weights.shape[0] != C:
            raise RuntimeError("filter must have shape (3, C, 1) and depth_weights (C, out_channels)")
        dev = input.device
        input, filter = conv3d._aligned16(input), conv3d._aligned16(filter)
        bias = None if biases is None else biases.reshape(-1).contiguous()
        with torch.cuda.device(dev):
            out = torch.empty(Nf, Cout, dtype=input.dtype, device=dev)
            nb = _lib.query("pb200_vertex2facet_pointwise_workspace_bytes", C, _precision)
            ws = torch.empty(max(nb, 1), dtype=torch.uint8, device=dev)
            _lib.call("pb200_vertex2facet_pointwise_forward", Nf, Nv, C, Cout, ptr(input), ptr(filter), ptr(face),
                      ptr(depth_weights), ptr(bias), 1 if relu else 0, ptr(out), _precision, ptr(ws), nb, stream_ptr(dev))
        ctx.relu = relu
        ctx.has_bias = biases is not None
        ctx.save_for_backward(input, filter, face, depth_weights, out)
        return out

    @staticmethod
    def backward(ctx, grad_out):
        input, filter, face, depth_weights, out = ctx.saved_tensors
        feats = conv3d.vertex2facet_forward(input, filter, face)
        g_feats, g_w, g_b = _pointwise_backward(grad_out.contiguous(), out, feats, depth_weights, ctx.relu)
        g_in, g_filter = conv3d.vertex2facet_backward(g_feats.contiguous(), input, filter, face)
        return g_in, g_filter, None, g_w, (g_b if ctx.has_bias else None), None


class F2VPointwiseFunction(torch.autograd.Function):
    @staticmethod
    def forward(ctx, input, filter, coeff, face, nf_count, vt_map, depth_weights, biases, relu):
        for t in (coeff, face, nf_count, vt_map):
            t.requires_grad = False
        conv3d._f2v_checks(input, filter, coeff, face, nf_count, vt_map)
        conv3d._check(depth_weights, "depth_weights", 2, torch.float32)
        Nf, C = input.shape
        K = filter.shape[0]
        NvOut, NvIn, Cout = nf_count.shape[0], vt_map.shape[0], depth_weights.shape[1]
        if filter.shape[2] != 1 or depth_weights.shape[0] != C:
            raise RuntimeError("filter must have shape (K, C, 1) and depth_weights (C, out_channels)")
        dev = input.device
        input, filter = conv3d._aligned16(input), conv3d._aligned16(filter)
        bias = None if biases is None else biases.reshape(-1).contiguous()
        with torch.cuda.device(dev):
            csr = vertex_csr(face, vt_map, NvIn, NvOut)
            out = torch.empty(NvOut, Cout, dtype=input.dtype, device=dev)
            nb = _lib.query("pb200_facet2vertex_pointwise_workspace_bytes", Nf, C, _precision)
            ws = torch.empty(max(nb, 1), dtype=torch.uint8, device=dev)
            _lib.call("pb200_facet2vertex_pointwise_forward", Nf, NvOut, C, K, Cout, ptr(input), ptr(filter), ptr(coeff),
                      ptr(nf_count), ptr(csr.rowptr), ptr(csr.entries), ptr(depth_weights), ptr(bias), 1 if relu else 0,
                      ptr(out), _precision, ptr(ws), nb, stream_ptr(dev))
        ctx.relu = relu
        ctx.has_bias = biases is not None
        ctx.save_for_backward(input, filter, coeff, face, nf_count, vt_map, depth_weights, out)
        return out

    @staticmethod
    def backward(ctx, grad_out):
        input, filter, coeff, face, nf_count, vt_map, depth_weights, out = ctx.saved_tensors
        feats = conv3d.facet2vertex_forward(input, filter, coeff, face, nf_count, vt_map)
        g_feats, g_w, g_b = _pointwise_backward(grad_out.contiguous(), out, feats, depth_weights, ctx.relu)
        g_in, g_filter = conv3d.facet2vertex_backward(g_feats.contiguous(), input, filter, coeff, face, nf_count, vt_map)
        return g_in, g_filter, None, None, None, None, g_w, (g_b if ctx.has_bias else None), None


class RowsPointwiseFunction(torch.autograd.Function):
    """out = act(rows @ weights + biases): the pointwise layer (the reference's PerItemConv3d,
    picasso/mesh/layers.py:198-240) as one tensor-core kernel forward and two backward."""

    @staticmethod
    def forward(ctx, rows, weights, biases, relu):
        conv3d._check(rows, "inputs", 2, torch.float32)
        conv3d._check(weights, "weights", 2, torch.float32)
        Nrows, C = rows.shape
        Cout = weights.shape[1]
        if weights.shape[0] != C:
            raise RuntimeError("weights must have shape (in_channels, out_channels)")
        dev = rows.device
        rows = conv3d._aligned16(rows)
        bias = None if biases is None else biases.reshape(-1).contiguous()
        with torch.cuda.device(dev):
            out = torch.empty(Nrows, Cout, dtype=rows.dtype, device=dev)
            nb = _lib.query("pb200_masked_rows_matmul_workspace_bytes", C, _precision)
            ws = torch.empty(max(nb, 1), dtype=torch.uint8, device=dev)
            _lib.call("pb200_rows_pointwise_forward", Nrows, C, Cout, ptr(rows), ptr(weights), ptr(bias), 1 if relu else 0,
                      ptr(out), _precision, ptr(ws), nb, stream_ptr(dev))
        ctx.relu = relu
        ctx.has_bias = biases is not None
        ctx.save_for_backward(rows, weights, out)
        return out

    @staticmethod
    def backward(ctx, grad_out):
        rows, weights, out = ctx.saved_tensors
        g_rows, g_w, g_b = _pointwise_backward(grad_out.contiguous(), out, rows, weights, ctx.relu)
        return g_rows, g_w, (g_b if ctx.has_bias else None), None


def rows_pointwise(rows, weights, biases, relu):
    return RowsPointwiseFunction.apply(rows, weights, biases, relu)


def vertex2facet_pointwise(input, filter, face, depth_weights, biases, relu):
    return V2FPointwiseFunction.apply(input, filter, face, depth_weights, biases, relu)


def facet2vertex_pointwise(input, filter, coeff, face, nf_count, vt_map, depth_weights, biases, relu):
    return F2VPointwiseFunction.apply(input, filter, coeff, face, nf_count, vt_map, depth_weights, biases, relu)
