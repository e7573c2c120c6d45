"""Operator API of the mesh convolutions: same classes, functions, argument order and
return conventions as the reference's picasso/mesh/pi_modules/conv3d.py, with the CUDA
work done by libpicasso_b200.so through its C ABI.

Checks mirror the reference binding (picasso/mesh/pi_modules/source/mesh_conv3d.cpp:
27-30 CUDA / contiguous / rank, :56,:100 filter channels, :138,:170 three V2F filters,
:211 F <= 50, :212-213 bary shape); a violated check raises RuntimeError.
"""
from __future__ import annotations

import torch

from ... import _lib
from ...topology import vertex_csr, ptr, stream_ptr

_f2f_precision = _lib.PREC_FP32


def set_f2f_precision(name: str) -> None:
    """Operand precision of the facet2facet contraction: 'fp32' (default: bf16 hi+lo operands,
    meets the 1e-4 relative gate), 'fp32_tf32x3' (tf32 hi+lo operands, about 2e-6), 'tf32' or
    'bf16' (single tensor-core operands), 'fp32_ffma' (no tensor cores); fp32 accumulation always."""
    global _f2f_precision
    _f2f_precision = _lib.PRECISIONS[name]


def get_f2f_precision() -> str:
    return {v: k for k, v in _lib.PRECISIONS.items()}[_f2f_precision]


def _check(t, name, dims, dtype):
    if not isinstance(t, torch.Tensor) or not t.is_cuda:
        raise RuntimeError(f"{name} must be a CUDA tensor")
    if not t.is_contiguous():
        raise RuntimeError(f"{name} must be contiguous")
    if t.dim() != dims:
        raise RuntimeError(f"{name} must have dimension of {dims}")
    if t.dtype != dtype:
        raise RuntimeError(f"{name} must have dtype {dtype}, got {t.dtype}")


def _aligned16(t):
    """The tensor-core kernels copy rows with 16-byte vector and bulk copies; a contiguous view
    that starts off a 16-byte boundary (a slice of a larger tensor) is moved to fresh storage."""
    return t if t.data_ptr() % 16 == 0 else t.clone()


def _ws(nbytes, dev):
    return torch.empty(max(int(nbytes), 1), dtype=torch.uint8, device=dev)


# ------------------------------------------------------------------------------ raw ops
def facet2facet_forward(textureIn, filter, baryCoeff, numTexture):
    _check(textureIn, "input", 2, torch.float32)
    _check(filter, "filter", 3, torch.float32)
    _check(baryCoeff, "bary_coeff", 2, torch.float32)
    _check(numTexture, "num_texture", 1, torch.int32)
    NiK, Cin = textureIn.shape
    Cout, _, F = filter.shape
    Nf = numTexture.shape[0]
    if filter.shape[1] != Cin:
        raise RuntimeError("input Channel size error of the filter.")
    if F > 50:
        raise RuntimeError("A maximum of 50 filters are supported in face2face convolution.")
    if baryCoeff.shape[1] != F:
        raise RuntimeError("Dimension of bary_coeff mismatches number of filters.")
    if baryCoeff.shape[0] != NiK:
        raise RuntimeError("The shape of bary_coeff should be (NiK, Dim)).")
    textureIn = _aligned16(textureIn)
    dev = textureIn.device
    with torch.cuda.device(dev):
        out = torch.empty(Nf, Cout, dtype=textureIn.dtype, device=dev)
        nb = _lib.query("pb200_facet2facet_forward_workspace_bytes", Nf, NiK, Cin, Cout, F, _f2f_precision)
        ws = _ws(nb, dev)
        _lib.call("pb200_facet2facet_forward", Nf, NiK, Cin, Cout, F, ptr(textureIn), ptr(filter), ptr(baryCoeff),
                  ptr(numTexture), ptr(out), _f2f_precision, ptr(ws), nb, stream_ptr(dev))
    return out


def facet2facet_backward(grad_output, textureIn, filter, baryCoeff, numTexture, baryPadded=None):
    """baryPadded (not in the reference's signature): topology.pad_rows(baryCoeff), for callers that keep it."""
    _check(textureIn, "input", 2, torch.float32)
    _check(filter, "filter", 3, torch.float32)
    _check(grad_output, "grad_output", 2, torch.float32)
    _check(baryCoeff, "bary_coeff", 2, torch.float32)
    _check(numTexture, "num_texture", 1, torch.int32)
    NiK, Cin = textureIn.shape
    Cout, _, F = filter.shape
    Nf = numTexture.shape[0]
    if filter.shape[1] != Cin:
        raise RuntimeError("input Channel size error of the filter.")
    if baryCoeff.shape[1] != F:
        raise RuntimeError("Dimension of bary_coeff mismatches number of filters.")
    if baryCoeff.shape[0] != NiK:
        raise RuntimeError("The shape of bary_coeff should be (NiK, Dim)).")
    if tuple(grad_output.shape) != (Nf, Cout):
        raise RuntimeError("grad_output must have shape (NfIn, out_channels)")
    grad_output, textureIn, baryCoeff = _aligned16(grad_output), _aligned16(textureIn), _aligned16(baryCoeff)
    dev = textureIn.device
    with torch.cuda.device(dev):
        gin = torch.empty(NiK, Cin, dtype=textureIn.dtype, device=dev)
        gf = torch.empty(Cout, Cin, F, dtype=textureIn.dtype, device=dev)
        nb = _lib.query("pb200_facet2facet_backward_workspace_bytes", Nf, NiK, Cin, Cout, F, _f2f_precision)
        ws = _ws(nb, dev)
        if baryPadded is not None and tuple(baryPadded.shape) != (NiK, _lib.query("pb200_padded_row_floats", F)):
            raise RuntimeError("baryPadded must have shape (NiK, padded row length)")
        _lib.call("pb200_facet2facet_backward_padded", Nf, NiK, Cin, Cout, F, ptr(grad_output), ptr(textureIn), ptr(filter),
                  ptr(baryCoeff), ptr(baryPadded), ptr(numTexture), ptr(gin), ptr(gf), _f2f_precision, ptr(ws), nb,
                  stream_ptr(dev))
    return gin, gf


def vertex2facet_forward(input, filter, face):
    _check(input, "input", 2, torch.float32)
    _check(filter, "filter", 3, torch.float32)
    _check(face, "face", 2, torch.int32)
    Nv, Cc = input.shape
    r = filter.shape[2]
    Nf = face.shape[0]
    if filter.shape[0] != 3 or filter.shape[1] != Cc:
        raise RuntimeError("3 filters required, or input Channel size error of the filter")
    if Nf > 0 and face.shape[1] != 3:
        raise RuntimeError("face must have shape (NfIn, 3)")
    dev = input.device
    with torch.cuda.device(dev):
        out = torch.empty(Nf, Cc * r, dtype=input.dtype, device=dev)
        _lib.call("pb200_vertex2facet_forward", Nf, Nv, Cc, r, ptr(input), ptr(filter), ptr(face), ptr(out),
                  stream_ptr(dev))
    return out


def vertex2facet_backward(grad_output, input, filter, face, csr=None):
    _check(input, "input", 2, torch.float32)
    _check(filter, "filter", 3, torch.float32)
    _check(grad_output, "grad_output", 2, torch.float32)
    _check(face, "face", 2, torch.int32)
    Nv, Cc = input.shape
    r = filter.shape[2]
    Nf = face.shape[0]
    if filter.shape[0] != 3 or filter.shape[1] != Cc:
        raise RuntimeError("3 filters required, or input Channel size error of the filter")
    if tuple(grad_output.shape) != (Nf, Cc * r):
        raise RuntimeError("grad_output must have shape (NfIn, out_channels)")
    dev = input.device
    with torch.cuda.device(dev):
        if csr is None:
            csr = vertex_csr(face, None, Nv, Nv)
        gin = torch.empty(Nv, Cc, dtype=input.dtype, device=dev)
        gf = torch.empty(3, Cc, r, dtype=input.dtype, device=dev)
        nb = _lib.query("pb200_vertex2facet_backward_workspace_bytes", Nf, Nv, Cc, r)
        ws = _ws(nb, dev)
        _lib.call("pb200_vertex2facet_backward", Nf, Nv, Cc, r, ptr(grad_output), ptr(input), ptr(filter), ptr(face),
                  ptr(csr.rowptr), ptr(csr.entries), ptr(gin), ptr(gf), ptr(ws), nb, stream_ptr(dev))
    return gin, gf


def _f2v_checks(input, filter, coeff, face, nfCount, vtMap):
    _check(input, "input", 2, torch.float32)
    _check(filter, "filter", 3, torch.float32)
    _check(coeff, "coeff", 2, torch.float32)
    _check(face, "face", 2, torch.int32)
    _check(nfCount, "nf_count", 1, torch.int32)
    _check(vtMap, "vt_map", 1, torch.int32)
    if filter.shape[1] != input.shape[1]:
        raise RuntimeError("Input Channel size error of the filter")
    if coeff.shape[0] != input.shape[0] or coeff.shape[1] != filter.shape[0]:
        raise RuntimeError("coeff must have shape (NfIn, filter_size)")
    if face.shape[0] != input.shape[0] or (face.shape[0] > 0 and face.shape[1] != 3):
        raise RuntimeError("face must have shape (NfIn, 3)")


def facet2vertex_forward(input, filter, coeff, face, nfCount, vtMap, csr=None):
    _f2v_checks(input, filter, coeff, face, nfCount, vtMap)
    Nf, Cc = input.shape
    K, _, r = filter.shape
    NvOut, NvIn = nfCount.shape[0], vtMap.shape[0]
    dev = input.device
    with torch.cuda.device(dev):
        if csr is None:
            csr = vertex_csr(face, vtMap, NvIn, NvOut)
        out = torch.empty(NvOut, Cc * r, dtype=input.dtype, device=dev)
        nb = _lib.query("pb200_facet2vertex_forward_workspace_bytes", Nf, Cc, r, K)
        ws = _ws(nb, dev)
        _lib.call("pb200_facet2vertex_forward", Nf, NvOut, Cc, r, K, ptr(input), ptr(filter), ptr(coeff),
                  ptr(nfCount), ptr(csr.rowptr), ptr(csr.entries), ptr(out), ptr(ws), nb, stream_ptr(dev))
    return out


def facet2vertex_backward(grad_output, input, filter, coeff, face, nfCount, vtMap):
    _f2v_checks(input, filter, coeff, face, nfCount, vtMap)
    _check(grad_output, "grad_output", 2, torch.float32)
    Nf, Cc = input.shape
    K, _, r = filter.shape
    NvOut, NvIn = nfCount.shape[0], vtMap.shape[0]
    if tuple(grad_output.shape) != (NvOut, Cc * r):
        raise RuntimeError("grad_output must have shape (NvOut, out_channels)")
    dev = input.device
    with torch.cuda.device(dev):
        vertex_csr(face, vtMap, NvIn, NvOut)     # validates the indices once per topology
        gin = torch.empty(Nf, Cc, dtype=input.dtype, device=dev)
        gf = torch.empty(K, Cc, r, dtype=input.dtype, device=dev)
        nb = _lib.query("pb200_facet2vertex_backward_workspace_bytes", Nf, Cc, r, K)
        ws = _ws(nb, dev)
        _lib.call("pb200_facet2vertex_backward", Nf, NvIn, NvOut, Cc, r, K, ptr(grad_output), ptr(input),
                  ptr(filter), ptr(coeff), ptr(face), ptr(nfCount), ptr(vtMap), ptr(gin), ptr(gf), ptr(ws), nb,
                  stream_ptr(dev))
    return gin, gf


# ------------------------------------------------------------------ autograd Functions
class f2f_Function(torch.autograd.Function):
    @staticmethod
    def forward(ctx, textureIn, filter, baryCoeff, numTexture):
        baryCoeff.requires_grad = False
        numTexture.requires_grad = False
        output = facet2facet_forward(textureIn, filter, baryCoeff, numTexture)
        variables = [textureIn, filter, baryCoeff, numTexture]
        ctx.save_for_backward(*variables)
        return output

    @staticmethod
    def backward(ctx, grad_output):
        grad_input, grad_filter = facet2facet_backward(grad_output.contiguous(), *ctx.saved_tensors)
        return grad_input, grad_filter, None, None


def facet2facet(textureIn, filter, baryCoeff, numTexture):
    '''
    Compute the feature of each triangular face from its interior (texture) samples.
    Input:
        textureIn:   (concat_NiK, in_channels) float32, features of the interior samples,
                     grouped by face
        filter:      (out_channels, in_channels, F) float32, F = number of bases
        baryCoeff:   (concat_NiK, F) float32, basis values of every sample
        numTexture:  (concat_NfIn) int32, INCLUSIVE CUMULATIVE number of samples per face
    Output:
        output:      (concat_NfIn, out_channels) float32
    '''
    return f2f_Function.apply(textureIn, filter, baryCoeff, numTexture)


class v2f_Function(torch.autograd.Function):
    @staticmethod
    def forward(ctx, input, filter, face):
        face.requires_grad = False
        output = vertex2facet_forward(input, filter, face)
        variables = [input, filter, face]
        ctx.save_for_backward(*variables)
        return output

    @staticmethod
    def backward(ctx, grad_output):
        grad_input, grad_filter = vertex2facet_backward(grad_output.contiguous(), *ctx.saved_tensors)
        return grad_input, grad_filter, None


def vertex2facet(input, filter, face):
    '''
    Input:
        input:  (concat_NvIn, in_channels) float32, vertex features
        filter: (3, in_channels, multiplier) float32
        face:   (concat_NfIn, 3) int32, vertex list of each facet
    Output:
        output: (concat_NfIn, in_channels*multiplier) float32
    '''
    return v2f_Function.apply(input, filter, face)


class f2v_Function(torch.autograd.Function):
    @staticmethod
    def forward(ctx, input, filter, coeff, face, nfCount, vtMap):
        coeff.requires_grad = False
        face.requires_grad = False
        nfCount.requires_grad = False
        vtMap.requires_grad = False
        output = facet2vertex_forward(input, filter, coeff, face, nfCount, vtMap)
        variables = [input, filter, coeff, face, nfCount, vtMap]
        ctx.save_for_backward(*variables)
        return output

    @staticmethod
    def backward(ctx, grad_output):
        grad_input, grad_filter = facet2vertex_backward(grad_output.contiguous(), *ctx.saved_tensors)
        return grad_input, grad_filter, None, None, None, None


def facet2vertex(input, filter, coeff, face, nfCount, vtMap):
    '''
    Input:
        input:   (concat_NfIn, in_channels) float32, facet features
        filter:  (K, in_channels, multiplier) float32
        coeff:   (concat_NfIn, K) float32, basis coefficients of each facet
        face:    (concat_NfIn, 3) int32
        nfCount: (concat_NvOut) int32, number of adjacent faces of each output vertex
        vtMap:   (concat_NvIn) int32, input to output vertex index mapping (-1 = dropped)
    Output:
        output:  (concat_NvOut, in_channels*multiplier) float32
    '''
    return f2v_Function.apply(input, filter, coeff, face, nfCount, vtMap)
