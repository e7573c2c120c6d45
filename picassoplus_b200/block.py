"""The benchmark's V2F -> F2F -> F2V block, chained through the public autograd Functions.

The reference has no such composite module; the block is defined as
    y   = vertex2facet(x, (SH(eye3) @ Wv) viewed as (3, Cin, 1), face)
    tex = y[f] repeated once per texture sample of face f
    z   = facet2facet(tex, Wf (Cout,Cin,K), SH(barycentrics), running sample count)
    o   = facet2vertex(z, Wo (K,Cout,1), SH(face normals), face, nfCount, vtMap)

conv_block_expanded runs it as written (row expansion, then the general facet2facet).  conv_block folds the
repetition into the operator: all samples of a face carry the same row, so the face operand of facet2facet,
(1/T_f) sum_k bary[k,d] tex[k,ci], is mean_k(bary[k,d]) * y[f,ci]; facet2facet over (y, per-face mean rows, one sample
per face) gives the same z and the same gradients for y and Wf, without writing or reading the expanded rows and
with one product per operand element instead of one multiply-add per sample.
"""
from __future__ import annotations

import torch

from . import _lib
from .mesh.pi_modules import conv3d
from .topology import FaceMeans, face_means, ptr, stream_ptr


class _ExpandRows(torch.autograd.Function):
    """out[k] = in[f] for every sample k of face f (torch.repeat_interleave with a fixed-order,
    atomics-free backward)."""

    @staticmethod
    def forward(ctx, inp, cum, n_samples):
        inp = inp.contiguous()
        ctx.save_for_backward(cum)
        ctx.shape = inp.shape
        dev = inp.device
        with torch.cuda.device(dev):
            out = torch.empty(n_samples, inp.shape[1], dtype=inp.dtype, device=dev)
            _lib.call("pb200_expand_rows_forward", inp.shape[0], n_samples, inp.shape[1], ptr(inp), ptr(cum), ptr(out),
                      stream_ptr(dev))
        return out

    @staticmethod
    def backward(ctx, g):
        (cum,) = ctx.saved_tensors
        g = g.contiguous()
        dev = g.device
        with torch.cuda.device(dev):
            gin = torch.empty(ctx.shape, dtype=g.dtype, device=dev)
            _lib.call("pb200_expand_rows_backward", ctx.shape[0], g.shape[0], ctx.shape[1], ptr(g), ptr(cum), ptr(gin),
                      stream_ptr(dev))
        return gin, None, None


def expand_rows(inp, cum, n_samples):
    return _ExpandRows.apply(inp, cum, n_samples)


def conv_block_expanded(x, Wv, Wf, Wo, face, cum, bary_sh, coeff, nf_count, vt_map, sh_eye):
    cin = x.shape[1]
    spatial = (sh_eye @ Wv).reshape(3, cin, 1)
    y = conv3d.vertex2facet(x, spatial, face)
    tex = expand_rows(y, cum, bary_sh.shape[0])
    z = conv3d.facet2facet(tex, Wf, bary_sh, cum)
    return conv3d.facet2vertex(z, Wo, coeff, face, nf_count, vt_map)


def one_sample_forward(face_rows, filter, weights, weights_padded=None):
    """facet2facet forward for exactly one sample per face: (Nf, Cin) rows, (Cout, Cin, F) filter, (Nf, F) weights;
    weights_padded: topology.pad_rows(weights) when the caller keeps it (saves the copy inside the call)."""
    conv3d._check(face_rows, "input", 2, torch.float32)
    conv3d._check(filter, "filter", 3, torch.float32)
    conv3d._check(weights, "weights", 2, torch.float32)
    Nf, Cin = face_rows.shape
    Cout, _, F = filter.shape
    if filter.shape[1] != Cin:
        raise RuntimeError("input Channel size error of the filter.")
    if F > 50:
        raise RuntimeError("A maximum of 50 filters are supported in face2face convolution.")
    if tuple(weights.shape) != (Nf, F):
        raise RuntimeError("weights must have shape (NfIn, number of filters)")
    face_rows, weights = conv3d._aligned16(face_rows), conv3d._aligned16(weights)
    if weights_padded is not None and tuple(weights_padded.shape) != (Nf, _lib.query("pb200_padded_row_floats", F)):
        raise RuntimeError("weights_padded must have shape (NfIn, padded row length)")
    dev = face_rows.device
    precision = conv3d._f2f_precision
    with torch.cuda.device(dev):
        out = torch.empty(Nf, Cout, dtype=face_rows.dtype, device=dev)
        nb = _lib.query("pb200_facet2facet_one_sample_forward_workspace_bytes", Nf, Cin, Cout, F, precision)
        ws = conv3d._ws(nb, dev)
        _lib.call("pb200_facet2facet_one_sample_forward", Nf, Cin, Cout, F, ptr(face_rows), ptr(filter), ptr(weights),
                  ptr(weights_padded), ptr(out), precision, ptr(ws), nb, stream_ptr(dev))
    return out


class _SharedRowsF2F(torch.autograd.Function):
    """facet2facet over one row per face shared by the face's samples: forward through the one-sample entry,
    backward through the general operator's backward over (rows, per-face mean weights, one sample per face)."""

    @staticmethod
    def forward(ctx, face_rows, filter, weights, one_each, weights_padded):
        face_rows, filter = face_rows.contiguous(), filter.contiguous()
        ctx.save_for_backward(face_rows, filter, weights, one_each)
        ctx.weights_padded = weights_padded
        return one_sample_forward(face_rows, filter, weights, weights_padded)

    @staticmethod
    def backward(ctx, grad_output):
        face_rows, filter, weights, one_each = ctx.saved_tensors
        gin, gf = conv3d.facet2facet_backward(grad_output.contiguous(), face_rows, filter, weights, one_each,
                                              baryPadded=ctx.weights_padded)
        return gin, gf, None, None, None


def facet2facet_shared_rows(face_rows, filter, bary_sh, cum):
    """facet2facet(repeat_interleave(face_rows, samples per face), filter, bary_sh, cum) without the expanded rows.
    bary_sh: the (NiK, F) sample weights, or their per-face means as topology.face_means / face_means_sph_harm
    return them (then cum is not looked at)."""
    fm = bary_sh if isinstance(bary_sh, FaceMeans) else face_means(bary_sh, cum)
    return _SharedRowsF2F.apply(face_rows, filter, fm.rows, fm.one_each, fm.rows_padded)


def conv_block(x, Wv, Wf, Wo, face, cum, bary_sh, coeff, nf_count, vt_map, sh_eye):
    cin = x.shape[1]
    spatial = (sh_eye @ Wv).reshape(3, cin, 1)
    y = conv3d.vertex2facet(x, spatial, face)
    z = facet2facet_shared_rows(y, Wf, bary_sh, cum)
    return conv3d.facet2vertex(z, Wo, coeff, face, nf_count, vt_map)
