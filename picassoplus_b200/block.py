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
from .topology import face_means, ptr, stream_ptr


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


def facet2facet_shared_rows(face_rows, filter, bary_sh, cum):
    """facet2facet(repeat_interleave(face_rows, samples per face), filter, bary_sh, cum) without the expanded rows."""
    fm = face_means(bary_sh, cum)
    return conv3d.facet2facet(face_rows, filter, fm.rows, fm.one_each)


def conv_block(x, Wv, Wf, Wo, face, cum, bary_sh, coeff, nf_count, vt_map, sh_eye):
    cin = x.shape[1]
    spatial = (sh_eye @ Wv).reshape(3, cin, 1)
    y = conv3d.vertex2facet(x, spatial, face)
    z = facet2facet_shared_rows(y, Wf, bary_sh, cum)
    return conv3d.facet2vertex(z, Wo, coeff, face, nf_count, vt_map)
