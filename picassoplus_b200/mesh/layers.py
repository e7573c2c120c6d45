"""Layer modules of the mesh convolutions (and of mesh pooling / unpooling) with the reference's
class names, constructor arguments, parameter names and parameter shapes
(picasso/mesh/layers.py:10-356),
so reference checkpoints load unchanged.  Each module = one operator from
pi_modules.conv3d followed by the pointwise stage: matmul -> + bias -> activation ->
BatchNorm1d(eps=1e-3)  (batch norm AFTER the activation, as in the reference)."""
from __future__ import annotations

from typing import List

import torch
import torch.nn as nn

from .pi_modules import conv3d, fused, pool3d, unpool3d
from ..math_utils import sph_harm_coeff


_fusion = True


def set_fusion(on: bool) -> None:
    """V2FConv3d / F2VConv3d run operator + depth_weights product + bias + ReLU as ONE kernel where the
    shapes allow it (depth multiplier 1, channels a multiple of 8, ReLU or no activation); off = the
    reference's sequence of separate kernels.  Batch norm stays a torch module either way."""
    global _fusion
    _fusion = bool(on)


def _filter_variable_(shape, stddev=1.0, use_xavier=True):
    w = nn.Parameter(torch.empty(shape))
    return nn.init.xavier_normal_(w) if use_xavier else nn.init.trunc_normal_(w, mean=0, std=stddev)


class SphHarmCoeff(nn.Module):
    """Spherical-harmonic coefficients of cartesian directions, degree <= l."""

    def __init__(self, l):
        super().__init__()
        self.l = l

    def __call__(self, cart_coords):
        return sph_harm_coeff(self.l, cart_coords)


class _PointwiseTail(nn.Module):
    """bias / activation / batch-norm stage shared by the three convolutions."""

    def _init_tail(self, out_channels, activation_fn, with_bn, bn_momentum):
        self.with_bn = with_bn
        self.activation_fn = activation_fn
        if with_bn:
            self.BatchNorm = nn.BatchNorm1d(out_channels, eps=0.001, momentum=bn_momentum)
        self.biases = nn.Parameter(torch.zeros(1, out_channels))

    def _tail(self, x):
        x = x + self.biases
        if self.activation_fn is not None:
            x = self.activation_fn(x)
        if self.with_bn:
            x = self.BatchNorm(x)
        return x

    def _fusable(self, x, channels, multiplier):
        return _fusion and fused.eligible(x, channels, multiplier, self.activation_fn)

    def _after_fused(self, x):
        return self.BatchNorm(x) if self.with_bn else x


class F2FConv3d(_PointwiseTail):
    """Facet-texture convolution; `weights` has shape (out_channels, in_channels, (L+1)^2)."""

    def __init__(self, in_channels, out_channels, spharm_L, use_xavier=True, stddev=1e-3,
                 activation_fn=nn.ReLU(), with_bn=True, bn_momentum=0.1):
        super().__init__()
        self.in_channels, self.out_channels = in_channels, out_channels
        self.L = spharm_L
        self.num_basis = (spharm_L + 1) ** 2
        self.use_xavier, self.stddev = use_xavier, stddev
        self.weights = _filter_variable_([out_channels, in_channels, self.num_basis], stddev, use_xavier)
        self._init_tail(out_channels, activation_fn, with_bn, bn_momentum)

    def forward(self, input_texture, bary_coeff, num_texture):
        assert self.in_channels == input_texture.shape[-1]
        assert self.num_basis == bary_coeff.shape[-1]
        running = torch.cumsum(num_texture, dim=0, dtype=torch.int)   # the operator wants the running count
        return self._tail(conv3d.facet2facet(input_texture, self.weights, bary_coeff, running))


class V2FConv3d(_PointwiseTail):
    """Vertex -> facet; the (3, Cin, mult) spatial filter is SH(eye(3)) @ spatial_weights."""

    def __init__(self, in_channels, out_channels, spharm_L, depth_multiplier=1, use_xavier=True, stddev=1e-3,
                 activation_fn=nn.ReLU(), with_bn=True, bn_momentum=0.1):
        super().__init__()
        self.in_channels, self.out_channels = in_channels, out_channels
        self.L = spharm_L
        self.num_basis = (spharm_L + 1) ** 2
        self.multiplier = depth_multiplier
        self.use_xavier, self.stddev = use_xavier, stddev
        self.spatial_weights = _filter_variable_([self.num_basis, in_channels * depth_multiplier], stddev, use_xavier)
        self.depth_weights = _filter_variable_([in_channels * depth_multiplier, out_channels], stddev, use_xavier)
        self._init_tail(out_channels, activation_fn, with_bn, bn_momentum)

    def forward(self, inputs, face):
        corners = sph_harm_coeff(self.L, torch.eye(3, device=inputs.device))
        spatial = (corners @ self.spatial_weights).reshape(3, self.in_channels, self.multiplier)
        if self._fusable(inputs, self.in_channels, self.multiplier):
            return self._after_fused(fused.vertex2facet_pointwise(inputs, spatial, face, self.depth_weights, self.biases,
                                                                  self.activation_fn is not None))
        feats = conv3d.vertex2facet(inputs, spatial, face)
        return self._tail(feats @ self.depth_weights)


class F2VConv3d(_PointwiseTail):
    """Facet -> vertex; `spatial_weights` has shape ((L+1)^2, Cin, mult)."""

    def __init__(self, in_channels, out_channels, spharm_L, depth_multiplier=1, use_xavier=True, stddev=1e-3,
                 activation_fn=nn.ReLU(), with_bn=True, bn_momentum=0.1):
        super().__init__()
        self.in_channels, self.out_channels = in_channels, out_channels
        self.L = spharm_L
        self.num_basis = (spharm_L + 1) ** 2
        self.multiplier = depth_multiplier
        self.use_xavier, self.stddev = use_xavier, stddev
        self.spatial_weights = _filter_variable_([self.num_basis, in_channels, depth_multiplier], stddev, use_xavier)
        self.depth_weights = _filter_variable_([in_channels * depth_multiplier, out_channels], stddev, use_xavier)
        self._init_tail(out_channels, activation_fn, with_bn, bn_momentum)

    def forward(self, inputs, face, nf_count, vt_map, filt_coeff):
        if self._fusable(inputs, self.in_channels, self.multiplier):
            return self._after_fused(fused.facet2vertex_pointwise(inputs, self.spatial_weights, filt_coeff, face, nf_count,
                                                                  vt_map, self.depth_weights, self.biases,
                                                                  self.activation_fn is not None))
        feats = conv3d.facet2vertex(inputs, self.spatial_weights, filt_coeff, face, nf_count, vt_map)
        return self._tail(feats @ self.depth_weights)


class V2VConv3d(nn.Module):
    """V2F then F2V; `dual_out_channels` and `dual_depth_multiplier` hold one value per stage."""

    def __init__(self, in_channels, dual_out_channels, spharm_L, dual_depth_multiplier: List[int],
                 use_xavier=True, stddev=1e-3, activation_fn=nn.ReLU(), with_bn=True, bn_momentum=0.1):
        super().__init__()
        self.V2F_conv3d = V2FConv3d(in_channels, dual_out_channels[0], spharm_L, dual_depth_multiplier[0],
                                    use_xavier, stddev, activation_fn, with_bn, bn_momentum)
        self.F2V_conv3d = F2VConv3d(dual_out_channels[0], dual_out_channels[1], spharm_L, dual_depth_multiplier[1],
                                    use_xavier, stddev, activation_fn, with_bn, bn_momentum)

    def forward(self, inputs, face, nf_count, vt_map, filt_coeff):
        return self.F2V_conv3d(self.V2F_conv3d(inputs, face), face, nf_count, vt_map, filt_coeff)


class Pool3d(nn.Module):
    """Mesh pooling over decimation clusters, 'max' (default) or 'avg' (reference:
    picasso/mesh/layers.py:263-284)."""

    def __init__(self, method='max'):
        super().__init__()
        self.method = method

    def forward(self, inputs, vt_replace, vt_map, vt_out):
        if self.method == 'max':
            return pool3d.maxPool(inputs, vt_replace, vt_map, vt_out)
        if self.method == 'avg':
            return pool3d.avgPool(inputs, vt_replace, vt_map, vt_out)
        raise ValueError("Unknow pooling method %s." % self.method)


class Unpool3d(nn.Module):
    """Mesh unpooling: every fine vertex takes the feature of its cluster's coarse vertex
    (reference: picasso/mesh/layers.py:287-298)."""

    @staticmethod
    def forward(inputs, vt_replace, vt_map):
        return unpool3d.interpolate(inputs, vt_replace, vt_map)


class PerItemConv3d(nn.Module):
    """Pointwise layer (per vertex, per facet, per point): matmul -> + biases -> activation -> batch norm, the
    reference's module of the same name (picasso/mesh/layers.py:198-240), parameters `weights`
    (in_channels, out_channels), `biases` (1, out_channels), `BatchNorm`.  With fusion on, an input width that is
    a multiple of 8 and ReLU or no activation, product + bias + activation are one tensor-core kernel, and so are
    the two products of the backward pass."""

    def __init__(self, in_channels, out_channels, use_xavier=True, stddev=1e-3, activation_fn=nn.ReLU(), with_bn=True,
                 bn_momentum=0.1):
        super().__init__()
        self.in_channels, self.out_channels = in_channels, out_channels
        self.use_xavier, self.stddev = use_xavier, stddev
        self.with_bn, self.activation_fn = with_bn, activation_fn
        if with_bn:
            self.BatchNorm = nn.BatchNorm1d(out_channels, eps=0.001, momentum=bn_momentum)
        self.weights = _filter_variable_([in_channels, out_channels], stddev=stddev, use_xavier=use_xavier)
        self.biases = nn.Parameter(torch.zeros(1, out_channels))

    def forward(self, inputs):
        if _fusion and inputs.dim() == 2 and fused.eligible(inputs, self.in_channels, 1, self.activation_fn):
            outputs = fused.rows_pointwise(inputs.contiguous(), self.weights, self.biases, self.activation_fn is not None)
        else:
            outputs = torch.matmul(inputs, self.weights) + self.biases
            if self.activation_fn is not None:
                outputs = self.activation_fn(outputs)
        return self.BatchNorm(outputs) if self.with_bn else outputs


class GlobalPool3d(nn.Module):
    """Pools all vertices of every sample of a batch into one row ('avg' or 'max'); nv_in (B,) = vertices per
    sample.  The reference (picasso/mesh/layers.py:242-260) goes through torch_scatter, whose scatter_max returns
    the pair (values, positions): 'max' returns that pair here as well."""

    def __init__(self, method='avg'):
        super().__init__()
        self.method = method

    def forward(self, inputs, nv_in):
        lengths = nv_in.to(torch.int64)
        if self.method == 'avg':
            return torch.segment_reduce(inputs, 'mean', lengths=lengths)
        if self.method == 'max':
            values = torch.segment_reduce(inputs, 'max', lengths=lengths)
            # position of the first vertex that attains the maximum, as an index into `inputs`
            B = lengths.shape[0]
            sample = torch.repeat_interleave(torch.arange(B, device=inputs.device), lengths)
            rows = torch.arange(inputs.shape[0], device=inputs.device).unsqueeze(1).expand_as(inputs)
            cand = torch.where(inputs == values[sample], rows, torch.full_like(rows, inputs.shape[0]))
            first = torch.full((B, inputs.shape[1]), inputs.shape[0], dtype=rows.dtype, device=inputs.device)
            first = first.scatter_reduce(0, sample.unsqueeze(1).expand_as(cand), cand, 'amin')
            return values, first
        raise ValueError("Unknow pooling method %s." % self.method)


class BuildF2VCoeff(nn.Module):
    """Fuzzy facet2vertex coefficients from face normals: softmax over `kernel_size` learned unit directions of the
    cosine between normal and direction, sharpened by 1/tau (picasso/mesh/layers.py:299-328); parameter
    `centers` (kernel_size, dim)."""

    def __init__(self, kernel_size, tau=0.1, dim=3, stddev=1.0):
        super().__init__()
        self.kernel_size, self.tau, self.dim, self.stddev = kernel_size, tau, dim, stddev
        self.centers = _filter_variable_([kernel_size, dim], stddev=stddev, use_xavier=False)

    def forward(self, face_normals):
        directions = self.centers / torch.sqrt(torch.sum(self.centers ** 2, dim=-1, keepdim=True))
        zeta = torch.matmul(face_normals, directions.to(face_normals.device).t()) / self.tau
        coeff = torch.exp(zeta)
        return coeff / torch.sum(coeff, dim=-1, keepdim=True)
