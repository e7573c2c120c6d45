"""The point-cloud convolution module with the reference's class name, constructor arguments and
parameter names (picasso/point/layers.py:19-75): depthwise SPH3D convolution (hard or fuzzy bins)
followed by the pointwise stage matmul -> + bias -> activation -> BatchNorm1d(eps=1e-3)."""
from __future__ import annotations

import torch.nn as nn

from ..mesh.layers import _PointwiseTail, _filter_variable_
from .pi_modules import conv3d


class PCloudConv3d(_PointwiseTail):
    def __init__(self, in_channels, out_channels, num_basis, depth_multiplier=1, use_xavier=True, stddev=1e-3,
                 activation_fn=nn.ReLU(), with_bn=True, bn_momentum=0.1):
        super().__init__()
        self.in_channels, self.out_channels = in_channels, out_channels
        self.num_basis = num_basis
        self.multiplier = depth_multiplier
        self.use_xavier, self.stddev = use_xavier, stddev
        self.spatial_weights = _filter_variable_([num_basis, in_channels, depth_multiplier], use_xavier=use_xavier)
        self.depth_weights = _filter_variable_([in_channels * depth_multiplier, out_channels], use_xavier=use_xavier)
        self._init_tail(out_channels, activation_fn, with_bn, bn_momentum)

    def forward(self, inputs, nn_count, nn_index, filt_index, filt_coeff=None):
        if filt_coeff is None:
            feats = conv3d.conv3d(inputs, self.spatial_weights, nn_count, nn_index, filt_index)
        else:
            feats = conv3d.fuzzyconv3d(inputs, self.spatial_weights, nn_count, nn_index, filt_index, filt_coeff)
        return self._tail(feats @ self.depth_weights)


# the pointwise layer is the same module for points, vertices and facets (picasso/point/layers.py:78-119)
from ..mesh.layers import PerItemConv3d  # noqa: E402,F401
