"""Spherical-harmonic basis on the GPU (replaces the elementwise torch composition of the
reference's picasso/math_utils.py:10-62 with one kernel)."""
from __future__ import annotations

import torch

from . import _lib
from .topology import ptr, stream_ptr


def sph_harm_coeff(L: int, cart_coords: torch.Tensor) -> torch.Tensor:
    """(N, (L+1)^2) basis values of the (N,3) points after projection to the unit sphere;
    same projection, angle conventions and column order as the reference
    (picasso/mesh/layers.py:341-356 + picasso/math_utils.py:10-62).  L >= 6 raises
    NotImplementedError like the reference."""
    if L >= 6 or L < 0:
        raise NotImplementedError
    if not cart_coords.is_cuda:
        raise RuntimeError("cart_coords must be a CUDA tensor")
    if cart_coords.dim() != 2 or cart_coords.shape[1] != 3:
        raise RuntimeError("cart_coords must have shape (N, 3)")
    xyz = cart_coords.detach().to(torch.float32).contiguous()
    dev = xyz.device
    with torch.cuda.device(dev):
        out = torch.empty(xyz.shape[0], (L + 1) ** 2, dtype=torch.float32, device=dev)
        _lib.call("pb200_sph_harm_coeff", xyz.shape[0], L, ptr(xyz), ptr(out), stream_ptr(dev))
    return out
