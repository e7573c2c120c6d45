from . import conv3d, decimate, fused, pool3d, unpool3d  # noqa: F401

__all__ = ['conv3d', 'decimate', 'pool3d', 'unpool3d']
