from . import conv3d  # noqa: F401

__all__ = ['conv3d']
