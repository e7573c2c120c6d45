from . import conv3d, decimate  # noqa: F401
