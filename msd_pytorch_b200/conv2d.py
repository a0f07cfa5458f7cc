"""2D convolution ops and modules (API of the reference's msd_pytorch/conv2d.py)."""
from ._convnd import make_namespace

_ns = make_namespace(2)
globals().update(_ns)
__all__ = sorted(_ns)
