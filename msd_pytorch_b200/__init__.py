"""msd_pytorch_b200: the Mixed-Scale Dense network hot path of ahendriksen/msd_pytorch,
rebuilt for NVIDIA B200 (sm_100a) behind the reference's Python API.

Importing the package loads ``lib/libmsd_b200.so``; it raises if the library has
not been built (``python -m msd_pytorch_b200.build``).  There is no CPU path.
"""
from . import _lib  # noqa: F401  (fails loudly when the CUDA library is missing)
from . import msd_custom_convolutions  # noqa: F401
from . import conv2d, conv3d  # noqa: F401
from .msd_block import MSDBlock, MSDBlock2d, MSDBlock3d, MSDBlockFunction, msd_block  # noqa: F401
from .msd_module import MSDFinalLayer, MSDModule  # noqa: F401
from .msd_regression_model import MSDRegressionModel  # noqa: F401
from .msd_segmentation_model import MSDSegmentationModel  # noqa: F401

__version__ = "0.1.0"


def install_as_reference_backend():
    """Register this package's op module under the reference's native module name,
    so that unmodified ``msd_pytorch`` Python code (``import msd_custom_convolutions as cc``)
    runs on the B200 kernels."""
    import sys

    sys.modules["msd_custom_convolutions"] = msd_custom_convolutions
    return msd_custom_convolutions
