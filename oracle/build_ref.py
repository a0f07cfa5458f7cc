"""Build the reference's own CUDA extension, unmodified, for use as a GPU-side checker.

TEST INFRASTRUCTURE ONLY.  Nothing in the product package imports this file or its output.

The reference (ahendriksen/msd_pytorch) has no CPU implementation of the MSD
convolutions: every entry point rejects CPU tensors
(msd_pytorch/msd_custom_convolutions.cpp:98).  Its ten native sources
(setup.py:148-161) do compile unchanged against the torch in this image, so this
script compiles them *where they lie* in the read-only reference checkout into
``oracle/_ref/`` (git-ignored) under the module name ``msd_custom_convolutions_ref``.
The stock ``setup.py`` is not used (it needs ``pytest-runner`` from an index).

The built module can only run on a machine with a GPU.  It is used
  * by ``tests/golden/make_golden_ref_cuda.py`` to produce golden vectors from the
    reference's kernels, and
  * by ``bench.py`` to report the reference's kernels' speed beside ours.

Usage:  python oracle/build_ref.py [/path/to/reference/checkout]
"""
import os
import sys

HERE = os.path.dirname(os.path.abspath(__file__))
OUT = os.path.join(HERE, "_ref")
NAME = "msd_custom_convolutions_ref"


def default_ref_root():
    """The reference checkout: ``$MSD_REFERENCE_ROOT``, else a directory ``reference`` beside
    this repository."""
    return os.environ.get("MSD_REFERENCE_ROOT") or os.path.join(os.path.dirname(os.path.dirname(HERE)), "reference")

SOURCES = [
    "msd_pytorch/msd_custom_convolutions.cpp",
    "msd_pytorch/msd_custom_convolutions/torch_cuda_dispatch.cu",
    "msd_pytorch/msd_custom_convolutions/conv2d_backward_k.cu",
    "msd_pytorch/msd_custom_convolutions/conv2d_backward_bias.cu",
    "msd_pytorch/msd_custom_convolutions/conv2d_backward_x.cu",
    "msd_pytorch/msd_custom_convolutions/conv2d_forward.cu",
    "msd_pytorch/msd_custom_convolutions/conv3d_backward_bias.cu",
    "msd_pytorch/msd_custom_convolutions/conv3d_backward_k.cu",
    "msd_pytorch/msd_custom_convolutions/conv3d_backward_x.cu",
    "msd_pytorch/msd_custom_convolutions/conv3d_forward.cu",
]


def built_path():
    """Path of the built shared object, or None."""
    p = os.path.join(OUT, NAME + ".so")
    return p if os.path.exists(p) else None


def build(ref_root=None, verbose=False):
    ref_root = ref_root or default_ref_root()
    if not os.path.isdir(ref_root):
        return built_path()
    os.makedirs(OUT, exist_ok=True)
    os.environ.setdefault("TORCH_CUDA_ARCH_LIST", "10.0")
    os.environ.setdefault("MAX_JOBS", str(os.cpu_count() or 4))
    from torch.utils import cpp_extension

    cpp_extension.load(
        name=NAME,
        sources=[os.path.join(ref_root, s) for s in SOURCES],
        extra_include_paths=[os.path.join(ref_root, "msd_pytorch")],
        build_directory=OUT,
        with_cuda=True,
        is_python_module=False,
        verbose=verbose,
    )
    return built_path()


def load():
    """Import the built module (needs a CUDA device to do anything useful)."""
    p = built_path()
    if p is None:
        raise FileNotFoundError("oracle/_ref is not built; run oracle/build_ref.py where the reference checkout exists")
    import importlib.util
    import torch  # noqa: F401  (registers the libraries the module links against)

    spec = importlib.util.spec_from_file_location(NAME, p)
    mod = importlib.util.module_from_spec(spec)
    spec.loader.exec_module(mod)
    return mod


if __name__ == "__main__":
    root = sys.argv[1] if len(sys.argv) > 1 else None
    print(build(root, verbose=True))
