"""Runs the REFERENCE's own test files (ahendriksen/msd_pytorch, msd_pytorch/tests/) on this
package's kernels, and a checkpoint round trip between the reference's model classes and ours.

TEST INFRASTRUCTURE.  Needs a CUDA device and a checkout of the reference, named by the
environment variable MSD_REFERENCE_ROOT (the directory that contains ``msd_pytorch/``).
Nothing of the reference is copied or modified: its files are imported where they lie.

    MSD_REFERENCE_ROOT=/path/to/msd_pytorch python tests/reference_suite/run.py backend  [pytest args]
    MSD_REFERENCE_ROOT=...                  python tests/reference_suite/run.py package  [pytest args]
    MSD_REFERENCE_ROOT=...                  python tests/reference_suite/run.py checkpoint <tmpdir>

``backend``  the reference's Python layers (conv2d.py, msd_block.py, msd_module.py, the model
             classes) run unchanged; only its native module ``msd_custom_convolutions`` is
             replaced by this package's op module (``install_as_reference_backend``).
``package``  the same test files, but every ``msd_pytorch.*`` module they import is this
             package's module of the same name: the tests then exercise our Python layers too.
``checkpoint`` a network saved by the reference's ``MSDRegressionModel.save`` is loaded by ours
             and vice versa (msd_model.py:310-342 of the reference), outputs compared.

Three adaptations of the ENVIRONMENT, none of the reference's files, are needed on a current
Python stack: stub modules for ``imageio`` and ``tifffile`` (imported by image_dataset.py,
which is not on the tested path), ``numpy.product`` (removed in NumPy 2; used by
msd_module.py:54) and ``collections.Iterable`` (removed in Python 3.10).
"""
import collections
import collections.abc
import os
import sys
import types

HERE = os.path.dirname(os.path.abspath(__file__))
REPO = os.path.dirname(os.path.dirname(HERE))

TEST_FILES = ["test_conv2d.py", "test_conv3d.py", "test_msd_block.py", "test_msd_module.py", "test_msd_model.py",
              "test_msd_regression_model.py", "test_msd_segmentation_model.py"]


def reference_root():
    root = os.environ.get("MSD_REFERENCE_ROOT")
    if not root or not os.path.isdir(os.path.join(root, "msd_pytorch")):
        raise SystemExit("MSD_REFERENCE_ROOT must name a checkout of ahendriksen/msd_pytorch")
    return os.path.abspath(root)


def environment_shims():
    import numpy as np

    for name in ("imageio", "tifffile"):
        if name not in sys.modules:
            try:
                __import__(name)
            except ImportError:
                sys.modules[name] = types.ModuleType(name)
    if not hasattr(np, "product"):
        np.product = np.prod
    if not hasattr(collections, "Iterable"):
        collections.Iterable = collections.abc.Iterable


def install(mode):
    """Make ``import msd_pytorch`` resolve as `mode` says; returns the directory of the tests."""
    root = reference_root()
    if REPO not in sys.path:
        sys.path.insert(0, REPO)
    environment_shims()
    import msd_pytorch_b200

    msd_pytorch_b200.install_as_reference_backend()
    if mode == "backend":
        sys.path.insert(0, root)
        import msd_pytorch  # noqa: F401  (the reference's package, on our native module)
    elif mode == "package":
        # a package object whose submodules are OURS, while `msd_pytorch.tests` still resolves to
        # the reference's test package through __path__
        pkg = types.ModuleType("msd_pytorch")
        pkg.__path__ = [os.path.join(root, "msd_pytorch")]
        pkg.__version__ = msd_pytorch_b200.__version__
        sys.modules["msd_pytorch"] = pkg
        import importlib

        for sub in ("conv2d", "conv3d", "msd_block", "msd_module", "msd_model", "msd_regression_model", "msd_segmentation_model"):
            mod = importlib.import_module("msd_pytorch_b200." + sub)
            sys.modules["msd_pytorch." + sub] = mod
            setattr(pkg, sub, mod)
        pkg.MSDRegressionModel = msd_pytorch_b200.MSDRegressionModel
        pkg.MSDSegmentationModel = msd_pytorch_b200.MSDSegmentationModel
    else:
        raise SystemExit("mode must be backend or package")
    return os.path.join(root, "msd_pytorch", "tests")


class _Failures:
    """pytest plugin: remembers the node ids that failed."""

    def __init__(self):
        self.failed = []

    def pytest_runtest_logreport(self, report):
        if report.failed and report.nodeid not in self.failed:
            self.failed.append(report.nodeid)


def run_tests(mode, extra):
    """Runs the files; a test that fails is repeated up to two more times on its own and counts
    as failed only if it fails every time.  (The reference's gradcheck tests draw UNSEEDED
    random inputs and compare against finite differences with a step of 1e-6: now and then a
    ReLU pre-activation lies within that step of zero and the numerical Jacobian is off.)"""
    import pytest

    tests = install(mode)
    root = os.path.dirname(os.path.dirname(tests))
    files = [os.path.join(tests, f) for f in TEST_FILES]
    # rootdir = the checkout, so that the files import as msd_pytorch.tests.*; no cache files are
    # written into the (possibly read-only) checkout
    base = ["-q", "-p", "no:cacheprovider", "--rootdir", root, "-W", "ignore"]
    seen = _Failures()
    rc = pytest.main(base + files + list(extra), plugins=[seen])
    if rc == 0 or not seen.failed or "--collect-only" in extra:
        return rc
    still = list(seen.failed)
    for attempt in range(2):
        again = _Failures()
        os.chdir(root)
        rc = pytest.main(base + still, plugins=[again])
        still = again.failed
        if not still:
            print("reference suite: %d test(s) failed once and passed when repeated: %s" % (len(seen.failed), ", ".join(seen.failed)))
            return 0
    print("reference suite: failed three times in a row: %s" % ", ".join(still))
    return 1


def checkpoint_roundtrip(tmpdir):
    """Reference-written checkpoint -> our model, ours -> the reference's; both 2D regression
    and segmentation, outputs compared on a random input."""
    import torch

    install("backend")
    import msd_pytorch as ref
    import msd_pytorch_b200 as ours

    torch.manual_seed(0)
    done = []
    for kind in ("regression", "segmentation"):
        args = (2, 3, 5, 1)
        mk = (lambda m: m.MSDRegressionModel(*args, dilations=[1, 2, 4])) if kind == "regression" else (lambda m: m.MSDSegmentationModel(*args, dilations=[1, 2, 4]))
        x = torch.randn(2, 2, 24, 32)
        for src_name, src, dst in (("reference", ref, ours), ("ours", ours, ref)):
            a, b = mk(src), mk(dst)
            for p in a.net.parameters():      # non-trivial parameters, scaling layers included
                p.data.normal_(0, 0.3)
            y = torch.randn(2, 3, 24, 32) if kind == "regression" else torch.randint(0, 3, (2, 1, 24, 32))
            a.learn(x, y)                     # gives the optimiser a state to save
            path = os.path.join(tmpdir, "%s_%s.torch" % (kind, src_name))
            a.save(path, 17)
            assert b.load(path) == 17
            ka, kb = list(a.net.state_dict().keys()), list(b.net.state_dict().keys())
            assert ka == kb, (ka, kb)
            for k, v in a.net.state_dict().items():
                assert torch.equal(v.cpu(), b.net.state_dict()[k].cpu()), k
            with torch.no_grad():
                oa, ob = a.net(x.cuda()), b.net(x.cuda())
            torch.testing.assert_close(oa, ob, rtol=1e-4, atol=1e-5)
            done.append("%s: %s -> %s" % (kind, src_name, "ours" if dst is ours else "reference"))
    print("checkpoint round trips ok:", "; ".join(done))
    return 0


if __name__ == "__main__":
    what = sys.argv[1] if len(sys.argv) > 1 else "backend"
    if what == "checkpoint":
        sys.exit(checkpoint_roundtrip(sys.argv[2]))
    sys.exit(run_tests(what, sys.argv[2:]))
