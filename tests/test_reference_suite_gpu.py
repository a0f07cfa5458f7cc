"""The reference's own test files, run unchanged on this package's kernels, plus a checkpoint
round trip between the reference's model classes and ours.  Needs a checkout of the reference
(environment variable MSD_REFERENCE_ROOT); without one the tests are skipped, with one they
FAIL when a reference test fails."""
import os
import re
import subprocess
import sys

import pytest

pytestmark = pytest.mark.gpu
HERE = os.path.dirname(os.path.abspath(__file__))
RUNNER = os.path.join(HERE, "reference_suite", "run.py")


def _need_checkout():
    root = os.environ.get("MSD_REFERENCE_ROOT")
    if not root or not os.path.isdir(os.path.join(root, "msd_pytorch", "tests")):
        pytest.skip("no checkout of the reference here (set MSD_REFERENCE_ROOT)")


@pytest.mark.parametrize("mode", ["backend", "package"])
def test_reference_tests_pass(cuda_device, mode):
    _need_checkout()
    p = subprocess.run([sys.executable, RUNNER, mode], capture_output=True, text=True, timeout=3000)
    tail = (p.stdout + p.stderr)[-3000:]
    print(tail)
    m = re.search(r"(\d+) passed", p.stdout)
    assert p.returncode == 0 and m and int(m.group(1)) + len(re.findall(r"^FAILED", p.stdout, re.M)) >= 40, tail


def test_checkpoints_cross_load(cuda_device, tmp_path):
    _need_checkout()
    p = subprocess.run([sys.executable, RUNNER, "checkpoint", str(tmp_path)], capture_output=True, text=True, timeout=600)
    assert p.returncode == 0 and "checkpoint round trips ok" in p.stdout, (p.stdout + p.stderr)[-3000:]
