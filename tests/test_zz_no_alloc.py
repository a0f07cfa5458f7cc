"""GPU test of msd_conv_relu_backward_k_noalloc, the weight-gradient entry point for callers
that cannot allocate device memory (plugins living inside another framework's memory pool,
serving loops that must not touch the allocator).  It keeps its scratch in an array built
into the library instead of taking a workspace.

Collected last on purpose (file name): if it fails, a run that stops at the first failure
has already run every other test.  Called through the C ABI, compared with the ordinary
entry point on two calls in a row, and safe to run alone or after the other tests."""
import ctypes

import pytest
import torch

import util
from util import assert_close

pytestmark = pytest.mark.gpu


def _call_both(dev, B, C, sp, d, seed):
    from msd_pytorch_b200 import _lib
    from msd_pytorch_b200 import msd_custom_convolutions as cc

    L = _lib.lib
    x, k, b, go = (t.to(dev) for t in util.make_op_inputs(B, C, 1, sp, torch.float32, seed, dev))
    y = torch.empty_like(go)
    cc.conv_relu_forward(x, k, b, y, d)
    want = torch.zeros_like(k)
    cc.conv_relu_backward_k(y, go, x, want, d)            # existing entry point (caller workspace)
    got = torch.zeros_like(k)
    rc = L.msd_conv_relu_backward_k_noalloc(_lib.MSD_F32, _lib.describe(y), _lib.describe(go), _lib.describe(x), got.data_ptr(), d,
                                            dev.index, _lib.stream_of(dev))
    assert rc == 0, L.msd_last_error_string()
    assert _lib.device_status(dev) == 0
    return got, want


def test_noalloc_matches_workspace_entry_point_twice(cuda_device):
    dev = cuda_device
    # two calls in a row with different shapes: the second sees the first one's leftovers in
    # the shared scratch array and must not be affected by them
    for (B, C, sp, d, seed) in [(2, 24, (96, 256), 5, 1), (1, 7, (10, 24, 64), 3, 2), (2, 24, (96, 256), 5, 1)]:
        got, want = _call_both(dev, B, C, sp, d, seed)
        assert_close(got, want, 1e-3, "noalloc vs workspace entry point")
        assert torch.equal(got, want), "same kernels, same reduction order: results must be identical"


def test_noalloc_accumulates_and_handles_generic_shapes(cuda_device):
    """Shapes the tuned kernel does not take (odd width) go through the generic kernel with the
    same built-in scratch; the gradient is added to what grad_kernel already holds."""
    from msd_pytorch_b200 import _lib
    from msd_pytorch_b200 import msd_custom_convolutions as cc

    dev = cuda_device
    L = _lib.lib
    x, k, b, go = (t.to(dev) for t in util.make_op_inputs(2, 3, 2, (13, 37), torch.float32, 3, dev))
    y = torch.empty_like(go)
    cc.conv_relu_forward(x, k, b, y, 2)
    want = torch.ones_like(k)
    cc.conv_relu_backward_k(y, go, x, want, 2)
    got = torch.ones_like(k)
    rc = L.msd_conv_relu_backward_k_noalloc(_lib.MSD_F32, _lib.describe(y), _lib.describe(go), _lib.describe(x), got.data_ptr(), 2, dev.index,
                                            _lib.stream_of(dev))
    assert rc == 0, L.msd_last_error_string()
    torch.cuda.synchronize()
    assert_close(got, want, 1e-3, "noalloc generic path")


def test_noalloc_rejects_shapes_beyond_the_fixed_scratch(cuda_device):
    from msd_pytorch_b200 import _lib

    dev = cuda_device
    L = _lib.lib
    assert L.msd_noalloc_scratch_bytes() == 4 << 20
    C = 600  # needs more partial-sum space than the built-in 4 MiB
    x = torch.zeros(1, C, 16, 16, device=dev)
    y = torch.zeros(1, 1, 16, 16, device=dev)
    gk = torch.zeros(1, C, 3, 3, device=dev)
    before = _lib.launch_counts()[0]
    rc = L.msd_conv_relu_backward_k_noalloc(_lib.MSD_F32, _lib.describe(y), _lib.describe(y), _lib.describe(x), gk.data_ptr(), 1, dev.index,
                                            _lib.stream_of(dev))
    assert rc == 5  # MSD_ERR_LIMIT
    assert b"built-in array" in L.msd_last_error_string()
    assert _lib.launch_counts()[0] == before, "a refused call must not launch anything"
