"""CPU tests of the C-ABI boundary: the library loads, exports every symbol that
include/msd_b200.h declares, and rejects bad arguments before touching a GPU."""
import ctypes
import os
import re

import pytest
import torch

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def declared_symbols():
    text = open(os.path.join(ROOT, "include", "msd_b200.h")).read()
    return sorted(set(re.findall(r"MSD_API[^;(]*?\b(msd_[a-z0-9_]+)\s*\(", text)))


def test_library_exports_every_declared_symbol():
    from msd_pytorch_b200 import _lib

    names = declared_symbols()
    assert len(names) >= 20
    raw = ctypes.CDLL(_lib.LIB_PATH)
    for n in names:
        assert hasattr(raw, n), "libmsd_b200.so does not export " + n
    assert set(names) == set(_lib.EXPORTED), "binding and header disagree"
    assert _lib.lib.msd_version() >= 100


def test_package_has_no_fallback(monkeypatch):
    """Without the shared library the package refuses to import."""
    from msd_pytorch_b200 import _lib

    monkeypatch.setattr(_lib, "LIB_PATH", os.path.join(ROOT, "does_not_exist.so"))
    with pytest.raises(ImportError):
        _lib._load()


def test_cpu_tensors_are_rejected():
    # msd_custom_convolutions.cpp:98: every op rejects CPU tensors.
    from msd_pytorch_b200 import msd_custom_convolutions as cc

    x = torch.zeros(1, 1, 4, 4)
    with pytest.raises(RuntimeError):
        cc.conv_forward(x, torch.zeros(1, 1, 3, 3), torch.zeros(1), torch.zeros(1, 1, 4, 4), 1, block_size=(0, 16, 16))


def _desc(shape, strides=None, ptr=256):
    from msd_pytorch_b200 import _lib

    d = _lib.MsdTensor()
    d.data = ptr
    d.ndim = len(shape)
    st = 1
    dense = []
    for s in reversed(shape):
        dense.insert(0, st)
        st *= s
    for k, s in enumerate(shape):
        d.size[k] = s
        d.stride[k] = (strides or dense)[k]
    return d


def test_c_abi_argument_errors_need_no_gpu():
    from msd_pytorch_b200 import _lib

    L = _lib.lib
    a, b = _desc((1, 2, 4, 4)), _desc((1, 1, 4, 4))
    # dilation 0 and dilation > size  (msd_custom_convolutions.cpp:39-52)
    assert L.msd_conv_forward(0, a, 256, 256, b, 0, None, 0, 0, None) == 1
    assert b"Dilation must be 1 or greater" in L.msd_last_error_string()
    assert L.msd_conv_forward(0, a, 256, 256, b, 5, None, 0, 0, None) == 1
    assert b"Dilation cannot be greater" in L.msd_last_error_string()
    # shape mismatch (msd_custom_convolutions.cpp:69-83)
    assert L.msd_conv_relu_forward(0, a, 256, 256, _desc((1, 1, 4, 5)), 1, None, 0, 0, None) == 1
    assert L.msd_conv_relu_forward(0, a, 256, 256, _desc((2, 1, 4, 4)), 1, None, 0, 0, None) == 1
    # rank mismatch, bad dtype, null pointers
    assert L.msd_conv_forward(0, a, 256, 256, _desc((1, 1, 1, 4, 4)), 1, None, 0, 0, None) == 1
    assert L.msd_conv_forward(7, a, 256, 256, b, 1, None, 0, 0, None) == 2
    assert L.msd_conv_forward(0, a, None, 256, b, 1, None, 0, 0, None) == 1
    assert L.msd_forward_workspace_bytes(0, 5, 1000) >= 12000 and L.msd_forward_workspace_bytes(0, 4, 1000) == 0
    # misaligned workspace
    assert L.msd_conv_backward_k(0, b, a, 256, 1, 13, 1 << 20, 0, None) == 3
    # block: channel count must be c_in + depth*width
    ptrs = (ctypes.c_void_p * 2)(256, 256)
    dil = (ctypes.c_int * 2)(1, 1)
    assert L.msd_block_forward(0, _desc((1, 4, 4, 4)), 1, 2, 1, ptrs, 256, dil, None, 0, 0, None) == 1
    assert L.msd_workspace_bytes(0, 4, 1 << 20, 100, 1) > 0


def test_noalloc_limit_boundaries_need_no_gpu():
    """The built-in scratch of msd_conv_relu_backward_k_noalloc holds the partial sums of up to
    356 input channels in 2D and 118 in 3D (one output channel); one more is refused with
    MSD_ERR_LIMIT before anything touches a GPU."""
    from msd_pytorch_b200 import _lib

    L = _lib.lib
    for shape, c_ok in (((1, 1, 16, 16), 356), ((1, 1, 8, 16, 16), 118)):
        nd = len(shape)
        assert L.msd_workspace_bytes(0, nd, 1 << 20, c_ok, 1) <= L.msd_noalloc_scratch_bytes() < L.msd_workspace_bytes(0, nd, 1 << 20, c_ok + 1, 1)
        y = _desc(shape)
        x = _desc((1, c_ok + 1) + shape[2:])
        assert L.msd_conv_relu_backward_k_noalloc(0, y, y, x, 256, 1, 0, None) == 5
        assert b"built-in array" in L.msd_last_error_string()
        x = _desc((1, c_ok) + shape[2:])
        assert L.msd_conv_relu_backward_k_noalloc(0, y, y, x, 256, 1, 0, None) != 5  # accepted as far as the limit goes (no GPU here)


def _plan(shape, c_in, dilations, dtype=0, wants=None, ws_bytes=64 << 20):
    from msd_pytorch_b200 import _lib

    L = _lib.lib
    depth = len(dilations)
    full = (shape[0], c_in + depth) + tuple(shape[1:])
    res, grad = _desc(full, ptr=1 << 20), _desc(full, ptr=1 << 30)
    dil = (ctypes.c_int * depth)(*dilations)
    codes = (ctypes.c_int * depth)()
    w = None if wants is None else bytes(wants)
    rc = L.msd_block_backward_plan(dtype, res, grad, c_in, depth, 1, dil, w, ws_bytes, codes)
    assert rc == 0, L.msd_last_error_string()
    return list(codes)


def test_block_backward_plan_mixes_tuned_and_generic_layers():
    """The layer-by-layer decisions of msd_block_backward, made on the host alone: a layer hands
    its gradient over gated only when the layer below runs a tuned kernel too, so a gated
    gradient never meets a kernel that would gate it again (dilations beyond the tuned range sit
    above, below and between tuned layers)."""
    TUNED, TOP, READS, BELOW = 1, 2, 4, 8
    # power-of-two dilations up to 32 on a 64 x 96 image: the top layer (d = 32) is generic
    assert _plan((2, 64, 96), 1, [1, 2, 4, 8, 16, 32]) == [TUNED | READS, TUNED | READS | BELOW, TUNED | READS | BELOW, TUNED | READS | BELOW, TUNED | BELOW, 0]
    # an untuned layer BELOW a tuned one: the tuned one must not gate for it
    assert _plan((2, 48, 64), 1, [20, 1]) == [0, TUNED | TOP]
    # ... and between two tuned ones
    assert _plan((2, 48, 64), 1, [1, 20, 2]) == [TUNED, 0, TUNED | TOP]
    # the same in 3D
    assert _plan((1, 24, 24, 32), 1, [2, 20, 1, 3]) == [TUNED, 0, TUNED | READS, TUNED | TOP | BELOW]
    # everything tuned: the top channel is gated in place, every other one by the layer above
    assert _plan((1, 32, 64), 1, [1, 2, 3, 4]) == [TUNED | READS, TUNED | READS | BELOW, TUNED | READS | BELOW, TUNED | TOP | BELOW]
    # float64 takes the generic kernels throughout
    assert _plan((1, 32, 64), 1, [1, 2, 3], dtype=1) == [0, 0, 0]
    # a layer whose weight gradient is not wanted runs the input-gradient-only kernel, which cannot gate
    assert _plan((1, 32, 64), 1, [1, 2, 3, 4], wants=[1, 1, 0, 1]) == [TUNED | READS, TUNED | BELOW, TUNED | READS, TUNED | TOP | BELOW]
    # every state is consistent: READS on layer i  <=>  BELOW on layer i + 1 (or TOP on the top layer never implies READS)
    for dil in ([1, 2, 4, 8, 16, 32], [20, 1], [1, 20, 2], [3, 17, 5, 18, 7], [1] * 12):
        codes = _plan((2, 64, 96), 1, dil)
        for i in range(len(dil) - 1):
            assert bool(codes[i] & READS) == bool(codes[i + 1] & BELOW), (dil, codes)
            if codes[i] & READS:
                assert codes[i] & TUNED, "a gated gradient must only reach a tuned layer"
