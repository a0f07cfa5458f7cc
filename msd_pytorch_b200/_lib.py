"""ctypes binding of ``libmsd_b200.so`` (the C ABI declared in ``include/msd_b200.h``).

There is no CPU or PyTorch fallback: if the shared library is missing, importing
this module raises, and every operation needs CUDA tensors.
"""
import ctypes
import os
import threading

import torch

_PKG = os.path.dirname(os.path.abspath(__file__))
LIB_PATH = os.path.join(_PKG, "lib", "libmsd_b200.so")

MSD_OK = 0
MSD_F32, MSD_F64 = 0, 1
MAX_DIMS = 5

FAMILY_FWD2D, FAMILY_BWD2D, FAMILY_FWD3D, FAMILY_BWD3D = 0, 1, 2, 3
SLAB_GRADIENT_IS_GATED, SLAB_GATE_CHANNEL_BELOW = 1, 2
SLAB_FORWARD_SUMS_ONLY, SLAB_FORWARD_GATHER_ONLY = 1, 2


class MsdTensor(ctypes.Structure):
    _fields_ = [
        ("data", ctypes.c_void_p),
        ("ndim", ctypes.c_int32),
        ("reserved", ctypes.c_int32),
        ("size", ctypes.c_int64 * MAX_DIMS),
        ("stride", ctypes.c_int64 * MAX_DIMS),
    ]


def _load():
    if not os.path.exists(LIB_PATH):
        raise ImportError(
            "msd_pytorch_b200: %s is missing. Build it with `python -m msd_pytorch_b200.build` "
            "(needs nvcc); there is no fallback implementation." % LIB_PATH
        )
    lib = ctypes.CDLL(LIB_PATH)
    T = ctypes.POINTER(MsdTensor)
    vp, i, sz, i64 = ctypes.c_void_p, ctypes.c_int, ctypes.c_size_t, ctypes.c_int64
    sigs = {
        "msd_version": (i, []),
        "msd_last_error_string": (ctypes.c_char_p, []),
        "msd_workspace_bytes": (sz, [i, i, i64, i64, i64]),
        "msd_forward_workspace_bytes": (sz, [i, i, i64]),
        "msd_conv_forward": (i, [i, T, vp, vp, T, i, vp, sz, i, vp]),
        "msd_conv_relu_forward": (i, [i, T, vp, vp, T, i, vp, sz, i, vp]),
        "msd_conv_backward_x": (i, [i, T, vp, T, i, i, vp]),
        "msd_conv_relu_backward_x": (i, [i, T, T, vp, T, i, i, vp]),
        "msd_conv_backward_k": (i, [i, T, T, vp, i, vp, sz, i, vp]),
        "msd_conv_relu_backward_k": (i, [i, T, T, T, vp, i, vp, sz, i, vp]),
        "msd_conv_backward_bias": (i, [i, T, vp, vp, sz, i, vp]),
        "msd_conv_relu_backward_bias": (i, [i, T, T, vp, vp, sz, i, vp]),
        "msd_block_forward": (i, [i, T, i, i, i, ctypes.POINTER(vp), vp, ctypes.POINTER(i), vp, sz, i, vp]),
        "msd_block_backward": (i, [i, T, T, i, i, i, ctypes.POINTER(vp), ctypes.POINTER(i), ctypes.POINTER(vp), vp, vp, sz, i, vp]),
        "msd_block_workspace_bytes": (sz, [i, i, i64, i, i, i]),
        "msd_block_backward_plan": (i, [i, T, T, i, i, i, ctypes.POINTER(i), ctypes.c_char_p, sz, ctypes.POINTER(i)]),
        "msd_final_forward": (i, [i, T, vp, vp, T, i, vp]),
        "msd_final_backward": (i, [i, T, T, vp, T, vp, vp, vp, sz, i, vp]),
        "msd_final_workspace_bytes": (sz, [i64, i64]),
        "msd_slab_layer_forward": (i, [T, i, vp, vp, i, i, i, i, vp, sz, i, vp]),
        "msd_slab_layer_backward": (i, [T, T, i, vp, i, i, i, vp, vp, i, vp, sz, i, vp]),
        "msd_tuning_num_variants": (i, [i]),
        "msd_tuning_set": (i, [i, i, i]),
        "msd_tuning_get": (i, [i, i]),
        "msd_launch_count": (i64, []),
        "msd_fast_launch_count": (i64, []),
        "msd_split_launch_count": (i64, []),
        "msd_mma_launch_count": (i64, []),
        "msd_reset_launch_count": (None, []),
        "msd_device_status": (i, [i, vp, ctypes.POINTER(ctypes.c_int)]),
        "msd_conv_relu_backward_k_noalloc": (i, [i, T, T, T, vp, i, i, vp]),
        "msd_noalloc_scratch_bytes": (sz, []),
        "msd_selftest_wait_timeout": (i, [ctypes.c_uint64, i, vp]),
    }
    for name, (res, args) in sigs.items():
        fn = getattr(lib, name)
        fn.restype = res
        fn.argtypes = args
    return lib


lib = _load()
EXPORTED = [
    "msd_version", "msd_last_error_string", "msd_workspace_bytes", "msd_forward_workspace_bytes",
    "msd_conv_forward", "msd_conv_relu_forward", "msd_conv_backward_x", "msd_conv_relu_backward_x",
    "msd_conv_backward_k", "msd_conv_relu_backward_k", "msd_conv_backward_bias", "msd_conv_relu_backward_bias",
    "msd_block_forward", "msd_block_backward", "msd_block_workspace_bytes", "msd_block_backward_plan",
    "msd_slab_layer_forward", "msd_slab_layer_backward",
    "msd_final_forward", "msd_final_backward", "msd_final_workspace_bytes",
    "msd_tuning_num_variants", "msd_tuning_set", "msd_tuning_get",
    "msd_launch_count", "msd_fast_launch_count", "msd_split_launch_count", "msd_mma_launch_count", "msd_reset_launch_count", "msd_device_status",
    "msd_conv_relu_backward_k_noalloc", "msd_noalloc_scratch_bytes", "msd_selftest_wait_timeout",
]


def dtype_code(dtype):
    if dtype == torch.float32:
        return MSD_F32
    if dtype == torch.float64:
        return MSD_F64
    raise RuntimeError("msd_pytorch_b200: expected a float32 or float64 tensor, got %s" % dtype)


def describe(t):
    """``msd_tensor_t`` for a 4- or 5-dimensional torch tensor (sizes and strides in elements)."""
    d = MsdTensor()
    d.data = t.data_ptr()
    d.ndim = t.dim()
    for k in range(t.dim()):
        d.size[k] = t.shape[k]
        d.stride[k] = t.stride(k)
    return d


def check(status):
    if status != MSD_OK:
        raise RuntimeError(lib.msd_last_error_string().decode("utf-8", "replace") or "msd_b200 error %d" % status)


def stream_of(device):
    return ctypes.c_void_p(torch.cuda.current_stream(device).cuda_stream)


# One scratch buffer per (device, stream): calls on one stream are ordered, so they may share it.
_ws_lock = threading.Lock()
_ws = {}


def workspace(device, nbytes):
    """A 256-byte aligned device scratch buffer of at least ``nbytes`` for the current stream."""
    key = (device.index, torch.cuda.current_stream(device).cuda_stream)
    with _ws_lock:
        buf = _ws.get(key)
        if buf is None or buf.numel() < nbytes:
            buf = torch.empty(max(int(nbytes), 1 << 20), dtype=torch.uint8, device=device)
            _ws[key] = buf
    assert buf.data_ptr() % 256 == 0
    return buf


def device_status(device):
    """Synchronise the current stream of ``device`` and return the device status word
    (0 = every bounded wait inside the kernels completed)."""
    out = ctypes.c_int(0)
    check(lib.msd_device_status(device.index, stream_of(device), ctypes.byref(out)))
    return out.value


def launch_counts():
    return int(lib.msd_launch_count()), int(lib.msd_fast_launch_count())
