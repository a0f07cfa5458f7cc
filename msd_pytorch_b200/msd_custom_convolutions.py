"""Drop-in for the reference's native module ``msd_custom_convolutions``.

Same eight functions, same positional arguments, same in-place / accumulate
semantics and the same failure behaviour (``RuntimeError``) as
msd_pytorch/msd_custom_convolutions.cpp:85-369 of ahendriksen/msd_pytorch; the
work is done by ``libmsd_b200.so`` through its C ABI.

``block_size`` is accepted for compatibility and ignored: tile shapes are chosen
by the library's per-shape launch table (see ``msd_pytorch_b200.autotune``).
2D versus 3D is chosen by tensor rank (4 or 5), as in the reference.
"""
import torch

from . import _lib

_lib_ = _lib.lib


def _same_gpu(c, *tensors):
    # checkAllSameGPU (msd_custom_convolutions.cpp:98)
    dev = None
    for t in tensors:
        if not isinstance(t, torch.Tensor):
            raise TypeError("%s: expected torch tensors" % c)
        if not t.is_cuda:
            raise RuntimeError("%s: expected all tensors to be CUDA tensors (the MSD convolutions have no CPU implementation)" % c)
        if dev is None:
            dev = t.device
        elif t.device != dev:
            raise RuntimeError("%s: expected all tensors on the same GPU, got %s and %s" % (c, dev, t.device))
    return dev


def _same_type(c, *tensors):
    # checkAllSameType (msd_custom_convolutions.cpp:99)
    dt = tensors[0].dtype
    for t in tensors[1:]:
        if t.dtype != dt:
            raise RuntimeError("%s: expected all tensors to have the same scalar type, got %s and %s" % (c, dt, t.dtype))
    return _lib.dtype_code(dt)


def _kernel_checks(c, kernel, ndim):
    # checkContiguous + checkKernel3x3 + checkDim (msd_custom_convolutions.cpp:25-37,100-109)
    if not kernel.is_contiguous():
        raise RuntimeError("%s: expected kernel to be contiguous" % c)
    if kernel.dim() not in (4, 5):
        raise RuntimeError("%s: Expected 4 or 5 dimensional kernel." % c)
    if any(s != 3 for s in kernel.shape[2:]):
        raise RuntimeError("%s: Kernel shape must be %s" % (c, "3x3" if kernel.dim() == 4 else "3x3x3"))
    if kernel.dim() != ndim:
        raise RuntimeError("%s: expected %d-dimensional tensors to go with a %d-dimensional kernel" % (c, kernel.dim(), kernel.dim()))


def _in_out_shape(c, a, b):
    # checkInOutShape (msd_custom_convolutions.cpp:69-83)
    if a.dim() != b.dim():
        raise RuntimeError("%s: expected tensors with the same number of dimensions, got %d and %d" % (c, a.dim(), b.dim()))
    if a.dim() not in (4, 5):
        raise RuntimeError("%s: expected 4- or 5-dimensional tensors, got %d dimensions" % (c, a.dim()))
    if a.shape[0] != b.shape[0]:
        raise RuntimeError("%s: Input batch dimension does not match output batch dimension. " % c)
    if tuple(a.shape[2:]) != tuple(b.shape[2:]):
        raise RuntimeError("%s: Input shape does not match output shape. " % c)


def _dilation(c, t, dilation):
    # checkDilation (msd_custom_convolutions.cpp:39-52)
    dilation = int(dilation)
    if dilation <= 0:
        raise RuntimeError("%s: Dilation must be 1 or greater" % c)
    if any(dilation > s for s in t.shape[2:]):
        raise RuntimeError("%s: Dilation cannot be greater than size of image. " % c)
    return dilation


def _bias_checks(c, bias, channels):
    if bias.dim() != 1:
        raise RuntimeError("%s: expected a 1-dimensional bias" % c)
    if bias.shape[0] != channels:
        raise RuntimeError("%s: Bias shape does not match output channels. " % c)
    if not bias.is_contiguous():
        raise RuntimeError("%s: expected bias to be contiguous" % c)


def _ws(dev, dtype, ndim, t, c_in, c_out):
    voxels = t.shape[0]
    for s in t.shape[2:]:
        voxels *= s
    n = _lib_.msd_workspace_bytes(dtype, ndim, voxels, c_in, c_out)
    buf = _lib.workspace(dev, n)
    return buf, n


def _forward(c, relu, input, kernel, bias, output, dilation):
    dev = _same_gpu(c, input, kernel, bias, output)
    dt = _same_type(c, input, kernel, bias, output)
    _in_out_shape(c, input, output)
    _kernel_checks(c, kernel, input.dim())
    if kernel.shape[1] != input.shape[1]:
        raise RuntimeError("%s: Kernel shape does not match input channels. " % c)
    if kernel.shape[0] != output.shape[1]:
        raise RuntimeError("%s: Kernel shape does not match output channels. " % c)
    _bias_checks(c, bias, output.shape[1])
    d = _dilation(c, input, dilation)
    fn = _lib_.msd_conv_relu_forward if relu else _lib_.msd_conv_forward
    voxels = input.shape[0]
    for s in input.shape[2:]:
        voxels *= s
    need = _lib_.msd_forward_workspace_bytes(dt, input.dim(), voxels)
    ws_ptr, ws_len = None, 0
    if need:
        buf = _lib.workspace(dev, need)
        ws_ptr, ws_len = buf.data_ptr(), buf.numel()
    _lib.check(fn(dt, _lib.describe(input), kernel.data_ptr(), bias.data_ptr(), _lib.describe(output), d, ws_ptr, ws_len, dev.index,
                  _lib.stream_of(dev)))


def conv_forward(input, kernel, bias, output, dilation, block_size=None):
    """output = bias + conv_dilation(input, kernel) with edge-inclusive reflection (overwrites ``output``)."""
    _forward("conv_forward", False, input, kernel, bias, output, dilation)


def conv_relu_forward(input, kernel, bias, output, dilation, block_size=None):
    """output = max(0, bias + conv_dilation(input, kernel)) (overwrites ``output``)."""
    _forward("conv_relu_forward", True, input, kernel, bias, output, dilation)


def _backward_x(c, output, grad_output, kernel, grad_input, dilation):
    tensors = (grad_output, kernel, grad_input) if output is None else (output, grad_output, kernel, grad_input)
    dev = _same_gpu(c, *tensors)
    dt = _same_type(c, *tensors)
    _in_out_shape(c, grad_input, grad_output)
    _kernel_checks(c, kernel, grad_output.dim())
    if kernel.shape[1] != grad_input.shape[1]:
        raise RuntimeError("%s: Kernel shape does not match input channels. " % c)
    if kernel.shape[0] != grad_output.shape[1]:
        raise RuntimeError("%s: Kernel shape does not match output channels. " % c)
    d = _dilation(c, grad_output, dilation)
    if output is None:
        _lib.check(_lib_.msd_conv_backward_x(dt, _lib.describe(grad_output), kernel.data_ptr(), _lib.describe(grad_input), d, dev.index,
                                             _lib.stream_of(dev)))
    else:
        if tuple(output.shape) != tuple(grad_output.shape):
            raise RuntimeError("%s: output and grad_output differ in shape" % c)
        _lib.check(_lib_.msd_conv_relu_backward_x(dt, _lib.describe(output), _lib.describe(grad_output), kernel.data_ptr(),
                                                  _lib.describe(grad_input), d, dev.index, _lib.stream_of(dev)))


def conv_backward_x(grad_output, kernel, grad_input, dilation, block_size=None):
    """grad_input += transpose of the forward convolution applied to ``grad_output``."""
    _backward_x("conv_backward_x", None, grad_output, kernel, grad_input, dilation)


def conv_relu_backward_x(output, grad_output, kernel, grad_input, dilation, block_size=None):
    """Same with the gradient gated by ``output > 0``."""
    _backward_x("conv_relu_backward_x", output, grad_output, kernel, grad_input, dilation)


def _backward_k(c, output, grad_output, input, grad_kernel, dilation):
    tensors = (grad_output, input, grad_kernel) if output is None else (output, grad_output, input, grad_kernel)
    dev = _same_gpu(c, *tensors)
    dt = _same_type(c, *tensors)
    _in_out_shape(c, input, grad_output)
    _kernel_checks(c, grad_kernel, input.dim())
    if grad_kernel.shape[1] != input.shape[1]:
        raise RuntimeError("%s: Kernel shape does not match input channels. " % c)
    if grad_kernel.shape[0] != grad_output.shape[1]:
        raise RuntimeError("%s: Kernel shape does not match output channels. " % c)
    d = _dilation(c, input, dilation)
    buf, n = _ws(dev, dt, input.dim(), grad_output, input.shape[1], grad_output.shape[1])
    if output is None:
        _lib.check(_lib_.msd_conv_backward_k(dt, _lib.describe(grad_output), _lib.describe(input), grad_kernel.data_ptr(), d, buf.data_ptr(),
                                             buf.numel(), dev.index, _lib.stream_of(dev)))
    else:
        if tuple(output.shape) != tuple(grad_output.shape):
            raise RuntimeError("%s: output and grad_output differ in shape" % c)
        _lib.check(_lib_.msd_conv_relu_backward_k(dt, _lib.describe(output), _lib.describe(grad_output), _lib.describe(input),
                                                  grad_kernel.data_ptr(), d, buf.data_ptr(), buf.numel(), dev.index, _lib.stream_of(dev)))


def conv_backward_k(grad_output, input, grad_kernel, dilation, block_size=None):
    """grad_kernel += gradient of the convolution weights (deterministic two-pass reduction)."""
    _backward_k("conv_backward_k", None, grad_output, input, grad_kernel, dilation)


def conv_relu_backward_k(output, grad_output, input, grad_kernel, dilation, block_size=None):
    """Same with the gradient gated by ``output > 0``."""
    _backward_k("conv_relu_backward_k", output, grad_output, input, grad_kernel, dilation)


def _backward_bias(c, output, grad_output, grad_bias):
    tensors = (grad_output, grad_bias) if output is None else (output, grad_output, grad_bias)
    dev = _same_gpu(c, *tensors)
    dt = _same_type(c, *tensors)
    if grad_output.dim() not in (4, 5):
        raise RuntimeError("%s: expected a 4- or 5-dimensional grad_output" % c)
    _bias_checks(c, grad_bias, grad_output.shape[1])
    buf, n = _ws(dev, dt, grad_output.dim(), grad_output, 1, grad_output.shape[1])
    if output is None:
        _lib.check(_lib_.msd_conv_backward_bias(dt, _lib.describe(grad_output), grad_bias.data_ptr(), buf.data_ptr(), buf.numel(), dev.index,
                                                _lib.stream_of(dev)))
    else:
        _in_out_shape(c, output, grad_output)
        if output.shape[1] != grad_output.shape[1]:
            raise RuntimeError("%s: output and grad_output differ in channels" % c)
        _lib.check(_lib_.msd_conv_relu_backward_bias(dt, _lib.describe(output), _lib.describe(grad_output), grad_bias.data_ptr(), buf.data_ptr(),
                                                     buf.numel(), dev.index, _lib.stream_of(dev)))


def conv_backward_bias(grad_output, grad_bias, block_size=None):
    """grad_bias += grad_output summed over batch and space."""
    _backward_bias("conv_backward_bias", None, grad_output, grad_bias)


def conv_relu_backward_bias(output, grad_output, grad_bias, block_size=None):
    """Same with the gradient gated by ``output > 0``."""
    _backward_bias("conv_relu_backward_bias", output, grad_output, grad_bias)
