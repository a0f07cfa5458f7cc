"""The Mixed-Scale Dense block: ``depth`` dilated 3x3 / 3x3x3 convolutions + bias + ReLU
over ONE dense channel buffer, forward and backward.

API of the reference's msd_pytorch/msd_block.py (MSDBlockFunction :7-134, MSDBlock
:140-209, MSDBlock2d/3d :212-249).  Unlike the reference, the per-layer loop does
not run in Python: ``msd_block_forward`` / ``msd_block_backward`` of the C ABI take
the whole buffer and enqueue every layer's kernel from native code.
"""
import ctypes
import math

import torch

from . import _lib
from . import msd_custom_convolutions as cc


def _uniform_width(weights):
    w0 = weights[0].shape[0]
    return w0 if all(w.shape[0] == w0 for w in weights) else None


def _pointer_array(tensors):
    arr = (ctypes.c_void_p * len(tensors))()
    for i, t in enumerate(tensors):
        arr[i] = None if t is None else t.data_ptr()
    return arr


def _int_array(values):
    arr = (ctypes.c_int * len(values))()
    for i, v in enumerate(values):
        arr[i] = int(v)
    return arr


def _voxels(t):
    v = t.shape[0]
    for s in t.shape[2:]:
        v *= s
    return v


def block_forward_(result, c_in, dilations, bias, weights):
    """Run all layers in place on ``result`` whose first ``c_in`` channels hold the input."""
    dev = result.device
    dt = _lib.dtype_code(result.dtype)
    width = _uniform_width(weights)
    if width is not None:
        need = _lib.lib.msd_forward_workspace_bytes(dt, result.dim(), _voxels(result))
        ws_ptr, ws_len = None, 0
        if need:
            ws = _lib.workspace(dev, need)
            ws_ptr, ws_len = ws.data_ptr(), ws.numel()
        _lib.check(_lib.lib.msd_block_forward(dt, _lib.describe(result), c_in, len(weights), width, _pointer_array(weights), bias.data_ptr(),
                                              _int_array(dilations), ws_ptr, ws_len, dev.index, _lib.stream_of(dev)))
        return
    start, bstart = c_in, 0
    for w, d in zip(weights, dilations):
        o = w.shape[0]
        cc.conv_relu_forward(result[:, :start], w, bias[bstart:bstart + o], result[:, start:start + o], d)
        start += o
        bstart += o


def block_backward_(result, gradients, c_in, dilations, weights, grad_weights, grad_bias):
    """Run all layers' backward in place on ``gradients`` (layers last to first)."""
    dev = result.device
    dt = _lib.dtype_code(result.dtype)
    width = _uniform_width(weights)
    if width is not None:
        n = _lib.lib.msd_block_workspace_bytes(dt, result.dim(), _voxels(result), c_in, len(weights), width)
        ws = _lib.workspace(dev, n)
        _lib.check(_lib.lib.msd_block_backward(dt, _lib.describe(result), _lib.describe(gradients), c_in, len(weights), width,
                                               _pointer_array(weights), _int_array(dilations), _pointer_array(grad_weights),
                                               None if grad_bias is None else grad_bias.data_ptr(), ws.data_ptr(), ws.numel(), dev.index,
                                               _lib.stream_of(dev)))
        return
    end = result.shape[1]
    bend = sum(w.shape[0] for w in weights)
    for idx in range(len(weights) - 1, -1, -1):
        w = weights[idx]
        o = w.shape[0]
        start, bstart = end - o, bend - o
        sub_out, sub_gout = result[:, start:end], gradients[:, start:end]
        cc.conv_relu_backward_x(sub_out, sub_gout, w, gradients[:, :start], dilations[idx])
        if grad_weights[idx] is not None:
            cc.conv_relu_backward_k(sub_out, sub_gout, result[:, :start], grad_weights[idx], dilations[idx])
        if grad_bias is not None:
            cc.conv_relu_backward_bias(sub_out, sub_gout, grad_bias[bstart:bend])
        end, bend = start, bstart


class MSDBlockFunction(torch.autograd.Function):
    """``msd_block(input, dilations, bias, *weights)`` -> the dense buffer
    ``[B, c_in + sum(width_i), *spatial]``, which is also what is saved for backward."""

    @staticmethod
    def forward(ctx, input, dilations, bias, *weights):
        depth = len(dilations)
        assert depth == len(weights), "number of weights does not match depth"
        if input.dim() not in (4, 5):
            raise ValueError("Input to MSDBlock must be 2D or 3D")
        num_out_channels = sum(w.shape[0] for w in weights)
        assert len(bias) == num_out_channels, "number of biases does not match number of output channels from weights"
        if not input.is_cuda:
            raise RuntimeError("msd_block: expected CUDA tensors (the MSD convolutions have no CPU implementation)")
        for i, w in enumerate(weights):
            if w.dtype != input.dtype or bias.dtype != input.dtype:
                raise RuntimeError("msd_block: expected all tensors to have the same scalar type")
            if not w.is_contiguous():
                raise RuntimeError("msd_block: expected weight%d to be contiguous" % i)
        ctx.dilations = list(dilations)
        ctx.depth = depth
        c_in = input.shape[1]
        result = input.new_empty(input.shape[0], c_in + num_out_channels, *input.shape[2:])
        result[:, :c_in] = input
        block_forward_(result, c_in, ctx.dilations, bias.contiguous(), [w.detach() for w in weights])
        ctx.save_for_backward(bias, result, *weights)
        return result

    @staticmethod
    def backward(ctx, grad_output):
        bias, result, *weights = ctx.saved_tensors
        assert grad_output.dim() in (4, 5), "Mismatched tensor dimensions."
        c_in = weights[0].shape[1]
        # The layers update the gradient buffer in place, so work on a private dense copy.
        gradients = grad_output.clone(memory_format=torch.contiguous_format)
        grad_bias = torch.zeros_like(bias) if ctx.needs_input_grad[2] else None
        grad_weights = [torch.zeros_like(w) if ctx.needs_input_grad[3 + i] else None for i, w in enumerate(weights)]
        block_backward_(result, gradients, c_in, ctx.dilations, [w.detach() for w in weights], grad_weights, grad_bias)
        return (gradients[:, :c_in], None, grad_bias, *grad_weights)


msd_block = MSDBlockFunction.apply


class MSDBlock(torch.nn.Module):
    """Dense block with ``len(dilations)`` layers of ``width`` channels each.

    Parameters are named ``bias`` (length depth*width) and ``weight{i}`` of shape
    ``(width, in_channels + width*i, 3, 3[, 3])`` so that state dicts are
    interchangeable with the reference's.  Output channels: in_channels + depth*width.
    """

    def __init__(self, in_channels, dilations, width=1, ndim=2):
        super().__init__()
        if ndim not in (2, 3):
            raise ValueError("ndim must be 2 or 3")
        self.kernel_size = (3,) * ndim
        self.width = width
        self.dilations = dilations
        depth = len(dilations)
        self.bias = torch.nn.Parameter(torch.empty(depth * width))
        self.weights = []
        for i in range(depth):
            weight = torch.nn.Parameter(torch.empty(width, in_channels + width * i, *self.kernel_size))
            self.register_parameter("weight{}".format(i), weight)
            self.weights.append(weight)
        self.reset_parameters()

    def reset_parameters(self):
        for weight in self.weights:
            torch.nn.init.kaiming_uniform_(weight, a=math.sqrt(5))
        fan_in, _ = torch.nn.init._calculate_fan_in_and_fan_out(self.weights[0])
        bound = 1 / math.sqrt(fan_in)
        torch.nn.init.uniform_(self.bias, -bound, bound)

    def forward(self, input):
        # Look the weights up by attribute: after .cuda(), DataParallel replication or
        # pruning the list built in __init__ may point at stale tensors.
        weights = (getattr(self, "weight{}".format(i)) for i in range(len(self.weights)))
        return msd_block(input, self.dilations, self.bias, *weights)


class MSDBlock2d(MSDBlock):
    def __init__(self, in_channels, dilations, width=1):
        super().__init__(in_channels, dilations, width=width, ndim=2)


class MSDBlock3d(MSDBlock):
    def __init__(self, in_channels, dilations, width=1):
        super().__init__(in_channels, dilations, width=width, ndim=3)
