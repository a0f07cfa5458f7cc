"""Single-convolution layer of the Python API, shared by ``conv2d`` and ``conv3d``.

Mirrors the op shims and the standalone autograd functions / modules of the
reference (msd_pytorch/conv2d.py:8-145, msd_pytorch/conv3d.py:8-149): each
function writes into a caller-supplied ``output`` tensor and the backward ops
accumulate into zero-initialised gradients.
"""
import torch
from torch.autograd import Function

from . import msd_custom_convolutions as cc


def make_namespace(ndim):
    """Build the functions and classes of ``conv{ndim}d`` as a dict of name -> object."""
    tag = "conv%dd" % ndim
    cls_tag = "Conv2d" if ndim == 2 else "Conv3D"
    ksize = (3,) * ndim

    def forward(input, weight, bias, output, dilation, block_size=None):
        cc.conv_forward(input, weight, bias, output, dilation, block_size=block_size)

    def backward_x(grad_output, weight, grad_input, dilation, block_size=None):
        cc.conv_backward_x(grad_output, weight, grad_input, dilation, block_size=block_size)

    def backward_k(grad_output, input, grad_weight, dilation, block_size=None):
        cc.conv_backward_k(grad_output, input, grad_weight, dilation, block_size=block_size)

    def backward_bias(grad_output, grad_bias, block_size=None):
        cc.conv_backward_bias(grad_output, grad_bias, block_size=block_size)

    def relu_forward(input, weight, bias, output, dilation, block_size=None):
        cc.conv_relu_forward(input, weight, bias, output, dilation, block_size=block_size)

    def relu_backward_x(output, grad_output, weight, grad_input, dilation, block_size=None):
        cc.conv_relu_backward_x(output, grad_output, weight, grad_input, dilation, block_size=block_size)

    def relu_backward_k(output, grad_output, input, grad_weight, dilation, block_size=None):
        cc.conv_relu_backward_k(output, grad_output, input, grad_weight, dilation, block_size=block_size)

    def relu_backward_bias(output, grad_output, grad_bias, block_size=None):
        cc.conv_relu_backward_bias(output, grad_output, grad_bias, block_size=block_size)

    class ConvFunction(Function):
        """``conv(input, weight, bias, output, stride, dilation)`` -> ``output`` (written in place)."""

        @staticmethod
        def forward(ctx, input, weight, bias, output, stride, dilation):
            ctx.save_for_backward(input, weight, bias)
            ctx.dilation = dilation
            forward(input, weight, bias, output.data, dilation)
            return output

        @staticmethod
        def backward(ctx, grad_output):
            input, weight, bias = ctx.saved_tensors
            grad_output = grad_output.contiguous()
            grad_input = torch.zeros_like(input)
            backward_x(grad_output, weight, grad_input, ctx.dilation)
            grad_weight = torch.zeros_like(weight)
            backward_k(grad_output, input, grad_weight, ctx.dilation)
            grad_bias = torch.zeros_like(bias)
            backward_bias(grad_output, grad_bias)
            return grad_input, grad_weight, grad_bias, None, None, None, None

    class ConvReluFunction(Function):
        """Same with a fused ReLU; the saved ``output`` gates the gradients."""

        @staticmethod
        def forward(ctx, input, weight, bias, output, stride, dilation):
            ctx.dilation = dilation
            relu_forward(input, weight, bias, output.data, dilation)
            ctx.save_for_backward(input, output, weight, bias)
            return output

        @staticmethod
        def backward(ctx, grad_output):
            input, output, weight, bias = ctx.saved_tensors
            grad_output = grad_output.contiguous()
            grad_input = torch.zeros_like(input)
            relu_backward_x(output, grad_output, weight, grad_input, ctx.dilation)
            grad_weight = torch.zeros_like(weight)
            relu_backward_k(output, grad_output, input, grad_weight, ctx.dilation)
            grad_bias = torch.zeros_like(bias)
            relu_backward_bias(output, grad_output, grad_bias)
            return grad_input, grad_weight, grad_bias, None, None, None, None

    def _module(fn, name):
        class _M(torch.nn.Module):
            def __init__(self, output, in_channels, out_channels, kernel_size=3, dilation=1):
                super().__init__()
                if kernel_size != 3:
                    raise ValueError("only 3-wide kernels are supported")
                self.weight = torch.nn.Parameter(torch.empty(out_channels, in_channels, *ksize, device="cuda"))
                self.bias = torch.nn.Parameter(torch.empty(out_channels, device="cuda"))
                self.output = output
                self.dilation = dilation
                self.stride = 1

            def forward(self, input):
                assert self.output.is_cuda
                return fn(input, self.weight, self.bias, self.output, self.stride, self.dilation)

        _M.__name__ = _M.__qualname__ = name
        return _M

    ConvFunction.__name__ = ConvFunction.__qualname__ = cls_tag + "Function"
    ConvReluFunction.__name__ = ConvReluFunction.__qualname__ = cls_tag + "ReluFunction"
    conv = ConvFunction.apply
    conv_relu = ConvReluFunction.apply
    return {
        tag + "_forward": forward,
        tag + "_backward_x": backward_x,
        tag + "_backward_k": backward_k,
        tag + "_backward_bias": backward_bias,
        tag + "_relu_forward": relu_forward,
        tag + "_relu_backward_x": relu_backward_x,
        tag + "_relu_backward_k": relu_backward_k,
        tag + "_relu_backward_bias": relu_backward_bias,
        cls_tag + "Function": ConvFunction,
        cls_tag + "ReluFunction": ConvReluFunction,
        tag: conv,
        tag + "_relu": conv_relu,
        cls_tag + "Module": _module(conv, cls_tag + "Module"),
        cls_tag + "ReluModule": _module(conv_relu, cls_tag + "ReluModule"),
    }
