"""MSD network module = dense block + final 1x1 layer (API of the reference's
msd_pytorch/msd_module.py:7-147)."""
from math import sqrt

import numpy as np
import torch

from . import _lib
from .msd_block import MSDBlock, _voxels, block_backward_, block_forward_

DEFAULT_DILATIONS = [1, 2, 3, 4, 5, 6, 7, 8, 9, 10]


def units_in_front(c_in, width, layer_depth):
    """Number of channels a layer sees: the inputs plus ``width`` per earlier layer
    (``layer_depth`` is zero-based)."""
    return c_in + width * layer_depth


def init_convolution_weights(conv_weight, c_in, c_out, width, depth):
    """Normal initialisation of Pelt & Sethian (PNAS 115(2), 2018): one standard
    deviation for all layers, sqrt(2 / (taps * (c_in + width*(depth-1)) + c_out))
    (msd_module.py:30-57)."""
    taps = int(np.prod(conv_weight.shape[2:]))
    conv_weight.normal_(0, sqrt(2 / (taps * (c_in + width * (depth - 1)) + c_out)))


class MSDFinalLayer(torch.nn.Module):
    """1x1 convolution over all channels of the dense buffer, as a ``Conv1d`` on the
    flattened spatial view; weight and bias start at zero (msd_module.py:60-88)."""

    def __init__(self, c_in, c_out):
        super().__init__()
        self.c_in = c_in
        self.c_out = c_out
        self.linear = torch.nn.Conv1d(c_in, c_out, 1)
        self.reset_parameters()

    def forward(self, input):
        # Same arithmetic as applying ``self.linear`` (a Conv1d with kernel size 1) to the
        # flattened view, written as one matrix product per sample: the layer is a pure
        # stream over the dense channel buffer and the GEMM path keeps it near copy speed,
        # forward and backward.
        b, c_in, *size = input.shape
        flat = input.reshape(b, c_in, -1)
        out = torch.matmul(self.linear.weight[:, :, 0], flat) + self.linear.bias[None, :, None]
        return out.view(b, self.c_out, *size)

    def reset_parameters(self):
        self.linear.weight.data.zero_()
        self.linear.bias.data.zero_()


def _final_kernels_apply(result, c_out):
    """The fused final-layer kernels take float32 CUDA buffers with 16-byte aligned rows and
    at most 8 output channels."""
    return result.is_cuda and result.dtype == torch.float32 and c_out <= 8 and result.shape[-1] % 4 == 0 and result.is_contiguous()


class MSDModuleFunction(torch.autograd.Function):
    """Dense block + final 1x1 layer as ONE autograd node.

    Same arithmetic as ``MSDFinalLayer(msd_block(input, ...))`` (msd_module.py:144-147 of the
    reference).  What the fusion removes is data movement: the final layer's backward writes
    the gradient of every channel straight into the buffer that the block backward updates
    in place, so the dense gradient tensor that autograd would pass between the two nodes,
    and the copy of it that the block backward must take (msd_block.py:83), never exist."""

    @staticmethod
    def forward(ctx, input, dilations, bias, final_weight, final_bias, *weights):
        depth = len(dilations)
        assert depth == len(weights), "number of weights does not match depth"
        for i, w in enumerate(weights):
            if w.dtype != input.dtype or bias.dtype != input.dtype or final_weight.dtype != input.dtype or final_bias.dtype != input.dtype:
                raise RuntimeError("MSDModule: expected all tensors to have the same scalar type")
            if not w.is_contiguous():
                raise RuntimeError("MSDModule: expected weight%d to be contiguous" % i)
        c_in = input.shape[1]
        c_total = c_in + sum(w.shape[0] for w in weights)
        c_out = final_weight.shape[0]
        result = input.new_empty(input.shape[0], c_total, *input.shape[2:])
        result[:, :c_in] = input
        block_forward_(result, c_in, list(dilations), bias.contiguous(), [w.detach() for w in weights])
        out = input.new_empty(input.shape[0], c_out, *input.shape[2:])
        dev = input.device
        fw = final_weight.detach().reshape(c_out, c_total).contiguous()
        _lib.check(_lib.lib.msd_final_forward(_lib.MSD_F32, _lib.describe(result), fw.data_ptr(), final_bias.detach().contiguous().data_ptr(),
                                              _lib.describe(out), dev.index, _lib.stream_of(dev)))
        ctx.dilations = list(dilations)
        ctx.c_in = c_in
        ctx.save_for_backward(bias, result, final_weight, *weights)
        return out

    @staticmethod
    def backward(ctx, grad_out):
        bias, result, final_weight, *weights = ctx.saved_tensors
        dev = result.device
        c_out, c_total = final_weight.shape[0], result.shape[1]
        grad_out = grad_out.contiguous()
        if grad_out.data_ptr() % 16:
            # a dense view that starts off a 16-byte boundary: the fused kernel reads 128-bit vectors
            grad_out = grad_out.clone(memory_format=torch.contiguous_format)
        gradients = torch.empty_like(result)
        fw = final_weight.detach().reshape(c_out, c_total).contiguous()
        gfw = torch.zeros_like(fw)
        gfb = torch.zeros(c_out, dtype=result.dtype, device=dev)
        ws = _lib.workspace(dev, _lib.lib.msd_final_workspace_bytes(c_total, c_out))
        _lib.check(_lib.lib.msd_final_backward(_lib.MSD_F32, _lib.describe(result), _lib.describe(grad_out), fw.data_ptr(), _lib.describe(gradients),
                                               gfw.data_ptr(), gfb.data_ptr(), ws.data_ptr(), ws.numel(), dev.index, _lib.stream_of(dev)))
        # one zero-filled buffer for all weight gradients (a single fill instead of one per layer)
        sizes = [w.numel() for w in weights]
        flat = torch.zeros(sum(sizes), dtype=result.dtype, device=dev)
        grad_weights, off = [], 0
        for w, n in zip(weights, sizes):
            grad_weights.append(flat[off:off + n].view_as(w) if ctx.needs_input_grad[5 + len(grad_weights)] else None)
            off += n
        grad_bias = torch.zeros_like(bias) if ctx.needs_input_grad[2] else None
        block_backward_(result, gradients, ctx.c_in, ctx.dilations, [w.detach() for w in weights], grad_weights, grad_bias)
        grad_input = gradients[:, :ctx.c_in] if ctx.needs_input_grad[0] else None
        return (grad_input, None, grad_bias, gfw.view_as(final_weight), gfb, *grad_weights)


class MSDModule(torch.nn.Module):
    """``MSDModule(c_in, c_out, depth, width, dilations, ndim)``: ``dilations`` is
    repeated cyclically over the ``depth`` layers."""

    def __init__(self, c_in, c_out, depth, width, dilations=DEFAULT_DILATIONS, ndim=2):
        super().__init__()
        self.c_in = c_in
        self.c_out = c_out
        self.depth = depth
        self.width = width
        if depth < 1:
            raise ValueError(f"Depth must be at least 1. Got: {depth}.")
        if width < 1:
            raise ValueError(f"Width must be at least 1. Got: {width}.")
        self.dilations = [dilations[i % len(dilations)] for i in range(depth)]
        self.msd_block = MSDBlock(self.c_in, self.dilations, self.width, ndim=ndim)
        self.final_layer = MSDFinalLayer(c_in=c_in + width * depth, c_out=c_out)
        self.reset_parameters()

    def reset_parameters(self):
        for w in self.msd_block.weights:
            init_convolution_weights(w.data, self.c_in, self.c_out, self.width, self.depth)
        self.msd_block.bias.data.zero_()
        self.final_layer.reset_parameters()

    def forward(self, input):
        blk = self.msd_block
        if input.dim() in (4, 5) and _final_kernels_apply(input, self.c_out) and input.shape[-1] * 4 % 16 == 0:
            weights = (getattr(blk, "weight{}".format(i)) for i in range(len(blk.weights)))
            return MSDModuleFunction.apply(input.contiguous(), blk.dilations, blk.bias, self.final_layer.linear.weight,
                                           self.final_layer.linear.bias, *weights)
        return self.final_layer(blk(input))
