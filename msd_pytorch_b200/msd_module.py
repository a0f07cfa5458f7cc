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
        b, c_in, *size = input.shape
        flat = input.reshape(b, c_in, -1)
        if input.dtype != torch.float32:
            # exactly the reference's arithmetic: the Conv1d itself on the flattened view
            return self.linear(flat).view(b, self.c_out, *size)
        # float32: the same sum written as one matrix product per sample; the layer is a pure
        # stream over the dense channel buffer and the GEMM path keeps it near copy speed,
        # forward and backward.
        out = torch.matmul(self.linear.weight[:, :, 0], flat) + self.linear.bias[None, :, None]
        return out.view(b, self.c_out, *size)

    def reset_parameters(self):
        self.linear.weight.data.zero_()
        self.linear.bias.data.zero_()


def _final_kernels_apply(result, c_out):
    """The fused final-layer kernels take float32 CUDA buffers with 16-byte aligned rows and
    at most 8 output channels."""
    return result.is_cuda and result.dtype == torch.float32 and c_out <= 8 and result.shape[-1] % 4 == 0 and result.is_contiguous()


def _scale_parts(conv):
    """(weight [c, c], bias [c]) of a 1x1(x1) convolution module used as a normalisation layer."""
    c = conv.weight.shape[0]
    return conv.weight.detach().reshape(c, c), conv.bias.detach()


class MSDModuleFunction(torch.autograd.Function):
    """Dense block + final 1x1 layer as ONE autograd node, optionally with the model's frozen
    normalisation layers folded in.

    Same arithmetic as ``scale_out(MSDFinalLayer(msd_block(scale_in(input), ...)))``
    (msd_module.py:144-147 and msd_model.py:8-45 of the reference).  What the fusion removes is
    data movement: the final layer's backward writes the gradient of every channel straight
    into the buffer that the block backward updates in place, so the dense gradient tensor that
    autograd would pass between the two nodes, and the copy of it that the block backward must
    take (msd_block.py:83), never exist.  The input normalisation happens in the copy that
    places the input into the channel buffer (one pass instead of two); the output
    normalisation is a c_out x c_out matrix applied to the final layer's WEIGHTS, so that the
    final layer's store already writes normalised values and no pass over the output is left.

    ``scales`` is ``(w_in [c_in, c_in], b_in [c_in], w_out [c_out, c_out], b_out [c_out])`` or
    None; the four are treated as constants (they are frozen in the models)."""

    @staticmethod
    def forward(ctx, input, dilations, bias, final_weight, final_bias, scales, *weights):
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
        fw = final_weight.detach().reshape(c_out, c_total)
        fb = final_bias.detach()
        ones = (1,) * (input.dim() - 2)
        if scales is None:
            result[:, :c_in] = input
            w_out = None
        else:
            w_in, b_in, w_out, b_out = scales
            if c_in == 1:
                torch.addcmul(b_in.view(1, 1, *ones), input, w_in.view(1, 1, *ones), out=result[:, :1])
            else:
                result[:, :c_in] = (torch.matmul(w_in, input.flatten(2)) + b_in.view(1, c_in, 1)).view_as(input)
            if w_out is not None:
                fb = torch.mv(w_out, fb) + b_out if c_out > 1 else fb * w_out.view(()) + b_out
                fw = torch.matmul(w_out, fw) if c_out > 1 else fw * w_out.view(())
        block_forward_(result, c_in, list(dilations), bias.contiguous(), [w.detach() for w in weights])
        out = input.new_empty(input.shape[0], c_out, *input.shape[2:])
        dev = input.device
        fw = fw.contiguous()
        _lib.check(_lib.lib.msd_final_forward(_lib.MSD_F32, _lib.describe(result), fw.data_ptr(), fb.contiguous().data_ptr(),
                                              _lib.describe(out), dev.index, _lib.stream_of(dev)))
        ctx.dilations = list(dilations)
        ctx.c_in = c_in
        ctx.w_in = None if scales is None else scales[0]
        ctx.w_out = w_out
        ctx.save_for_backward(bias, result, fw, final_weight, *weights)
        return out

    @staticmethod
    def backward(ctx, grad_out):
        bias, result, fw, final_weight, *weights = ctx.saved_tensors
        dev = result.device
        c_out, c_total = fw.shape[0], result.shape[1]
        grad_out = grad_out.contiguous()
        if grad_out.data_ptr() % 16:
            # a dense view that starts off a 16-byte boundary: the fused kernel reads 128-bit vectors
            grad_out = grad_out.clone(memory_format=torch.contiguous_format)
        gradients = torch.empty_like(result)
        gfw = torch.zeros_like(fw)
        gfb = torch.zeros(c_out, dtype=result.dtype, device=dev)
        ws = _lib.workspace(dev, _lib.lib.msd_final_workspace_bytes(c_total, c_out))
        _lib.check(_lib.lib.msd_final_backward(_lib.MSD_F32, _lib.describe(result), _lib.describe(grad_out), fw.data_ptr(), _lib.describe(gradients),
                                               gfw.data_ptr(), gfb.data_ptr(), ws.data_ptr(), ws.numel(), dev.index, _lib.stream_of(dev)))
        if ctx.w_out is not None:
            # fw = w_out @ final_weight: gradients with respect to the layer's own parameters
            if c_out > 1:
                gfw, gfb = torch.matmul(ctx.w_out.t(), gfw), torch.mv(ctx.w_out.t(), gfb)
            else:
                gfw, gfb = gfw * ctx.w_out.view(()), gfb * ctx.w_out.view(())
        # one zero-filled buffer for all weight gradients (a single fill instead of one per layer)
        sizes = [w.numel() for w in weights]
        flat = torch.zeros(sum(sizes), dtype=result.dtype, device=dev)
        grad_weights, off = [], 0
        for w, n in zip(weights, sizes):
            grad_weights.append(flat[off:off + n].view_as(w) if ctx.needs_input_grad[6 + len(grad_weights)] else None)
            off += n
        grad_bias = torch.zeros_like(bias) if ctx.needs_input_grad[2] else None
        block_backward_(result, gradients, ctx.c_in, ctx.dilations, [w.detach() for w in weights], grad_weights, grad_bias)
        grad_input = None
        if ctx.needs_input_grad[0]:
            grad_input = gradients[:, :ctx.c_in]
            if ctx.w_in is not None:
                if ctx.c_in == 1:
                    grad_input = grad_input * ctx.w_in.view(())
                else:
                    grad_input = torch.matmul(ctx.w_in.t(), grad_input.flatten(2)).view(grad_input.shape)
        return (grad_input, None, grad_bias, gfw.view_as(final_weight), gfb, None, *grad_weights)


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

    def _fused_applies(self, input):
        return input.dim() in (4, 5) and _final_kernels_apply(input, self.c_out) and input.shape[-1] * 4 % 16 == 0

    def forward(self, input):
        return self.forward_scaled(input, None, None)

    def forward_scaled(self, input, scale_in=None, scale_out=None):
        """``scale_out(self(scale_in(input)))`` for frozen 1x1 normalisation layers (either may
        be None).  On the fused path the two layers cost no pass over the data of their own."""
        blk = self.msd_block
        frozen = all(not p.requires_grad for m in (scale_in, scale_out) if m is not None for p in m.parameters())
        if self._fused_applies(input) and frozen:
            weights = (getattr(blk, "weight{}".format(i)) for i in range(len(blk.weights)))
            scales = None
            if scale_in is not None or scale_out is not None:
                dev, dt = input.device, input.dtype
                w_in, b_in = _scale_parts(scale_in) if scale_in is not None else (torch.eye(self.c_in, device=dev, dtype=dt), torch.zeros(self.c_in, device=dev, dtype=dt))
                w_out, b_out = _scale_parts(scale_out) if scale_out is not None else (None, None)
                scales = (w_in, b_in, w_out, b_out)
            return MSDModuleFunction.apply(input.contiguous(), blk.dilations, blk.bias, self.final_layer.linear.weight,
                                           self.final_layer.linear.bias, scales, *weights)
        x = input if scale_in is None else scale_in(input)
        y = self.final_layer(blk(x))
        return y if scale_out is None else scale_out(y)
