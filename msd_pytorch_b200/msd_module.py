"""MSD network module = dense block + final 1x1 layer (API of the reference's
msd_pytorch/msd_module.py:7-147)."""
from math import sqrt

import numpy as np
import torch

from .msd_block import MSDBlock

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
        return self.final_layer(self.msd_block(input))
