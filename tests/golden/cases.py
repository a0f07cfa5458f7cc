"""Seeded input cases shared by the golden-vector generators and the tests.

Inputs come from ``numpy.random.RandomState`` so that they are bit-identical on every
machine and library version.
"""
import numpy as np

# name, batch, c_in, c_out, spatial, dilation
OP_CASES = [
    ("2d_small", 2, 3, 2, (9, 11), 3),
    ("2d_size_eq_dilation", 1, 2, 1, (4, 5), 4),
    ("2d_wide", 1, 2, 1, (6, 40), 5),
    ("2d_aligned", 2, 3, 2, (16, 32), 3),
    ("3d_small", 1, 2, 2, (5, 6, 7), 2),
    ("3d_aligned", 1, 2, 2, (8, 8, 16), 2),
    ("3d_size_eq_dilation", 1, 1, 1, (3, 3, 4), 3),
    ("2d_dilation10", 1, 3, 1, (12, 24), 10),
    ("3d_dilation10", 1, 2, 1, (10, 11, 16), 10),
    ("3d_ragged_size_eq_dilation", 2, 2, 2, (5, 7, 9), 5),
]

# name, batch, c_in, depth, width, spatial, dilations
BLOCK_CASES = [
    ("block2d", 2, 1, 6, 1, (16, 32), [1, 2, 3, 4, 5, 6]),
    ("block2d_w2", 1, 2, 3, 2, (9, 8), [1, 2, 4]),
    ("block3d", 1, 1, 4, 1, (8, 8, 16), [1, 2, 3, 1]),
    ("block3d_ragged", 1, 1, 3, 1, (5, 7, 9), [1, 2, 3]),
    ("deep_block2d", 1, 1, 14, 1, (12, 20), [1 + (i % 10) for i in range(14)]),
    ("deep_block3d", 1, 1, 12, 1, (10, 11, 12), [1 + (i % 10) for i in range(12)]),
]


def op_inputs(case):
    name, B, C, O, sp, d = case
    rs = np.random.RandomState(abs(hash_name(name)) % (2 ** 31))
    x = rs.randn(B, C, *sp)
    k = rs.randn(O, C, *([3] * len(sp))) / np.sqrt(C * 3 ** len(sp))
    b = rs.randn(O)
    g = rs.randn(B, O, *sp)
    return dict(x=x, k=k, b=b, g=g, d=d)


def block_inputs(case):
    name, B, c_in, depth, width, sp, dil = case
    rs = np.random.RandomState(abs(hash_name(name)) % (2 ** 31))
    taps = 3 ** len(sp)
    x = rs.randn(B, c_in, *sp)
    ws = [rs.randn(width, c_in + i * width, *([3] * len(sp))) * np.sqrt(2.0 / (taps * (c_in + i * width))) for i in range(depth)]
    bias = 0.1 * rs.randn(depth * width)
    gout = rs.randn(B, c_in + depth * width, *sp)
    return dict(x=x, weights=ws, bias=bias, gout=gout, dilations=dil)


def hash_name(name):
    h = 2166136261
    for ch in name.encode():
        h = ((h ^ ch) * 16777619) & 0xFFFFFFFF
    return h
