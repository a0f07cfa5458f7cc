"""Helpers shared by the GPU parity tests."""
import numpy as np
import torch

from oracle import msd_oracle as O

# Tolerances of the parity gate: forward activations rtol 1e-4 in float32, gradients rtol
# 1e-3 (reduction order); float64 is compared far more tightly.
FWD_TOL = {torch.float32: 1e-4, torch.float64: 1e-11}
GRAD_TOL = {torch.float32: 1e-3, torch.float64: 1e-10}


def assert_close(actual, expected, rtol, what=""):
    """|a - e| <= rtol * (|e| + scale), scale = RMS of the expected tensor (so that values
    that cancel to ~0 are measured against the tensor's magnitude)."""
    a = actual.detach().double().cpu()
    e = expected.detach().double().cpu()
    assert a.shape == e.shape, (what, a.shape, e.shape)
    scale = float(e.pow(2).mean().sqrt()) if e.numel() else 0.0
    err = (a - e).abs()
    bound = rtol * (e.abs() + scale) + 1e-30
    bad = err > bound
    if bad.any():
        idx = int(torch.argmax(err - bound))
        raise AssertionError("%s: %d of %d elements off; worst at flat index %d: got %r want %r (rtol %g, scale %g)"
                             % (what, int(bad.sum()), a.numel(), idx, a.flatten()[idx].item(), e.flatten()[idx].item(), rtol, scale))


def make_op_inputs(B, C, Oc, sp, dtype, seed, device):
    g = torch.Generator().manual_seed(seed)
    nd = len(sp)
    x = torch.randn(B, C, *sp, generator=g, dtype=torch.float64)
    k = torch.randn(Oc, C, *([3] * nd), generator=g, dtype=torch.float64) / np.sqrt(C * 3 ** nd)
    b = torch.randn(Oc, generator=g, dtype=torch.float64)
    go = torch.randn(B, Oc, *sp, generator=g, dtype=torch.float64)
    return [t.to(dtype) for t in (x, k, b, go)]


def oracle_all(x, k, b, go, d, relu):
    """Float64 oracle results (y, gx, gk, gb) for float inputs given as CPU tensors."""
    x, k, b, go = (t.double() for t in (x, k, b, go))
    y = torch.empty_like(go)
    gx, gk, gb = torch.zeros_like(x), torch.zeros_like(k), torch.zeros_like(b)
    if relu:
        O.conv_relu_forward(x, k, b, y, d)
        O.conv_relu_backward_x(y, go, k, gx, d)
        O.conv_relu_backward_k(y, go, x, gk, d)
        O.conv_relu_backward_bias(y, go, gb)
    else:
        O.conv_forward(x, k, b, y, d)
        O.conv_backward_x(go, k, gx, d)
        O.conv_backward_k(go, x, gk, d)
        O.conv_backward_bias(go, gb)
    return y, gx, gk, gb


def cuda_all(cc, x, k, b, go, d, relu, y=None, gx=None):
    """Same four results from the CUDA ops (tensors already on the GPU)."""
    y = torch.empty_like(go) if y is None else y
    gx = torch.zeros_like(x) if gx is None else gx
    gk, gb = torch.zeros_like(k), torch.zeros_like(b)
    if relu:
        cc.conv_relu_forward(x, k, b, y, d)
        cc.conv_relu_backward_x(y, go, k, gx, d)
        cc.conv_relu_backward_k(y, go, x, gk, d)
        cc.conv_relu_backward_bias(y, go, gb)
    else:
        cc.conv_forward(x, k, b, y, d)
        cc.conv_backward_x(go, k, gx, d)
        cc.conv_backward_k(go, x, gk, d)
        cc.conv_backward_bias(go, gb)
    return y, gx, gk, gb


def gate_safe(y_oracle, margin=1e-3):
    """True where the ReLU pre-activation is far enough from 0 that float32 rounding cannot
    flip the gate.  (y == 0 exactly means 'off' in both implementations, but a value within
    rounding of 0 may be on in one and off in the other.)"""
    return (y_oracle == 0) | (y_oracle > margin)
