"""CPU tests that pin the oracle (oracle/msd_oracle.py).

They restate, for the CPU oracle, every invariant the reference's own GPU tests hold for
the convolution path (ahendriksen/msd_pytorch, msd_pytorch/tests/test_conv2d.py,
test_conv3d.py, test_msd_block.py), and check the oracle against the committed golden
vectors, including the ones produced by the reference's own CUDA kernels.
"""
import os

import numpy as np
import pytest
import torch

import cases
from oracle import msd_oracle as O

GOLD = os.path.join(os.path.dirname(__file__), "golden")
dd = torch.float64


def test_reflect_map():
    # kernel_utils.cuh:30-38: -k -> k-1, n-1+k -> n-k; NOT torch's "reflect" padding.
    assert [O.reflect(i, 5) for i in range(-3, 8)] == [2, 1, 0, 0, 1, 2, 3, 4, 4, 3, 2]
    x = torch.arange(5.0).view(1, 1, 1, 5).expand(1, 1, 5, 5)
    assert O.symmetric_pad(x, 2)[0, 0, 2].tolist() == [1, 0, 0, 1, 2, 3, 4, 4, 3]


@pytest.mark.parametrize("case", cases.OP_CASES, ids=lambda c: c[0])
def test_vectorised_equals_loops_golden(case):
    """Vectorised oracle == loop restatement (stored as golden vectors)."""
    gold = np.load(os.path.join(GOLD, "oracle_ops.npz"))
    a = cases.op_inputs(case)
    x, k, b, g = (torch.from_numpy(a[n]) for n in ("x", "k", "b", "g"))
    d = a["d"]
    for relu in (False, True):
        tag = case[0] + ("_relu" if relu else "_lin")
        y = torch.empty_like(g)
        gx, gk, gb = torch.zeros_like(x), torch.zeros_like(k), torch.zeros_like(b)
        if relu:
            O.conv_relu_forward(x, k, b, y, d)
            O.conv_relu_backward_x(y, g, k, gx, d)
            O.conv_relu_backward_k(y, g, x, gk, d)
            O.conv_relu_backward_bias(y, g, gb)
        else:
            O.conv_forward(x, k, b, y, d)
            O.conv_backward_x(g, k, gx, d)
            O.conv_backward_k(g, x, gk, d)
            O.conv_backward_bias(g, gb)
        for name, val in (("y", y), ("gx", gx), ("gk", gk), ("gb", gb)):
            np.testing.assert_allclose(val.numpy(), gold[tag + "_" + name], rtol=1e-11, atol=1e-11, err_msg=tag + name)


def _ref_cuda(name):
    p = os.path.join(GOLD, name)
    if not os.path.exists(p):
        pytest.skip("golden vectors from the reference's CUDA kernels not present: " + name)
    return np.load(p)


@pytest.mark.parametrize("case", cases.OP_CASES, ids=lambda c: c[0])
def test_oracle_matches_reference_cuda_ops(case):
    """The oracle reproduces what the reference's own kernels computed on a B200 (float64)."""
    ref = _ref_cuda("ref_cuda_ops.npz")
    gold = np.load(os.path.join(GOLD, "oracle_ops.npz"))
    for relu in ("_lin", "_relu"):
        for name in ("y", "gx", "gk", "gb"):
            key = case[0] + relu + "_" + name
            if key not in ref.files:
                pytest.skip(key + " not recorded")
            np.testing.assert_allclose(gold[key], ref[key], rtol=1e-9, atol=1e-10, err_msg=key)
        # float32 forward of the reference against the float64 oracle: forward tolerance 1e-4
        key = case[0] + relu + "_f32_y"
        np.testing.assert_allclose(ref[key], gold[case[0] + relu + "_y"], rtol=1e-4, atol=1e-4, err_msg=key)


@pytest.mark.parametrize("case", cases.BLOCK_CASES, ids=lambda c: c[0])
def test_oracle_matches_reference_cuda_block(case):
    ref = _ref_cuda("ref_cuda_block.npz")
    gold = np.load(os.path.join(GOLD, "oracle_block.npz"))
    if case[0] + "_result" not in ref.files:
        pytest.skip(case[0] + " not recorded")
    for key in gold.files:
        if key.startswith(case[0] + "_"):
            np.testing.assert_allclose(gold[key], ref[key], rtol=1e-9, atol=1e-10, err_msg=key)
            # the reference's float32 kernels against the float64 oracle, at the parity gate's
            # tolerances (forward 1e-4, gradients 1e-3, relative to |value| + RMS)
            k32 = case[0] + "_f32" + key[len(case[0]):]
            if k32 in ref.files:
                e = gold[key]
                tol = (1e-4 if key.endswith("_result") else 1e-3) * (np.abs(e) + np.sqrt(np.mean(e * e)))
                assert np.all(np.abs(ref[k32] - e) <= tol + 1e-30), k32


# ---- the reference's own test invariants, restated on the oracle ---------------------------

@pytest.mark.parametrize("nd", [2, 3])
@pytest.mark.parametrize("dilation", [1, 3, 10])
def test_interior_equals_zero_padded_torch_conv(nd, dilation):
    # test_conv2d.py:126-185 / test_conv3d.py:322-373: away from the border the op is a plain
    # zero-padded dilated convolution.
    torch.manual_seed(1)
    size = 2 * dilation + 1 if nd == 3 else 29
    sp = (size,) * nd
    x = torch.randn(2, 3, *sp, dtype=dd)
    k = torch.randn(5, 3, *([3] * nd), dtype=dd)
    b = torch.randn(5, dtype=dd)
    y = torch.empty(2, 5, *sp, dtype=dd)
    O.conv_forward(x, k, b, y, dilation)
    conv = torch.nn.functional.conv2d if nd == 2 else torch.nn.functional.conv3d
    z = conv(x, k, b, padding=dilation, dilation=dilation)
    sl = (slice(None), slice(None)) + (slice(dilation, -dilation),) * nd
    torch.testing.assert_close(y[sl], z[sl], rtol=1e-12, atol=1e-12)


@pytest.mark.parametrize("sp,d", [((7, 13), 3), ((5, 6), 5), ((11, 7, 9), 3)])
def test_backward_x_is_adjoint(sp, d):
    # test_conv2d.py:218-260 / test_conv3d.py:109-150: <A f, g> == <f, A^T g>
    torch.manual_seed(2)
    nd = len(sp)
    for _ in range(5):
        f = torch.randn(2, 3, *sp, dtype=dd)
        g = torch.randn(2, 2, *sp, dtype=dd)
        k = torch.randn(2, 3, *([3] * nd), dtype=dd)
        Af = torch.empty_like(g)
        O.conv_forward(f, k, torch.zeros(2, dtype=dd), Af, d)
        ATg = torch.zeros_like(f)
        O.conv_backward_x(g, k, ATg, d)
        assert abs((Af * g).sum() - (f * ATg).sum()) < 1e-9


@pytest.mark.parametrize("sp,d", [((25, 33), 10), ((9, 11, 7), 4)])
def test_backward_k_is_adjoint(sp, d):
    # test_conv2d.py:263-311 / test_conv3d.py:153-207: the op is linear in the kernel.
    torch.manual_seed(3)
    nd = len(sp)
    x = torch.randn(2, 2, *sp, dtype=dd)
    g = torch.randn(2, 3, *sp, dtype=dd)
    k = torch.randn(3, 2, *([3] * nd), dtype=dd)
    Ak = torch.empty_like(g)
    O.conv_forward(x, k, torch.zeros(3, dtype=dd), Ak, d)
    gk = torch.zeros_like(k)
    O.conv_backward_k(g, x, gk, d)
    assert abs((Ak * g).sum() - (k * gk).sum()) < 1e-8


def test_backward_bias_is_a_sum():
    # test_conv2d.py:314-330
    g = torch.randn(3, 4, 5, 6, dtype=dd)
    gb = torch.zeros(4, dtype=dd)
    O.conv_backward_bias(g, gb)
    torch.testing.assert_close(gb, g.sum((0, 2, 3)))


def test_zero_known_answer():
    # test_conv2d.py:109-123: all-zero input and weights give an all-zero output.
    y = torch.ones(2, 3, 8, 8, dtype=dd)
    O.conv_relu_forward(torch.zeros(2, 2, 8, 8, dtype=dd), torch.zeros(3, 2, 3, 3, dtype=dd), torch.zeros(3, dtype=dd), y, 2)
    assert y.abs().sum() == 0


def test_dilation_limits():
    # test_conv2d.py:76-90: on a 2x2 image dilation 1 and 2 work, 3 raises.
    x = torch.zeros(1, 1, 2, 2, dtype=dd)
    k = torch.zeros(1, 1, 3, 3, dtype=dd)
    b = torch.zeros(1, dtype=dd)
    for d in (1, 2):
        O.conv_forward(x, k, b, torch.empty_like(x), d)
    with pytest.raises(RuntimeError):
        O.conv_forward(x, k, b, torch.empty_like(x), 3)


@pytest.mark.parametrize("nd", [2, 3])
def test_block_gradcheck(nd):
    # test_msd_block.py:26-66: numerical gradients of the whole block in float64.
    torch.manual_seed(4)
    sp = (7, 6) if nd == 2 else (4, 5, 4)
    dil = [1, 2, 3]
    width, c_in = 2, 2
    x = torch.randn(1, c_in, *sp, dtype=dd, requires_grad=True)
    ws = [torch.randn(width, c_in + i * width, *([3] * nd), dtype=dd, requires_grad=True) for i in range(3)]
    bias = torch.randn(3 * width, dtype=dd, requires_grad=True)
    assert torch.autograd.gradcheck(lambda x, b, *w: O.MSDBlockOracleFunction.apply(x, dil, b, *w), (x, bias, *ws), atol=1e-5, rtol=1e-4)


@pytest.mark.parametrize("case", cases.BLOCK_CASES, ids=lambda c: c[0])
def test_block_equals_autograd_of_composition(case):
    """The in-place block backward equals autograd through pad+conv+relu+concat."""
    a = cases.block_inputs(case)
    x = torch.from_numpy(a["x"]).requires_grad_(True)
    ws = [torch.from_numpy(w).requires_grad_(True) for w in a["weights"]]
    bias = torch.from_numpy(a["bias"]).requires_grad_(True)
    nd = x.dim() - 2
    conv = torch.nn.functional.conv2d if nd == 2 else torch.nn.functional.conv3d
    feats = x
    off = 0
    for w, d in zip(ws, a["dilations"]):
        o = w.shape[0]
        new = torch.relu(conv(O.symmetric_pad(feats, d), w, bias[off:off + o], dilation=d))
        feats = torch.cat([feats, new], 1)
        off += o
    gout = torch.from_numpy(a["gout"])
    feats.backward(gout)
    gold = np.load(os.path.join(GOLD, "oracle_block.npz"))
    name = case[0]
    np.testing.assert_allclose(feats.detach().numpy(), gold[name + "_result"], rtol=1e-10, atol=1e-10)
    np.testing.assert_allclose(x.grad.numpy(), gold[name + "_gi"], rtol=1e-9, atol=1e-9)
    np.testing.assert_allclose(bias.grad.numpy(), gold[name + "_gb"], rtol=1e-9, atol=1e-9)
    for i, w in enumerate(ws):
        np.testing.assert_allclose(w.grad.numpy(), gold[name + "_gw%d" % i], rtol=1e-9, atol=1e-9)
