"""GPU parity tests of the eight convolution ops against the CPU oracle, through the
Python op module and therefore through the C ABI.  Element-wise including borders."""
import pytest
import torch

import util
from util import FWD_TOL, GRAD_TOL, assert_close

pytestmark = pytest.mark.gpu


@pytest.fixture(scope="module")
def cc(cuda_device):
    from msd_pytorch_b200 import msd_custom_convolutions

    return msd_custom_convolutions


SHAPES_2D = [
    # B, C_in, C_out, spatial, dilation
    (2, 3, 5, (29, 29), 1),
    (2, 3, 5, (29, 29), 3),
    (1, 2, 3, (21, 21), 10),
    (3, 1, 1, (7, 13), 3),
    (1, 5, 2, (4, 4), 4),       # size == dilation
    (1, 1, 1, (2, 2), 2),
    (2, 2, 2, (1, 5), 1),       # 1 x 5 image
    (1, 3, 1, (37, 53), 7),     # prime sizes
    (2, 4, 1, (64, 96), 5),
    (1, 7, 1, (40, 128), 10),
    (1, 3, 1, (130, 70), 2),
]
SHAPES_3D = [
    (1, 2, 3, (7, 7, 7), 3),
    (2, 3, 1, (5, 6, 7), 1),
    (1, 1, 1, (3, 3, 4), 3),    # size == dilation
    (1, 2, 1, (11, 7, 33), 3),
    (1, 3, 1, (12, 16, 40), 4),
    (1, 2, 2, (21, 21, 21), 10),
]


def run_case(cc, dev, shape, dtype, relu, seed=0):
    B, C, Oc, sp, d = shape
    x, k, b, go = util.make_op_inputs(B, C, Oc, sp, dtype, seed, dev)
    want = util.oracle_all(x, k, b, go, d, relu)
    got = util.cuda_all(cc, x.to(dev), k.to(dev), b.to(dev), go.to(dev), d, relu)
    torch.cuda.synchronize()
    y_o, gx_o, gk_o, gb_o = want
    y, gx, gk, gb = got
    assert_close(y, y_o, FWD_TOL[dtype], "forward")
    if relu and dtype == torch.float32:
        # Gradients are compared with the oracle's gate evaluated on the GPU's own output, so a
        # pre-activation within rounding of zero cannot turn into a spurious mismatch.
        y64 = y.double().cpu()
        from oracle import msd_oracle as O
        gx_o, gk_o, gb_o = torch.zeros_like(gx_o), torch.zeros_like(gk_o), torch.zeros_like(gb_o)
        O.conv_relu_backward_x(y64, go.double(), k.double(), gx_o, d)
        O.conv_relu_backward_k(y64, go.double(), x.double(), gk_o, d)
        O.conv_relu_backward_bias(y64, go.double(), gb_o)
    assert_close(gx, gx_o, GRAD_TOL[dtype], "grad_input")
    assert_close(gk, gk_o, GRAD_TOL[dtype], "grad_kernel")
    assert_close(gb, gb_o, GRAD_TOL[dtype], "grad_bias")


@pytest.mark.parametrize("relu", [False, True], ids=["lin", "relu"])
@pytest.mark.parametrize("dtype", [torch.float32, torch.float64], ids=["f32", "f64"])
@pytest.mark.parametrize("shape", SHAPES_2D, ids=lambda s: "x".join(map(str, s[3])) + "_d%d_c%d_o%d" % (s[4], s[1], s[2]))
def test_ops_2d(cc, cuda_device, shape, dtype, relu):
    run_case(cc, cuda_device, shape, dtype, relu)


@pytest.mark.parametrize("relu", [False, True], ids=["lin", "relu"])
@pytest.mark.parametrize("dtype", [torch.float32, torch.float64], ids=["f32", "f64"])
@pytest.mark.parametrize("shape", SHAPES_3D, ids=lambda s: "x".join(map(str, s[3])) + "_d%d_c%d_o%d" % (s[4], s[1], s[2]))
def test_ops_3d(cc, cuda_device, shape, dtype, relu):
    run_case(cc, cuda_device, shape, dtype, relu)


@pytest.mark.parametrize("nd", [2, 3])
@pytest.mark.parametrize("dtype", [torch.float32, torch.float64], ids=["f32", "f64"])
def test_channel_slice_views_and_accumulate(cc, cuda_device, nd, dtype):
    """Inputs/outputs are channel slices of ONE dense buffer (msd_block.py:42-46) and the
    gradient ops add to what is already there (conv2d_backward_x.cu:103)."""
    dev = cuda_device
    sp = (24, 40) if nd == 2 else (6, 10, 24)
    B, C, d = 2, 4, 3
    x, k, b, go = util.make_op_inputs(B, C, 1, sp, dtype, 5, dev)
    buf = torch.zeros(B, C + 3, *sp, dtype=dtype, device=dev)
    buf[:, :C] = x.to(dev)
    gbuf = torch.randn(B, C + 3, *sp, dtype=dtype, device=dev)
    gbuf[:, C:C + 1] = go.to(dev)
    before = gbuf[:, :C].clone()
    kd, bd = k.to(dev), b.to(dev)
    cc.conv_relu_forward(buf[:, :C], kd, bd, buf[:, C:C + 1], d)
    cc.conv_relu_backward_x(buf[:, C:C + 1], gbuf[:, C:C + 1], kd, gbuf[:, :C], d)
    gk = torch.ones_like(kd)
    gb = torch.full_like(bd, 2.0)
    cc.conv_relu_backward_k(buf[:, C:C + 1], gbuf[:, C:C + 1], buf[:, :C], gk, d)
    cc.conv_relu_backward_bias(buf[:, C:C + 1], gbuf[:, C:C + 1], gb)
    torch.cuda.synchronize()
    from oracle import msd_oracle as O
    y_o = torch.empty_like(go, dtype=torch.float64)
    O.conv_relu_forward(x.double(), k.double(), b.double(), y_o, d)
    assert_close(buf[:, C:C + 1], y_o, FWD_TOL[dtype], "forward into slice")
    assert float(buf[:, C + 1:].abs().sum()) == 0, "wrote outside the output slice"
    y64 = buf[:, C:C + 1].double().cpu()
    gx_o = before.double().cpu()
    O.conv_relu_backward_x(y64, go.double(), k.double(), gx_o, d)
    gk_o = torch.ones_like(k, dtype=torch.float64)
    O.conv_relu_backward_k(y64, go.double(), x.double(), gk_o, d)
    gb_o = torch.full_like(b, 2.0, dtype=torch.float64)
    O.conv_relu_backward_bias(y64, go.double(), gb_o)
    assert_close(gbuf[:, :C], gx_o, GRAD_TOL[dtype], "grad_input accumulate")
    assert_close(gk, gk_o, GRAD_TOL[dtype], "grad_kernel accumulate")
    assert_close(gb, gb_o, GRAD_TOL[dtype], "grad_bias accumulate")


def test_general_strides(cc, cuda_device):
    """Arbitrary strides: spatially transposed and batch/channel-permuted views."""
    dev = cuda_device
    x, k, b, go = util.make_op_inputs(2, 3, 2, (12, 18), torch.float32, 9, dev)
    want = util.oracle_all(x, k, b, go, 2, True)
    xs = x.to(dev).permute(0, 1, 3, 2).contiguous().permute(0, 1, 3, 2)      # x-stride != 1
    gos = go.to(dev).permute(1, 0, 2, 3).contiguous().permute(1, 0, 2, 3)    # batch/channel swapped
    y = torch.empty(2, 2, 18, 12, device=dev).permute(0, 1, 3, 2)
    gx = torch.zeros(3, 2, 12, 18, device=dev).permute(1, 0, 2, 3)
    got = util.cuda_all(cc, xs, k.to(dev), b.to(dev), gos, 2, True, y=y, gx=gx)
    torch.cuda.synchronize()
    assert_close(got[0], want[0], 1e-4, "forward")
    from oracle import msd_oracle as O
    y64 = got[0].double().cpu()
    gx_o, gk_o = torch.zeros_like(want[1]), torch.zeros_like(want[2])
    O.conv_relu_backward_x(y64, go.double(), k.double(), gx_o, 2)
    O.conv_relu_backward_k(y64, go.double(), x.double(), gk_o, 2)
    assert_close(got[1], gx_o, 1e-3, "grad_input")
    assert_close(got[2], gk_o, 1e-3, "grad_kernel")


def test_weight_and_bias_gradients_are_deterministic(cc, cuda_device):
    dev = cuda_device
    x, k, b, go = (t.to(dev) for t in util.make_op_inputs(4, 6, 1, (96, 160), torch.float32, 3, dev))
    y = torch.empty_like(go)
    cc.conv_relu_forward(x, k, b, y, 4)
    runs = []
    for _ in range(3):
        gk, gb = torch.zeros_like(k), torch.zeros_like(b)
        cc.conv_relu_backward_k(y, go, x, gk, 4)
        cc.conv_relu_backward_bias(y, go, gb)
        runs.append((gk.clone(), gb.clone()))
    torch.cuda.synchronize()
    for gk, gb in runs[1:]:
        assert torch.equal(gk, runs[0][0]) and torch.equal(gb, runs[0][1])


def test_errors(cc, cuda_device):
    """test_conv2d.py:76-106: dilation > size and mixed dtypes raise RuntimeError."""
    dev = cuda_device
    x = torch.zeros(1, 1, 2, 2, device=dev, dtype=torch.float64)
    k = torch.zeros(1, 1, 3, 3, device=dev, dtype=torch.float64)
    b = torch.zeros(1, device=dev, dtype=torch.float64)
    for d in (1, 2):
        cc.conv_forward(x, k, b, torch.empty_like(x), d, block_size=(0, 16, 16))
        cc.conv_relu_forward(x, k, b, torch.empty_like(x), d, block_size=(0, 16, 16))
    for fn in (cc.conv_forward, cc.conv_relu_forward):
        with pytest.raises(RuntimeError):
            fn(x, k, b, torch.empty_like(x), 3, block_size=(0, 16, 16))
        with pytest.raises(RuntimeError):
            fn(x, k, b, torch.empty_like(x), 0)
        with pytest.raises(RuntimeError):
            fn(x.float(), k, b, torch.empty_like(x), 1)
        with pytest.raises(RuntimeError):  # kernel must be 3x3
            fn(x, torch.zeros(1, 1, 3, 5, device=dev, dtype=torch.float64), b, torch.empty_like(x), 1)
        with pytest.raises(RuntimeError):  # kernel must be contiguous
            fn(torch.zeros(1, 2, 2, 2, device=dev, dtype=torch.float64),
               torch.zeros(1, 3, 3, 2, device=dev, dtype=torch.float64).permute(0, 3, 1, 2), b, torch.empty_like(x), 1)
        with pytest.raises(RuntimeError):
            fn(x, k, b, torch.empty(1, 1, 2, 3, device=dev, dtype=torch.float64), 1)
        with pytest.raises(RuntimeError):
            fn(x, k, torch.zeros(2, device=dev, dtype=torch.float64), torch.empty_like(x), 1)
    torch.cuda.synchronize()


def test_zero_known_answer_and_inplace_contract(cc, cuda_device):
    """test_conv2d.py:109-123 and :73: zeros in, zeros out; the supplied output IS written."""
    from msd_pytorch_b200 import conv2d, conv3d

    dev = cuda_device
    for mod, fn, sp in ((conv2d, conv2d.conv2d_relu, (8, 8)), (conv3d, conv3d.conv3d_relu, (5, 6, 7))):
        x = torch.zeros(2, 2, *sp, device=dev, dtype=torch.float64)
        k = torch.zeros(3, 2, *([3] * len(sp)), device=dev, dtype=torch.float64)
        b = torch.zeros(3, device=dev, dtype=torch.float64)
        out = torch.ones(2, 3, *sp, device=dev, dtype=torch.float64)
        y = fn(x, k, b, out, 1, 2)
        assert y.data_ptr() == out.data_ptr()
        assert float(out.abs().sum()) == 0
