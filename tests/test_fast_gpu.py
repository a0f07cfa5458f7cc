"""GPU parity tests aimed at the tuned sm_100a kernels (float32, one output channel):
TMA-staged forward and the register-resident fused backward.  Shapes are chosen to cover
several tiles per block, ragged tile edges, every benchmark dilation, dilation == size and
the three backward modes; each test asserts that the tuned path really ran and that no
bounded wait inside the kernels ran out."""
import pytest
import torch

import util
from util import assert_close

pytestmark = pytest.mark.gpu


@pytest.fixture(scope="module")
def cc(cuda_device):
    from msd_pytorch_b200 import msd_custom_convolutions

    return msd_custom_convolutions


def _counts():
    from msd_pytorch_b200 import _lib

    return _lib.launch_counts()


def _status(dev):
    from msd_pytorch_b200 import _lib

    return _lib.device_status(dev)


def check_layer(cc, dev, B, C, sp, d, relu=True, seed=0, expect_fast=3):
    from oracle import msd_oracle as O

    x, k, b, go = util.make_op_inputs(B, C, 1, sp, torch.float32, seed, dev)
    xd, kd, bd, god = (t.to(dev) for t in (x, k, b, go))
    before = _counts()
    y, gx, gk, gb = util.cuda_all(cc, xd, kd, bd, god, d, relu)
    assert _status(dev) == 0, "a bounded wait inside a kernel ran out"
    after = _counts()
    assert after[1] - before[1] >= expect_fast, "tuned kernels did not run (forward, backward_x, backward_k)"
    y_o = torch.empty_like(go, dtype=torch.float64)
    (O.conv_relu_forward if relu else O.conv_forward)(x.double(), k.double(), b.double(), y_o, d)
    assert_close(y, y_o, 1e-4, "forward")
    y64 = y.double().cpu()
    gx_o, gk_o, gb_o = torch.zeros_like(x, dtype=torch.float64), torch.zeros_like(k, dtype=torch.float64), torch.zeros(1, dtype=torch.float64)
    if relu:
        O.conv_relu_backward_x(y64, go.double(), k.double(), gx_o, d)
        O.conv_relu_backward_k(y64, go.double(), x.double(), gk_o, d)
        O.conv_relu_backward_bias(y64, go.double(), gb_o)
    else:
        O.conv_backward_x(go.double(), k.double(), gx_o, d)
        O.conv_backward_k(go.double(), x.double(), gk_o, d)
        O.conv_backward_bias(go.double(), gb_o)
    assert_close(gx, gx_o, 1e-3, "grad_input")
    assert_close(gk, gk_o, 1e-3, "grad_kernel")
    assert_close(gb, gb_o, 1e-3, "grad_bias")


@pytest.mark.parametrize("d", [1, 2, 3, 4, 5, 6, 7, 8, 9, 10, 16])
def test_2d_every_dilation(cc, cuda_device, d):
    # the TMA forward covers dilations 1..10; 16 exercises the fused backward only
    check_layer(cc, cuda_device, 2, 5, (72, 200), d, seed=d, expect_fast=3 if d <= 10 else 2)


@pytest.mark.parametrize("d", [1, 2, 3, 4, 5, 6, 7, 8, 9, 10])
def test_3d_every_dilation(cc, cuda_device, d):
    check_layer(cc, cuda_device, 1, 3, (12, 20, 136), d, seed=100 + d, expect_fast=4)


@pytest.mark.parametrize("sp,d", [((16, 16), 16), ((10, 16), 10), ((33, 64), 7), ((5, 260), 5), ((130, 20), 3), ((512, 512), 10)])
def test_2d_edges(cc, cuda_device, sp, d):
    check_layer(cc, cuda_device, 1, 3, sp, d, seed=7, expect_fast=3 if d <= 10 else 2)


@pytest.mark.parametrize("sp,d", [((10, 10, 16), 10), ((3, 40, 24), 3), ((9, 5, 132), 4), ((32, 32, 64), 6)])
def test_3d_edges(cc, cuda_device, sp, d):
    check_layer(cc, cuda_device, 2, 2, sp, d, seed=8, expect_fast=4)


def test_many_tiles_per_block_and_many_channels(cc, cuda_device):
    """More tiles than thread blocks (persistent round-robin) and a deep channel loop."""
    check_layer(cc, cuda_device, 4, 40, (256, 512), 9, seed=11)
    check_layer(cc, cuda_device, 2, 20, (40, 48, 128), 5, seed=12, expect_fast=4)


def test_linear_variants(cc, cuda_device):
    check_layer(cc, cuda_device, 2, 4, (48, 160), 3, relu=False, seed=13)
    check_layer(cc, cuda_device, 1, 4, (8, 24, 64), 2, relu=False, seed=14, expect_fast=4)


@pytest.mark.parametrize("nd", [2, 3])
def test_fused_block_backward_matches_separate_ops(cuda_device, nd):
    """msd_block_backward (one fused kernel per layer) == the three single ops per layer."""
    from msd_pytorch_b200 import msd_custom_convolutions as cc
    from msd_pytorch_b200.msd_block import block_backward_, block_forward_

    dev = cuda_device
    torch.manual_seed(5)
    sp = (96, 256) if nd == 2 else (20, 24, 128)
    depth, B = 12, 2
    dil = [1 + (i % 10) for i in range(depth)]
    ws = [torch.randn(1, 1 + i, *([3] * nd), device=dev) * (2.0 / (3 ** nd * (1 + i))) ** 0.5 for i in range(depth)]
    bias = 0.05 * torch.randn(depth, device=dev)
    res = torch.empty(B, 1 + depth, *sp, device=dev)
    res[:, :1] = torch.randn(B, 1, *sp, device=dev)
    block_forward_(res, 1, dil, bias, ws)
    gout = torch.randn_like(res)
    g1 = gout.clone()
    gw1 = [torch.zeros_like(w) for w in ws]
    gb1 = torch.zeros_like(bias)
    block_backward_(res, g1, 1, dil, ws, gw1, gb1)
    g2 = gout.clone()
    gw2 = [torch.zeros_like(w) for w in ws]
    gb2 = torch.zeros_like(bias)
    for i in range(depth - 1, -1, -1):
        n = 1 + i
        cc.conv_relu_backward_x(res[:, n:n + 1], g2[:, n:n + 1], ws[i], g2[:, :n], dil[i])
        cc.conv_relu_backward_k(res[:, n:n + 1], g2[:, n:n + 1], res[:, :n], gw2[i], dil[i])
        cc.conv_relu_backward_bias(res[:, n:n + 1], g2[:, n:n + 1], gb2[i:i + 1])
    assert _status(dev) == 0
    assert_close(g1[:, :1], g2[:, :1], 1e-5, "grad_input")
    assert_close(gb1, gb2, 1e-5, "grad_bias")
    for a, b in zip(gw1, gw2):
        assert_close(a, b, 1e-5, "grad_weight")
    # determinism of the fused path
    g3 = gout.clone()
    gw3 = [torch.zeros_like(w) for w in ws]
    gb3 = torch.zeros_like(bias)
    block_backward_(res, g3, 1, dil, ws, gw3, gb3)
    torch.cuda.synchronize()
    assert torch.equal(g1[:, :1], g3[:, :1]) and torch.equal(gb1, gb3) and all(torch.equal(a, b) for a, b in zip(gw1, gw3))


@pytest.mark.parametrize("variant", [0, 1, 2, 3, 4, 5, 6, 7, 8])
@pytest.mark.parametrize("d", [1, 2, 3, 4, 5, 6, 7, 8, 9, 10])
def test_forward_launch_variants(cc, cuda_device, d, variant):
    """Every tile-shape variant of the TMA forward gives the oracle's result, including
    tiles on all four image borders, ragged last tiles and several tiles per block."""
    from msd_pytorch_b200 import _lib
    from oracle import msd_oracle as O

    dev = cuda_device
    assert _lib.lib.msd_tuning_num_variants(_lib.FAMILY_FWD2D) == 9
    _lib.check(_lib.lib.msd_tuning_set(_lib.FAMILY_FWD2D, d, variant))
    try:
        x, k, b, go = util.make_op_inputs(3, 4, 1, (150, 300), torch.float32, 40 + d, dev)
        y = torch.empty_like(go, device=dev)
        before = _counts()
        cc.conv_relu_forward(x.to(dev), k.to(dev), b.to(dev), y, d)
        assert _status(dev) == 0
        assert _counts()[1] - before[1] == 1
        y_o = torch.empty_like(go, dtype=torch.float64)
        O.conv_relu_forward(x.double(), k.double(), b.double(), y_o, d)
        assert_close(y, y_o, 1e-4, "forward variant %d" % variant)
    finally:
        _lib.lib.msd_tuning_set(_lib.FAMILY_FWD2D, d, -1)


@pytest.mark.parametrize("variant", [0, 1, 2, 3])
@pytest.mark.parametrize("d", [1, 2, 3, 4, 5, 6, 7, 8, 9, 10])
def test_forward3d_launch_variants(cc, cuda_device, d, variant):
    """All variants of the 3D forward (plane-wise TMA kernel + z-gather) match the oracle on a
    volume with ragged tiles in y and x and every z-plane near a border for large dilations."""
    from msd_pytorch_b200 import _lib
    from oracle import msd_oracle as O

    dev = cuda_device
    assert _lib.lib.msd_tuning_num_variants(_lib.FAMILY_FWD3D) == 4
    _lib.check(_lib.lib.msd_tuning_set(_lib.FAMILY_FWD3D, d, variant))
    try:
        x, k, b, go = util.make_op_inputs(2, 3, 1, (11, 50, 140), torch.float32, 70 + d, dev)
        y = torch.empty_like(go, device=dev)
        before = _counts()
        cc.conv_relu_forward(x.to(dev), k.to(dev), b.to(dev), y, d)
        assert _status(dev) == 0
        assert _counts()[1] - before[1] == 2
        y_o = torch.empty_like(go, dtype=torch.float64)
        O.conv_relu_forward(x.double(), k.double(), b.double(), y_o, d)
        assert_close(y, y_o, 1e-4, "forward3d variant %d" % variant)
    finally:
        _lib.lib.msd_tuning_set(_lib.FAMILY_FWD3D, d, -1)


@pytest.mark.parametrize("sp,B,depth", [((13, 23, 256), 2, 22), ((10, 11, 128), 1, 30), ((24, 40, 384), 1, 15)])
def test_backward3d_role_split_variant(cuda_device, sp, B, depth):
    """The role-split 3D backward (variant 1: X warps + K warps; layers of 8 (10 for dilations above 5) and more input
    channels) == the three single ops per layer, which the tests above hold against the oracle:
    ragged tiles in y, one and several tiles in x (both x borders in one tile when X == 128),
    every dilation 1..10, channel counts that are and are not multiples of the stage's 4."""
    from msd_pytorch_b200 import _lib
    from msd_pytorch_b200 import msd_custom_convolutions as cc
    from msd_pytorch_b200.msd_block import block_backward_, block_forward_

    dev = cuda_device
    assert _lib.lib.msd_tuning_num_variants(_lib.FAMILY_BWD3D) == 3
    torch.manual_seed(17)
    dil = [1 + (i % 10) for i in range(depth)]
    ws = [torch.randn(1, 1 + i, 3, 3, 3, device=dev) * (2.0 / (27 * (1 + i))) ** 0.5 for i in range(depth)]
    bias = 0.05 * torch.randn(depth, device=dev)
    res = torch.empty(B, 1 + depth, *sp, device=dev)
    res[:, :1] = torch.randn(B, 1, *sp, device=dev)
    block_forward_(res, 1, dil, bias, ws)
    gout = torch.randn_like(res)
    g2 = gout.clone()
    gw2 = [torch.zeros_like(w) for w in ws]
    gb2 = torch.zeros_like(bias)
    for i in range(depth - 1, -1, -1):
        n = 1 + i
        cc.conv_relu_backward_x(res[:, n:n + 1], g2[:, n:n + 1], ws[i], g2[:, :n], dil[i])
        cc.conv_relu_backward_k(res[:, n:n + 1], g2[:, n:n + 1], res[:, :n], gw2[i], dil[i])
        cc.conv_relu_backward_bias(res[:, n:n + 1], g2[:, n:n + 1], gb2[i:i + 1])
    for d in range(1, 11):
        _lib.check(_lib.lib.msd_tuning_set(_lib.FAMILY_BWD3D, d, 1))
    try:
        g1 = gout.clone()
        gw1 = [torch.zeros_like(w) for w in ws]
        gb1 = torch.zeros_like(bias)
        block_backward_(res, g1, 1, dil, ws, gw1, gb1)
        assert _status(dev) == 0
        assert_close(g1[:, :1], g2[:, :1], 1e-5, "grad_input")
        assert_close(gb1, gb2, 1e-5, "grad_bias")
        for i, (a, b) in enumerate(zip(gw1, gw2)):
            assert_close(a, b, 1e-5, "grad_weight of layer %d" % i)
        g3 = gout.clone()
        gw3 = [torch.zeros_like(w) for w in ws]
        gb3 = torch.zeros_like(bias)
        block_backward_(res, g3, 1, dil, ws, gw3, gb3)
        torch.cuda.synchronize()
        assert torch.equal(g1[:, :1], g3[:, :1]) and torch.equal(gb1, gb3) and all(torch.equal(a, b) for a, b in zip(gw1, gw3))
    finally:
        for d in range(1, 11):
            _lib.lib.msd_tuning_set(_lib.FAMILY_BWD3D, d, -1)


@pytest.mark.parametrize("sp", [(12, 22, 128), (11, 18, 256)], ids=["x128", "x256"])
def test_role_split_3d_backward_against_cpu_oracle(cuda_device, sp):
    """The role-split 3D backward kernel (X warps + K warps, used for X % 128 == 0) directly
    against the float64 CPU oracle: a depth-22 block with ragged Z and Y so that every
    dilation 1..10 runs with at least 12 input channels, the split variant forced, and the
    number of its launches asserted."""
    from oracle import msd_oracle as O
    from msd_pytorch_b200 import _lib
    from msd_pytorch_b200.msd_block import msd_block

    dev = cuda_device
    L = _lib.lib
    depth = 22
    dil = [1 + (i % 10) for i in range(depth)]
    g = torch.Generator().manual_seed(515)
    x = torch.randn(1, 1, *sp, generator=g)
    ws = [torch.randn(1, 1 + i, 3, 3, 3, generator=g) * (2.0 / (27 * (1 + i))) ** 0.5 for i in range(depth)]
    bias = 0.05 * torch.randn(depth, generator=g)
    gout = torch.randn(1, 1 + depth, *sp, generator=g)
    res_o = O.msd_block_forward(x.double(), dil, bias.double(), [w.double() for w in ws])
    old = [L.msd_tuning_get(_lib.FAMILY_BWD3D, d) for d in range(1, 11)]
    try:
        for d in range(1, 11):
            assert L.msd_tuning_set(_lib.FAMILY_BWD3D, d, 1) == 0
        split0 = L.msd_split_launch_count()
        xd = x.to(dev).requires_grad_(True)
        wd = [w.to(dev).requires_grad_(True) for w in ws]
        bd = bias.to(dev).requires_grad_(True)
        res = msd_block(xd, dil, bd, *wd)
        res.backward(gout.to(dev))
        torch.cuda.synchronize()
        # layers with >= 8 input channels (dilation <= 5) or >= 12 (above) take the split kernel
        expect = sum(1 for i in range(depth) if 1 + i >= (8 if dil[i] <= 5 else 10))
        assert L.msd_split_launch_count() - split0 == expect
        assert _lib.device_status(dev) == 0
    finally:
        for d, v in zip(range(1, 11), old):
            L.msd_tuning_set(_lib.FAMILY_BWD3D, d, v)
    assert_close(res.detach(), res_o, 1e-4, "activations")
    gi_o, gb_o, gws_o = O.msd_block_backward(res.detach().double().cpu(), gout.double(), dil, bias.double(), [w.double() for w in ws])
    assert_close(xd.grad, gi_o, 1e-3, "grad_input")
    assert_close(bd.grad, gb_o, 1e-3, "grad_bias")
    for i, (w, e) in enumerate(zip(wd, gws_o)):
        assert_close(w.grad, e, 1e-3, "grad_weight%d" % i)


@pytest.mark.parametrize("sp,B", [((37, 128), 3), ((50, 256), 2), ((21, 384), 1)], ids=["x128", "x256", "x384"])
def test_role_split_2d_backward_against_cpu_oracle(cuda_device, sp, B):
    """The role-split backward in 2D (launch variant 2 of the 2D backward: X warps, K warps
    with the ninth tap shared out over the tap lanes, builder warps) directly against the
    float64 CPU oracle: a depth-24 block with ragged Y, both x borders in one tile (X = 128)
    and interior tiles (X = 384), every dilation 1..10, channel counts 1..24 (ring stages of
    four channels that are full, partly filled and single), the number of its launches
    asserted, and two runs bit-identical."""
    from oracle import msd_oracle as O
    from msd_pytorch_b200 import _lib
    from msd_pytorch_b200.msd_block import block_backward_, block_forward_

    dev = cuda_device
    L = _lib.lib
    assert L.msd_tuning_num_variants(_lib.FAMILY_BWD2D) == 3
    depth = 24
    dil = [1 + (i % 10) for i in range(depth)]
    g = torch.Generator().manual_seed(616)
    x = torch.randn(B, 1, *sp, generator=g)
    ws = [torch.randn(1, 1 + i, 3, 3, generator=g) * (2.0 / (9 * (1 + i))) ** 0.5 for i in range(depth)]
    bias = 0.05 * torch.randn(depth, generator=g)
    gout = torch.randn(B, 1 + depth, *sp, generator=g)
    res_o = O.msd_block_forward(x.double(), dil, bias.double(), [w.double() for w in ws])
    gi_o, gb_o, gws_o = O.msd_block_backward(res_o, gout.double(), dil, bias.double(), [w.double() for w in ws])
    wd = [w.to(dev) for w in ws]
    res = torch.empty(B, 1 + depth, *sp, device=dev)
    res[:, :1] = x.to(dev)
    block_forward_(res, 1, dil, bias.to(dev), wd)
    assert_close(res, res_o, 1e-4, "activations")
    old = [L.msd_tuning_get(_lib.FAMILY_BWD2D, d) for d in range(1, 11)]
    try:
        for d in range(1, 11):
            assert L.msd_tuning_set(_lib.FAMILY_BWD2D, d, 2) == 0
        runs = []
        for _ in range(2):
            split0 = L.msd_split_launch_count()
            g1 = gout.to(dev)
            gw1 = [torch.zeros_like(w) for w in wd]
            gb1 = torch.zeros(depth, device=dev)
            block_backward_(res, g1, 1, dil, wd, gw1, gb1)
            assert _status(dev) == 0
            assert L.msd_split_launch_count() - split0 == depth
            runs.append((g1[:, :1].clone(), gb1, gw1))
    finally:
        for d, v in zip(range(1, 11), old):
            L.msd_tuning_set(_lib.FAMILY_BWD2D, d, v)
    (gi, gb, gws), (gi2, gb2, gws2) = runs
    assert torch.equal(gi, gi2) and torch.equal(gb, gb2) and all(torch.equal(a, b) for a, b in zip(gws, gws2))
    assert_close(gi, gi_o, 1e-3, "grad_input")
    assert_close(gb, gb_o, 1e-3, "grad_bias")
    for i, (w, e) in enumerate(zip(gws, gws_o)):
        assert_close(w, e, 1e-3, "grad_weight%d" % i)


def test_bounded_wait_runs_out_and_reports(cuda_device):
    """A wait on a barrier nobody arrives at gives up after its time limit: the kernel returns
    by itself, the device status word carries the code, reading it clears it, and the next
    ordinary call works."""
    import time
    from msd_pytorch_b200 import _lib
    from msd_pytorch_b200 import msd_custom_convolutions as cc

    dev = cuda_device
    L = _lib.lib
    assert _lib.device_status(dev) == 0
    t0 = time.time()
    assert L.msd_selftest_wait_timeout(1_000_000, dev.index, _lib.stream_of(dev)) == 0  # 1 ms
    assert _lib.device_status(dev) == 99  # MSD_STATUS_SELFTEST_TIMEOUT; synchronises the stream
    assert time.time() - t0 < 5.0, "the wait must end after about a millisecond"
    assert _lib.device_status(dev) == 0, "reading the status clears it"
    assert L.msd_selftest_wait_timeout(10, dev.index, _lib.stream_of(dev)) == 1  # limit outside [1e3, 1e9]
    x = torch.randn(1, 2, 32, 64, device=dev)
    y = torch.empty(1, 1, 32, 64, device=dev)
    cc.conv_relu_forward(x, torch.randn(1, 2, 3, 3, device=dev), torch.zeros(1, device=dev), y, 2)
    torch.cuda.synchronize()
    assert torch.isfinite(y).all() and _lib.device_status(dev) == 0


def _force_bwd3d(L, lib, variant):
    old = [L.msd_tuning_get(lib.FAMILY_BWD3D, d) for d in range(1, 13)]
    for d in range(1, 13):
        assert L.msd_tuning_set(lib.FAMILY_BWD3D, d, variant) == 0
    return old


def _restore_bwd3d(L, lib, old):
    for d, v in zip(range(1, 13), old):
        L.msd_tuning_set(lib.FAMILY_BWD3D, d, v)


@pytest.mark.parametrize("C,d,sp", [(8, 1, (6, 8, 128)), (23, 3, (7, 10, 128)), (50, 2, (5, 9, 256)), (50, 10, (12, 11, 128)), (64, 4, (4, 6, 128)),
                                    (65, 12, (13, 14, 128)), (72, 5, (6, 7, 128))],
                         ids=["c8_d1", "c23_d3", "c50_d2_x256", "c50_d10", "c64_d4", "c65_d12", "c72_d5"])
def test_backward3d_tensor_core_variant_single_layer(cuda_device, C, d, sp):
    """One layer's fused backward with the input gradient on the tensor cores (3D backward variant
    2: TF32 MMAs with error-compensated operand splitting; weight gradient on the CUDA cores)
    against the float64 CPU oracle, gradient tolerances of the parity gate; odd row counts and
    channel counts that are no multiple of the ring stage included."""
    from oracle import msd_oracle as O
    from msd_pytorch_b200 import _lib
    from msd_pytorch_b200.msd_block import block_backward_

    dev = cuda_device
    L = _lib.lib
    g = torch.Generator().manual_seed(1000 + C + d)
    res = torch.randn(1, C + 1, *sp, generator=g)
    res[:, C] = torch.relu(res[:, C])                      # the layer's output channel: about half the gates closed
    grad = torch.randn(1, C + 1, *sp, generator=g)
    w = torch.randn(1, C, 3, 3, 3, generator=g) * (2.0 / (27 * C)) ** 0.5
    gx_o = grad[:, :C].double().clone()
    gk_o = torch.zeros(1, C, 3, 3, 3, dtype=torch.float64)
    gb_o = torch.zeros(1, dtype=torch.float64)
    O.conv_relu_backward_x(res[:, C:].double(), grad[:, C:].double(), w.double(), gx_o, d)
    O.conv_relu_backward_k(res[:, C:].double(), grad[:, C:].double(), res[:, :C].double(), gk_o, d)
    O.conv_relu_backward_bias(res[:, C:].double(), grad[:, C:].double(), gb_o)
    old = _force_bwd3d(L, _lib, 2)
    try:
        n0 = L.msd_mma_launch_count()
        rd, gd, wd = res.to(dev), grad.to(dev), w.to(dev)
        gw, gb = torch.zeros_like(wd), torch.zeros(1, device=dev)
        block_backward_(rd, gd, C, [d], [wd], [gw], gb)
        torch.cuda.synchronize()
        assert _lib.device_status(dev) == 0
        assert L.msd_mma_launch_count() - n0 == 1, "the tensor-core kernel did not run"
    finally:
        _restore_bwd3d(L, _lib, old)

    def worst(a, e):
        e = e.double()
        return float(((a.double().cpu() - e).abs() / (e.abs() + e.pow(2).mean().sqrt())).max())

    print("tensor-core backward C=%d d=%d: worst relative deviation gin %.3g, gk %.3g, gb %.3g"
          % (C, d, worst(gd[:, :C], gx_o), worst(gw, gk_o), worst(gb, gb_o)))
    assert_close(gd[:, :C], gx_o, 1e-3, "grad_input")
    assert_close(gw, gk_o, 1e-3, "grad_kernel")
    assert_close(gb, gb_o, 1e-3, "grad_bias")
    assert worst(gd[:, :C], gx_o) < 2e-5 and worst(gw, gk_o) < 2e-5, "3xTF32 should be as accurate as float32"


def test_backward3d_tensor_core_variant_in_a_block(cuda_device):
    """A depth-22 block whose layers with 8 and more input channels run on the tensor cores,
    against the float64 oracle (gated hand-over between the layers included)."""
    from oracle import msd_oracle as O
    from msd_pytorch_b200 import _lib
    from msd_pytorch_b200.msd_block import msd_block

    dev = cuda_device
    L = _lib.lib
    depth, sp = 22, (12, 22, 128)
    dil = [1 + (i % 10) for i in range(depth)]
    g = torch.Generator().manual_seed(77)
    x = torch.randn(1, 1, *sp, generator=g)
    ws = [torch.randn(1, 1 + i, 3, 3, 3, generator=g) * (2.0 / (27 * (1 + i))) ** 0.5 for i in range(depth)]
    bias = 0.05 * torch.randn(depth, generator=g)
    gout = torch.randn(1, 1 + depth, *sp, generator=g)
    old = _force_bwd3d(L, _lib, 2)
    try:
        n0 = L.msd_mma_launch_count()
        xd = x.to(dev).requires_grad_(True)
        wd = [w.to(dev).requires_grad_(True) for w in ws]
        bd = bias.to(dev).requires_grad_(True)
        res = msd_block(xd, dil, bd, *wd)
        res.backward(gout.to(dev))
        torch.cuda.synchronize()
        assert L.msd_mma_launch_count() - n0 == sum(1 for i in range(depth) if 1 + i >= 8)
        assert _lib.device_status(dev) == 0
    finally:
        _restore_bwd3d(L, _lib, old)
    gi_o, gb_o, gws_o = O.msd_block_backward(res.detach().double().cpu(), gout.double(), dil, bias.double(), [w.double() for w in ws])
    assert_close(xd.grad, gi_o, 1e-3, "grad_input")
    assert_close(bd.grad, gb_o, 1e-3, "grad_bias")
    for i, (w, e) in enumerate(zip(wd, gws_o)):
        assert_close(w.grad, e, 1e-3, "grad_weight%d" % i)
