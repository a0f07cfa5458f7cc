"""GPU parity tests of the dense block, module and model API (mirrors the reference's
msd_pytorch/tests/test_msd_block.py, test_msd_module.py, test_msd_regression_model.py,
test_msd_segmentation_model.py, test_msd_model.py) plus golden-vector checks."""
import os

import numpy as np
import pytest
import torch

import cases
import util
from util import FWD_TOL, GRAD_TOL, assert_close

pytestmark = pytest.mark.gpu
GOLD = os.path.join(os.path.dirname(__file__), "golden")


def run_block(dev, a, dtype):
    from msd_pytorch_b200.msd_block import msd_block

    x = torch.from_numpy(a["x"]).to(dev, dtype).requires_grad_(True)
    ws = [torch.from_numpy(w).to(dev, dtype).requires_grad_(True) for w in a["weights"]]
    bias = torch.from_numpy(a["bias"]).to(dev, dtype).requires_grad_(True)
    res = msd_block(x, a["dilations"], bias, *ws)
    res.backward(torch.from_numpy(a["gout"]).to(dev, dtype))
    torch.cuda.synchronize()
    return res.detach(), x.grad, bias.grad, [w.grad for w in ws]


@pytest.mark.parametrize("dtype", [torch.float32, torch.float64], ids=["f32", "f64"])
@pytest.mark.parametrize("case", cases.BLOCK_CASES, ids=lambda c: c[0])
def test_block_against_golden(cuda_device, case, dtype):
    """Block forward/backward against the oracle's golden vectors and, where recorded, the
    vectors the reference's own CUDA kernels produced."""
    a = cases.block_inputs(case)
    res, gi, gb, gws = run_block(cuda_device, a, dtype)
    files = [np.load(os.path.join(GOLD, "oracle_block.npz"))]
    ref = os.path.join(GOLD, "ref_cuda_block.npz")
    if os.path.exists(ref):
        files.append(np.load(ref))
    name = case[0]
    for gold in files:
        if name + "_result" not in gold.files:
            continue  # recorded by the oracle only
        assert_close(res, torch.from_numpy(gold[name + "_result"]), FWD_TOL[dtype] * (1 if dtype == torch.float64 else 3), "result")
        # gradient tolerance: in float32 a ReLU gate within rounding of zero may flip; these
        # small cases were checked to have no such element (min |pre-activation| >> 1e-6).
        assert_close(gi, torch.from_numpy(gold[name + "_gi"]), GRAD_TOL[dtype], "grad_input")
        assert_close(gb, torch.from_numpy(gold[name + "_gb"]), GRAD_TOL[dtype], "grad_bias")
        for i, gw in enumerate(gws):
            assert_close(gw, torch.from_numpy(gold[name + "_gw%d" % i]), GRAD_TOL[dtype], "grad_weight%d" % i)


@pytest.mark.parametrize("case", cases.OP_CASES, ids=lambda c: c[0])
def test_ops_against_golden(cuda_device, case):
    from msd_pytorch_b200 import msd_custom_convolutions as cc

    dev = cuda_device
    a = cases.op_inputs(case)
    files = [np.load(os.path.join(GOLD, "oracle_ops.npz"))]
    ref = os.path.join(GOLD, "ref_cuda_ops.npz")
    if os.path.exists(ref):
        files.append(np.load(ref))
    for dtype in (torch.float64, torch.float32):
        x, k, b, g = (torch.from_numpy(a[n]).to(dev, dtype) for n in ("x", "k", "b", "g"))
        for relu in (False, True):
            y, gx, gk, gb = util.cuda_all(cc, x, k, b, g, a["d"], relu)
            torch.cuda.synchronize()
            tag = case[0] + ("_relu" if relu else "_lin")
            for gold in files:
                assert_close(y, torch.from_numpy(gold[tag + "_y"]), FWD_TOL[dtype], tag + " y")
                assert_close(gx, torch.from_numpy(gold[tag + "_gx"]), GRAD_TOL[dtype], tag + " gx")
                assert_close(gk, torch.from_numpy(gold[tag + "_gk"]), GRAD_TOL[dtype], tag + " gk")
                assert_close(gb, torch.from_numpy(gold[tag + "_gb"]), GRAD_TOL[dtype], tag + " gb")


def _network_case(nd, depth, B, sp, c_out, seed):
    g = torch.Generator().manual_seed(seed)
    taps = 3 ** nd
    x = torch.randn(B, 1, *sp, generator=g)
    ws = [torch.randn(1, 1 + i, *([3] * nd), generator=g) * (2.0 / (taps * (1 + i))) ** 0.5 for i in range(depth)]
    bias = 0.05 * torch.randn(depth, generator=g)
    fw = torch.randn(c_out, 1 + depth, generator=g) / (1 + depth) ** 0.5
    fb = 0.1 * torch.randn(c_out, generator=g)
    dil = [1 + (i % 10) for i in range(depth)]
    return x, ws, bias, fw, fb, dil, g


@pytest.mark.parametrize("nd,depth,B,sp", [(2, 30, 1, (256, 256)), (2, 12, 2, (64, 96)), (3, 10, 1, (24, 32, 40))],
                         ids=["c1_2d_256_depth30", "2d_small", "3d_small"])
def test_network_step_matches_oracle(cuda_device, nd, depth, B, sp):
    """Forward + backward of block -> final 1x1 layer -> MSE against the float64 CPU oracle,
    with seeded non-zero final-layer weights (the reference zero-initialises them, which
    would make every block gradient vanish).  Includes the CPU-runnable benchmark config
    (2D 256x256, depth 30, dilations 1..10 cycling)."""
    from oracle import msd_oracle as O
    from msd_pytorch_b200.msd_block import msd_block

    dev = cuda_device
    x, ws, bias, fw, fb, dil, g = _network_case(nd, depth, B, sp, 1, 1001)
    target = torch.randn(B, 1, *sp, generator=g)
    loss_o, res_o, gi_o, gb_o, gws_o, gfw_o, gfb_o = O.msd_network_step(
        x.double(), target.double(), dil, bias.double(), [w.double() for w in ws], fw.double(), fb.double(), "mse")

    xd = x.to(dev).requires_grad_(True)
    wd = [w.to(dev).requires_grad_(True) for w in ws]
    bd = bias.to(dev).requires_grad_(True)
    fwd, fbd = fw.to(dev).requires_grad_(True), fb.to(dev).requires_grad_(True)
    res = msd_block(xd, dil, bd, *wd)
    out = torch.einsum("oc,bcv->bov", fwd, res.reshape(B, 1 + depth, -1)) + fbd[None, :, None]
    loss = torch.nn.functional.mse_loss(out.reshape(B, 1, *sp), target.to(dev))
    loss.backward()
    torch.cuda.synchronize()
    assert_close(res.detach(), res_o, 1e-4, "activations")
    assert abs(loss.item() - loss_o.item()) <= 1e-4 * abs(loss_o.item())
    assert_close(xd.grad, gi_o, 1e-3, "grad_input")
    assert_close(bd.grad, gb_o, 1e-3, "grad_bias")
    assert_close(fwd.grad, gfw_o, 1e-3, "grad_final_weight")
    assert_close(torch.cat([w.grad.flatten() for w in wd]), torch.cat([w.flatten() for w in gws_o]), 1e-3, "grad_weights")


@pytest.mark.parametrize("nd", [2, 3])
def test_block_gradcheck(cuda_device, nd):
    # test_msd_block.py:26-66
    from msd_pytorch_b200.msd_block import MSDBlock2d, MSDBlock3d

    torch.manual_seed(0)
    sp = (7, 9) if nd == 2 else (4, 5, 6)
    blk = (MSDBlock2d if nd == 2 else MSDBlock3d)(2, [1, 2, 3], width=2).to(cuda_device).double()
    x = torch.randn(2, 2, *sp, dtype=torch.float64, device=cuda_device, requires_grad=True)
    assert torch.autograd.gradcheck(blk, (x,), atol=1e-5, rtol=1e-4, nondet_tol=1e-9)
    params = tuple(blk.parameters())

    def f(*ps):
        return torch.func.functional_call(blk, {n: p for (n, _), p in zip(blk.named_parameters(), ps)}, (x.detach(),))

    assert torch.autograd.gradcheck(f, params, atol=1e-5, rtol=1e-4, nondet_tol=1e-9)


def test_module_gradcheck_and_final_layer(cuda_device):
    # test_msd_module.py:19-41 (depth 9, width 2, all parameters re-randomised) and :44-84
    from msd_pytorch_b200.msd_module import MSDFinalLayer, MSDModule

    torch.manual_seed(1)
    dev = cuda_device
    net = MSDModule(2, 3, 9, 2, [1, 2, 3, 4]).to(dev).double()
    for p in net.parameters():
        p.data.normal_(0, 0.3)
    x = torch.randn(1, 2, 9, 8, dtype=torch.float64, device=dev, requires_grad=True)
    assert torch.autograd.gradcheck(net, (x,), atol=1e-4, rtol=1e-3, nondet_tol=1e-9)
    for conv, sp in ((torch.nn.Conv2d, (5, 6)), (torch.nn.Conv3d, (3, 4, 5))):
        fl = MSDFinalLayer(4, 2).to(dev)
        fl.linear.weight.data.normal_()
        fl.linear.bias.data.normal_()
        c = conv(4, 2, 1).to(dev)
        c.weight.data.copy_(fl.linear.weight.data.view_as(c.weight))
        c.bias.data.copy_(fl.linear.bias.data)
        z = torch.randn(2, 4, *sp, device=dev)
        # 5e-3: cuDNN may run the comparison convolutions in TF32
        torch.testing.assert_close(fl(z), c(z), rtol=5e-3, atol=5e-3)


def test_untrained_module_outputs_zero_and_validation(cuda_device):
    # test_msd_module.py:11-16,133-137
    from msd_pytorch_b200.msd_module import MSDModule

    net = MSDModule(1, 1, 5, 1, ndim=3).to(cuda_device)
    assert float(net(torch.randn(1, 1, 10, 11, 12, device=cuda_device)).abs().sum()) == 0
    with pytest.raises(ValueError):
        MSDModule(1, 1, 0, 1)
    with pytest.raises(ValueError):
        MSDModule(1, 1, 1, 0)


@pytest.mark.parametrize("ndim", [2, 3])
def test_regression_model_api(cuda_device, tmp_path, ndim):
    # test_msd_regression_model.py:8-61,79-143; test_msd_model.py:6-35
    from torch.utils.data import DataLoader, TensorDataset
    from msd_pytorch_b200 import MSDRegressionModel

    torch.manual_seed(2)
    sp = (20, 24) if ndim == 2 else (8, 10, 12)
    model = MSDRegressionModel(2, 3, 6, 2, dilations=[1, 2, 4, 8] if ndim == 2 else [1, 2, 3], loss="L1", ndim=ndim)
    with pytest.raises(ValueError):
        MSDRegressionModel(1, 1, 1, 1, loss="nope")
    ds = TensorDataset(torch.randn(4, 2, *sp), torch.randn(4, 3, *sp))
    dl = DataLoader(ds, batch_size=2)
    model.set_normalization(dl)
    before = [p.detach().clone() for p in model.msd.parameters()]
    model.train(dl, 5)
    assert all(not torch.equal(a, b.detach()) for a, b in zip(before, model.msd.parameters())), "all parameters must change"
    assert model.validate(dl) > 0 and model.get_loss() > 0
    assert model.get_output().shape == (2, 3, *sp)
    path = str(tmp_path / "net.torch")
    model.save(path, 7)
    saved = [p.detach().clone() for p in model.net.parameters()]
    for p in model.net.parameters():
        p.data.fill_(18.3)
    assert model.load(path) == 7
    assert all(torch.equal(a, b.detach()) for a, b in zip(saved, model.net.parameters()))
    keys = set(model.net.state_dict().keys())
    assert {"0.weight", "1.msd_block.bias", "1.msd_block.weight0", "1.final_layer.linear.weight", "2.bias"} <= keys


def test_segmentation_model_api(cuda_device):
    # test_msd_segmentation_model.py:8-57,78-139
    from msd_pytorch_b200 import MSDSegmentationModel

    torch.manual_seed(3)
    model = MSDSegmentationModel(1, 4, 5, 1)
    x = torch.randn(2, 1, 32, 40)
    labels = torch.randint(0, 4, (2, 1, 32, 40))
    before = [p.detach().clone() for p in model.msd.parameters()]
    for _ in range(6):
        model.learn(x, labels)
    assert all(not torch.equal(a, b.detach()) for a, b in zip(before, model.msd.parameters()))
    with pytest.raises(ValueError):
        model.set_target(labels + 4)
    assert "1.0.msd_block.weight0" in model.net.state_dict()


def test_data_parallel_smoke(cuda_device):
    # test_msd_regression_model.py:64-76: parallel=True runs a forward and a learn step.
    from msd_pytorch_b200 import MSDRegressionModel

    model = MSDRegressionModel(1, 1, 3, 1, parallel=True)
    x = torch.zeros(4, 1, 100, 100)
    model.forward(x, x)
    model.learn(x, x)


def test_reference_python_layers_run_on_this_backend(cuda_device):
    """install_as_reference_backend() exposes the op module under the reference's native
    module name with the reference's calling convention (five positional args + block_size)."""
    import msd_pytorch_b200

    cc = msd_pytorch_b200.install_as_reference_backend()
    import msd_custom_convolutions as again

    assert again is cc
    dev = cuda_device
    x = torch.randn(1, 2, 16, 16, device=dev)
    y = torch.empty(1, 1, 16, 16, device=dev)
    again.conv_relu_forward(x, torch.randn(1, 2, 3, 3, device=dev), torch.zeros(1, device=dev), y, 2, block_size=(0, 16, 16))
    torch.cuda.synchronize()
    assert torch.isfinite(y).all()


@pytest.mark.parametrize("nd,depth,B,sp,c_out", [(2, 10, 2, (64, 96), 1), (2, 6, 2, (40, 72), 4), (3, 6, 1, (12, 24, 40), 3)],
                         ids=["2d_regression", "2d_4_classes", "3d_3_outputs"])
def test_fused_module_matches_oracle_and_unfused(cuda_device, nd, depth, B, sp, c_out):
    """MSDModule (block + final 1x1 layer as one autograd node, gradients written in place)
    against the float64 CPU oracle and against the unfused composition of the same modules."""
    from oracle import msd_oracle as O
    from msd_pytorch_b200.msd_module import MSDModule, MSDModuleFunction

    dev = cuda_device
    x, ws, bias, fw, fb, dil, g = _network_case(nd, depth, B, sp, c_out, 77)
    target = torch.randn(B, c_out, *sp, generator=g)
    loss_o, res_o, gi_o, gb_o, gws_o, gfw_o, gfb_o = O.msd_network_step(
        x.double(), target.double(), dil, bias.double(), [w.double() for w in ws], fw.double(), fb.double(), "mse")
    net = MSDModule(1, c_out, depth, 1, dilations=dil, ndim=nd).to(dev)
    with torch.no_grad():
        for i, w in enumerate(ws):
            getattr(net.msd_block, "weight%d" % i).copy_(w)
        net.msd_block.bias.copy_(bias)
        net.final_layer.linear.weight.copy_(fw.unsqueeze(-1))
        net.final_layer.linear.bias.copy_(fb)
    xd = x.to(dev).requires_grad_(True)
    out = net(xd)
    assert isinstance(out.grad_fn, MSDModuleFunction._backward_cls) or "MSDModuleFunction" in type(out.grad_fn).__name__
    loss = torch.nn.functional.mse_loss(out, target.to(dev))
    loss.backward()
    torch.cuda.synchronize()
    assert abs(loss.item() - loss_o.item()) <= 1e-4 * abs(loss_o.item())
    assert_close(xd.grad, gi_o, 1e-3, "grad_input")
    assert_close(net.msd_block.bias.grad, gb_o, 1e-3, "grad_bias")
    assert_close(net.final_layer.linear.weight.grad.squeeze(-1), gfw_o, 1e-3, "grad_final_weight")
    assert_close(net.final_layer.linear.bias.grad, gfb_o, 1e-3, "grad_final_bias")
    for i, gw_o in enumerate(gws_o):
        assert_close(getattr(net.msd_block, "weight%d" % i).grad, gw_o, 1e-3, "grad_weight%d" % i)
    # unfused composition of the same modules
    fused = [p.grad.clone() for p in net.parameters()]
    for p in net.parameters():
        p.grad = None
    x2 = x.to(dev).requires_grad_(True)
    out2 = net.final_layer(net.msd_block(x2))
    torch.nn.functional.mse_loss(out2, target.to(dev)).backward()
    assert_close(out, out2, 1e-5, "fused vs unfused output")
    assert_close(xd.grad, x2.grad, 1e-4, "fused vs unfused grad_input")
    for a, p in zip(fused, net.parameters()):
        assert_close(a, p.grad, 1e-4, "fused vs unfused parameter gradient")


def _block_case(nd, B, sp, dil, seed):
    g = torch.Generator().manual_seed(seed)
    taps = 3 ** nd
    depth = len(dil)
    x = torch.randn(B, 1, *sp, generator=g)
    ws = [torch.randn(1, 1 + i, *([3] * nd), generator=g) * (2.0 / (taps * (1 + i))) ** 0.5 for i in range(depth)]
    bias = 0.05 * torch.randn(depth, generator=g)
    gout = torch.randn(B, 1 + depth, *sp, generator=g)
    return x, ws, bias, gout


@pytest.mark.parametrize("nd,sp,dil", [
    (2, (64, 96), [1, 2, 4, 8, 16, 32]),   # power-of-two dilations (msd_module.py:103-105 of the reference)
    (2, (48, 64), [20, 1]),                # an untuned layer BELOW a tuned one
    (2, (48, 64), [1, 20, 2]),             # ... and between two tuned ones
    (3, (24, 24, 32), [2, 20, 1, 3]),      # the same in 3D
    (2, (40, 40), [17, 18, 33]),           # no tuned layer at all
], ids=["pow2_to_32", "20_1", "1_20_2", "3d_2_20_1_3", "all_generic"])
def test_block_mixes_tuned_and_generic_layers(cuda_device, nd, sp, dil):
    """A float32 block whose layers alternate between the tuned kernels and the generic ones
    (dilations beyond the tuned range): the gated gradient hand-over between layers must only
    happen between two tuned layers.  Forward and all gradients against the float64 oracle."""
    from oracle import msd_oracle as O
    from msd_pytorch_b200 import _lib
    from msd_pytorch_b200.msd_block import msd_block

    dev = cuda_device
    x, ws, bias, gout = _block_case(nd, 2, sp, dil, 31 + len(dil))
    res_o = O.msd_block_forward(x.double(), dil, bias.double(), [w.double() for w in ws])
    before = _lib.launch_counts()
    xd = x.to(dev).requires_grad_(True)
    wd = [w.to(dev).requires_grad_(True) for w in ws]
    bd = bias.to(dev).requires_grad_(True)
    res = msd_block(xd, dil, bd, *wd)
    res.backward(gout.to(dev))
    torch.cuda.synchronize()
    after = _lib.launch_counts()
    assert _lib.device_status(dev) == 0
    if max(dil) > 16 and min(dil) <= 10:
        assert after[1] > before[1] and (after[0] - before[0]) > (after[1] - before[1]), "expected tuned AND generic launches"
    assert_close(res.detach(), res_o, 1e-4, "activations")
    # gradients with the gate taken from the GPU's own activations
    gi_o, gb_o, gws_o = O.msd_block_backward(res.detach().double().cpu(), gout.double(), dil, bias.double(), [w.double() for w in ws])
    assert_close(xd.grad, gi_o, 1e-3, "grad_input")
    assert_close(bd.grad, gb_o, 1e-3, "grad_bias")
    for i, (w, e) in enumerate(zip(wd, gws_o)):
        assert_close(w.grad, e, 1e-3, "grad_weight%d" % i)


def test_block_backward_with_frozen_weights_between_tuned_layers(cuda_device):
    """Layers whose weight gradient is not wanted run the input-gradient-only kernel, which
    cannot gate the channel below: the layer under it must then gate from the activations."""
    from oracle import msd_oracle as O
    from msd_pytorch_b200.msd_block import msd_block

    dev = cuda_device
    dil = [1, 2, 3, 4, 5]
    x, ws, bias, gout = _block_case(2, 1, (32, 64), dil, 5)
    xd = x.to(dev).requires_grad_(True)
    wd = [w.to(dev).requires_grad_(i % 2 == 0) for i, w in enumerate(ws)]
    bd = bias.to(dev).requires_grad_(True)
    res = msd_block(xd, dil, bd, *wd)
    res.backward(gout.to(dev))
    torch.cuda.synchronize()
    gi_o, gb_o, gws_o = O.msd_block_backward(res.detach().double().cpu(), gout.double(), dil, bias.double(), [w.double() for w in ws])
    assert_close(xd.grad, gi_o, 1e-3, "grad_input")
    assert_close(bd.grad, gb_o, 1e-3, "grad_bias")
    for i, (w, e) in enumerate(zip(wd, gws_o)):
        if i % 2 == 0:
            assert_close(w.grad, e, 1e-3, "grad_weight%d" % i)
        else:
            assert w.grad is None


def test_weights_written_by_the_preceding_kernel_are_seen(cuda_device):
    """A weight tensor produced by the kernel enqueued just before an op (an initialiser, an
    optimiser step) must be the one the op uses: the tuned kernels stage their weights early
    and may only overlap a predecessor that cannot write them."""
    from msd_pytorch_b200 import msd_custom_convolutions as cc
    from oracle import msd_oracle as O

    dev = cuda_device
    g = torch.Generator().manual_seed(9)
    x = torch.randn(2, 24, 128, 256, generator=g)
    k_new = torch.randn(1, 24, 3, 3, generator=g) / 15
    b = torch.zeros(1)
    xd, bd = x.to(dev), b.to(dev)
    kd = torch.zeros(1, 24, 3, 3, device=dev)
    k_src = k_new.to(dev)
    y = torch.empty(2, 1, 128, 256, device=dev)
    big = torch.empty(64 << 20, device=dev)
    for _ in range(3):
        kd.zero_()
        big.normal_()          # a long kernel, then the write of the weights right before the op
        kd.copy_(k_src)
        cc.conv_relu_forward(xd, kd, bd, y, 3)
        torch.cuda.synchronize()
        y_o = torch.empty(2, 1, 128, 256, dtype=torch.float64)
        O.conv_relu_forward(x.double(), k_new.double(), b.double(), y_o, 3)
        assert_close(y, y_o, 1e-4, "forward after a weight write")


@pytest.mark.parametrize("ndim,c_in,c_out,seg", [(2, 1, 1, False), (3, 1, 1, False), (2, 2, 3, False), (2, 1, 4, True)],
                         ids=["2d_1to1", "3d_1to1", "2d_2to3", "segmentation"])
def test_normalisation_layers_folded_into_the_module(cuda_device, ndim, c_in, c_out, seg):
    """model.net (normalisation folded into the block's first load and the final layer's
    store) against the plain composition scale_out(msd(scale_in(x))) of the same modules:
    outputs, parameter gradients and the input gradient; state-dict keys as in the reference."""
    from msd_pytorch_b200 import MSDRegressionModel, MSDSegmentationModel

    torch.manual_seed(11)
    dev = cuda_device
    sp = (24, 32) if ndim == 2 else (8, 12, 16)
    model = (MSDSegmentationModel(c_in, c_out, 5, 1, ndim=ndim) if seg else MSDRegressionModel(c_in, c_out, 5, 1, ndim=ndim))
    for p in model.msd.parameters():
        p.data.normal_(0, 0.3)
    for sm in (model.scale_in,) + (() if seg else (model.scale_out,)):
        sm.weight.data.normal_(0, 1.0)     # a full matrix, not only a diagonal
        sm.bias.data.normal_(0, 1.0)
    keys = list(model.net.state_dict().keys())
    assert keys[0] == "0.weight" and ("1.0.msd_block.bias" if seg else "1.msd_block.bias") in keys
    x = torch.randn(2, c_in, *sp, device=dev)
    x1 = x.clone().requires_grad_(True)
    out = model.net(x1)
    out.square().sum().backward()
    got = [p.grad.clone() for p in model.msd.parameters()]
    for p in model.msd.parameters():
        p.grad = None
    x2 = x.clone().requires_grad_(True)
    y = model.msd(model.scale_in(x2))
    y = torch.log_softmax(y, dim=1) if seg else model.scale_out(y)
    y.square().sum().backward()
    assert_close(out, y, 1e-5, "output")
    assert_close(x1.grad, x2.grad, 1e-4, "grad_input")
    for a, p in zip(got, model.msd.parameters()):
        assert_close(a, p.grad, 1e-4, "parameter gradient")
    assert all(p.grad is None for p in model.scale_in.parameters())


@pytest.mark.parametrize("seed", [0, 1, 2])
def test_block_gradcheck_reference_configuration(cuda_device, seed):
    """The configuration of the reference's own 2D block gradcheck (test_msd_block.py:27-46:
    3 input channels, 13x21, dilations 1..3, width 1, float64), seeded, against the oracle
    and against finite differences."""
    from oracle import msd_oracle as O
    from msd_pytorch_b200.msd_block import MSDBlock2d

    torch.manual_seed(seed)
    dev = cuda_device
    net = MSDBlock2d(3, [1, 2, 3]).to(dev).double()
    x = torch.randn(2, 3, 13, 21, dtype=torch.float64, device=dev, requires_grad=True)
    res = net(x)
    gout = torch.randn_like(res)
    res.backward(gout)
    ws = [getattr(net, "weight%d" % i).detach().cpu() for i in range(3)]
    res_o = O.msd_block_forward(x.detach().cpu(), [1, 2, 3], net.bias.detach().cpu(), ws)
    gi_o, gb_o, gws_o = O.msd_block_backward(res_o, gout.cpu(), [1, 2, 3], net.bias.detach().cpu(), ws)
    assert_close(res.detach(), res_o, 1e-11, "result")
    assert_close(x.grad, gi_o, 1e-10, "grad_input")
    assert_close(net.bias.grad, gb_o, 1e-10, "grad_bias")
    for i, e in enumerate(gws_o):
        assert_close(getattr(net, "weight%d" % i).grad, e, 1e-10, "grad_weight%d" % i)
    assert torch.autograd.gradcheck(net, (x.detach().clone().requires_grad_(True),), atol=1e-5, rtol=1e-3, nondet_tol=1e-9)


def test_inference_forward_keeps_nothing(cuda_device):
    """Inference (``model.net(x)`` under ``no_grad``, examples/getting_started.py:160-175 of the
    reference): same output as the training forward, and the dense channel buffer is released
    as soon as the output exists (nothing is saved for a backward pass)."""
    from msd_pytorch_b200 import MSDRegressionModel

    dev = cuda_device
    torch.manual_seed(5)
    model = MSDRegressionModel(1, 1, 20, 1, ndim=2)
    for p in model.msd.parameters():
        p.data.normal_(0, 0.2)
    x = torch.randn(2, 1, 256, 256, device=dev)
    y_train = model.net(x)
    torch.cuda.synchronize()
    held = torch.cuda.memory_allocated(dev)
    del y_train
    torch.cuda.synchronize()
    base = torch.cuda.memory_allocated(dev)
    with torch.no_grad():
        y = model.net(x)
    torch.cuda.synchronize()
    after = torch.cuda.memory_allocated(dev)
    buffer_bytes = 2 * 21 * 256 * 256 * 4
    assert held - base >= buffer_bytes, "the training forward keeps the channel buffer for its backward"
    assert after - base < buffer_bytes // 4, "the inference forward must not keep the channel buffer"
    y2 = model.net(x)
    assert torch.equal(y, y2.detach())


def test_data_parallel_two_gpus(cuda_device):
    """``parallel=True`` (nn.DataParallel, msd_regression_model.py:78-79 of the reference) on two
    GPUs: the ops are called from one host thread per GPU on tensors of that GPU; the result
    equals the single-GPU model with the same parameters."""
    if torch.cuda.device_count() < 2:
        pytest.skip("needs two GPUs")
    from msd_pytorch_b200 import MSDRegressionModel

    torch.manual_seed(6)
    single = MSDRegressionModel(1, 2, 8, 1, ndim=2)
    for p in single.msd.parameters():
        p.data.normal_(0, 0.2)
    multi = MSDRegressionModel(1, 2, 8, 1, ndim=2, parallel=True)
    multi.net.module.load_state_dict(single.net.state_dict())
    x, t = torch.randn(4, 1, 64, 96), torch.randn(4, 2, 64, 96)
    l1 = single.forward(x, t)
    l2 = multi.forward(x, t)
    assert abs(l1 - l2) <= 1e-5 * abs(l1)
    assert_close(multi.output, single.output, 1e-5, "DataParallel output")
    multi.learn(x, t)
