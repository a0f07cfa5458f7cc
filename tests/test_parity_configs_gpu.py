"""Element-wise parity on the benchmark configurations themselves, against the REFERENCE's own
CUDA kernels (its ten native sources compiled unmodified into ``oracle/_ref``).

For each configuration the benchmark's seeded inputs and weights go through this package's
public model API (dense block + fused final 1x1 layer + loss, forward and backward) and
through a replay of the reference's op sequence (msd_pytorch/msd_block.py:40-58 forward loop,
:88-130 backward loop) on the reference's kernels.  The reference's float64 instantiation is
the truth; its float32 instantiation is run beside it and its deviation recorded for
context.  Tolerances are the parity gate's: activations rtol 1e-4, gradients rtol 1e-3,
relative to |value| + RMS(tensor).  The gradient truth is computed with the ReLU gates taken
from this package's own float32 activations (a pre-activation within rounding of zero may be
'on' in one precision and 'off' in the other; that is not a kernel error).
"""
import json
import os

import pytest
import torch

import bench
from util import assert_close

pytestmark = pytest.mark.gpu


def _ref_module():
    from oracle import build_ref

    if build_ref.built_path() is None:
        pytest.fail("oracle/_ref (the reference's CUDA extension) is not built; run `python __graft_entry__.py` where the "
                    "reference checkout is available")
    return build_ref.load()


def _block_sizes(nd):
    # the reference's default launch shapes (msd_pytorch/conv2d.py:8-37, conv3d.py:8-37)
    if nd == 2:
        return {"f": (0, 16, 16), "x": (0, 16, 16), "k": (0, 16, 16), "b": (0, 16, 16)}
    return {"f": (2, 2, 32), "x": (2, 4, 16), "k": (2, 8, 16), "b": (8, 8, 8)}


def ref_forward(cc, x, ws, bias, dil):
    """MSDBlockFunction.forward of the reference on its own kernels."""
    nd = x.dim() - 2
    bs = _block_sizes(nd)
    depth = len(ws)
    res = x.new_empty((x.shape[0], 1 + depth) + tuple(x.shape[2:]))
    res[:, :1] = x
    for i in range(depth):
        cc.conv_relu_forward(res[:, :1 + i], ws[i], bias[i:i + 1], res[:, 1 + i:2 + i], dil[i], block_size=bs["f"])
    return res


def ref_backward(cc, res, grads, ws, dil):
    """MSDBlockFunction.backward of the reference on its own kernels; ``grads`` is updated in
    place like the reference's private clone.  Returns (grad_bias, [grad_weight_i])."""
    nd = res.dim() - 2
    bs = _block_sizes(nd)
    depth = len(ws)
    gb = res.new_zeros(depth)
    gws = [None] * depth
    for i in range(depth - 1, -1, -1):
        n = 1 + i
        so, sg = res[:, n:n + 1], grads[:, n:n + 1]
        cc.conv_relu_backward_x(so, sg, ws[i], grads[:, :n], dil[i], block_size=bs["x"])
        gws[i] = torch.zeros_like(ws[i])
        cc.conv_relu_backward_k(so, sg, res[:, :n], gws[i], dil[i], block_size=bs["k"])
        cc.conv_relu_backward_bias(so, sg, gb[i:i + 1], block_size=bs["b"])
    return gb, gws


def _worst(actual, expected):
    a, e = actual.detach().double(), expected.detach().double()
    scale = float(e.pow(2).mean().sqrt())
    return float(((a - e).abs() / (e.abs() + scale + 1e-300)).max())


def _head(res, fw, fb, y, loss):
    """Final 1x1 layer + loss on the dense buffer (float64): loss value and its gradient with
    respect to the layer's output."""
    B, C = res.shape[:2]
    out = (torch.einsum("oc,bcv->bov", fw, res.reshape(B, C, -1)) + fb[None, :, None]).reshape((B, fw.shape[0]) + tuple(res.shape[2:]))
    out.requires_grad_(True)
    if loss == "nll":
        val = torch.nn.functional.nll_loss(torch.log_softmax(out, dim=1), y)
    else:
        val = torch.nn.functional.mse_loss(out, y)
    (gout,) = torch.autograd.grad(val, out)
    return val.detach(), out.detach(), gout


CASES = [
    # name, config, batch (None: the configuration's own)
    ("c2_2d_512_depth100_batch8", "c2", None),
    ("c3_2d_1024_depth100_4classes_batch2", "c3", 2),
    ("c4_3d_128_depth50_batch2", "c4", None),
]


@pytest.mark.parametrize("name,config,batch", CASES, ids=[c[0] for c in CASES])
def test_benchmark_config_matches_reference_kernels(cuda_device, name, config, batch):
    from msd_pytorch_b200 import _lib
    from msd_pytorch_b200.msd_block import block_forward_

    dev = cuda_device
    cc = _ref_module()
    cfg = dict(bench.CONFIGS[config])
    nd, depth = cfg["ndim"], cfg["depth"]
    B = batch or cfg["batch"]
    dil = [1 + (i % 10) for i in range(depth)]
    x, y = bench.make_data(cfg, B, 1000)
    ws, fw, fb = bench.make_weights(cfg, 4242)
    xd = x.to(dev)
    yd = (y.squeeze(1) if cfg["loss"] == "nll" else y).to(dev)
    ws_d = [w.to(dev) for w in ws]
    bias = torch.zeros(depth, device=dev)
    report = {"config": config, "batch": B}

    # ---- activations: this package's block forward against the reference kernels ----
    res = torch.empty((B, 1 + depth) + tuple(cfg["spatial"]), device=dev)
    res[:, :1] = xd
    before = _lib.launch_counts()
    block_forward_(res, 1, dil, bias, ws_d)
    torch.cuda.synchronize()
    assert _lib.launch_counts()[1] - before[1] >= depth, "the tuned kernels did not run"
    truth_res = ref_forward(cc, xd.double(), [w.double() for w in ws_d], bias.double(), dil)
    ref32_res = ref_forward(cc, xd, ws_d, bias, dil)
    torch.cuda.synchronize()
    report["activations_worst"] = _worst(res, truth_res)
    report["activations_worst_reference_f32"] = _worst(ref32_res, truth_res)
    assert_close(res, truth_res, 1e-4, "activations")
    del truth_res, ref32_res

    # ---- gradients: the public model API (block + fused final layer + loss) ----
    model = bench.build_model(cfg, dev)
    xg = xd.clone().requires_grad_(True)
    out = model.net(xg)
    loss = model.criterion(out, yd)
    loss.backward()
    torch.cuda.synchronize()
    assert _lib.device_status(dev) == 0

    res64 = res.double()
    fw64, fb64 = fw.squeeze(-1).to(dev).double(), fb.to(dev).double()
    loss64, out64, gout64 = _head(res64, fw64, fb64, yd if cfg["loss"] == "nll" else yd.double(), cfg["loss"])
    assert abs(loss.item() - loss64.item()) <= 1e-4 * abs(loss64.item())
    if cfg["loss"] == "nll":
        assert_close(out, torch.log_softmax(out64, dim=1), 1e-4, "network output")
    else:
        assert_close(out, out64, 1e-4, "network output")
    C = 1 + depth
    flat = gout64.reshape(B, gout64.shape[1], -1)
    gfw64 = torch.einsum("bov,bcv->oc", flat, res64.reshape(B, C, -1))
    gfb64 = flat.sum(dim=(0, 2))
    grads64 = torch.einsum("oc,bov->bcv", fw64, flat).reshape(res64.shape).contiguous()
    grads32 = grads64.float()
    w64 = [w.double() for w in ws_d]
    gb64, gws64 = ref_backward(cc, res64, grads64, w64, dil)
    gb32, gws32 = ref_backward(cc, res, grads32, ws_d, dil)  # the reference in float32, for context
    torch.cuda.synchronize()

    blk = model.msd.msd_block
    ours_gw = torch.cat([getattr(blk, "weight%d" % i).grad.flatten() for i in range(depth)])
    truth_gw = torch.cat([g.flatten() for g in gws64])
    report["grad_input_worst"] = _worst(xg.grad, grads64[:, :1])
    report["grad_weights_worst"] = max(_worst(getattr(blk, "weight%d" % i).grad, gws64[i]) for i in range(depth))
    report["grad_bias_worst"] = _worst(blk.bias.grad, gb64)
    report["grad_input_worst_reference_f32"] = _worst(grads32[:, :1], grads64[:, :1])
    report["grad_weights_worst_reference_f32"] = max(_worst(gws32[i], gws64[i]) for i in range(depth))
    out_dir = os.environ.get("MSD_PARITY_REPORT_DIR")
    if out_dir:
        os.makedirs(out_dir, exist_ok=True)
        with open(os.path.join(out_dir, "parity_%s.json" % config), "w") as f:
            json.dump(report, f)
    print("parity", json.dumps(report))

    assert_close(xg.grad, grads64[:, :1], 1e-3, "grad_input")
    assert_close(blk.bias.grad, gb64, 1e-3, "grad_bias")
    for i in range(depth):
        assert_close(getattr(blk, "weight%d" % i).grad, gws64[i], 1e-3, "grad_weight%d" % i)
    assert_close(ours_gw, truth_gw, 1e-3, "all weight gradients as one vector")
    assert_close(model.msd.final_layer.linear.weight.grad.squeeze(-1), gfw64, 1e-3, "grad_final_weight")
    assert_close(model.msd.final_layer.linear.bias.grad, gfb64, 1e-3, "grad_final_bias")
