"""GPU test of the z-slab decomposition: N virtual ranks on one GPU (separate local buffers,
halo exchange by copies) must reproduce the undecomposed block — forward bit-identical,
input gradient bit-identical, weight/bias gradients within the reduction tolerance."""
import pytest
import torch

from util import assert_close

pytestmark = pytest.mark.gpu


@pytest.mark.parametrize("X,depth", [(136, 7), (128, 15)])
@pytest.mark.parametrize("world", [2, 3])
def test_virtual_slabs_match_single_device(cuda_device, world, X, depth):
    # X = 128 with 8 (10 for dilations above 5) and more input channels runs the role-split 3D backward in slab mode
    from msd_pytorch_b200 import _lib
    from msd_pytorch_b200.distributed import SlabBlock, SlabPlan, VirtualRanks, slab_backward, slab_forward
    from msd_pytorch_b200.msd_block import block_backward_, block_forward_

    dev = cuda_device
    torch.manual_seed(21)
    Z, Y = 36, 24
    dil = [1, 2, 3, 4, 5, 6, 10] if depth == 7 else [1 + (i % 10) for i in range(depth)]
    halo = 10
    ws = [torch.randn(1, 1 + i, 3, 3, 3, device=dev) * (2.0 / (27 * (1 + i))) ** 0.5 for i in range(depth)]
    bias = 0.05 * torch.randn(depth, device=dev)
    x = torch.randn(1, 1, Z, Y, X, device=dev)
    gout = torch.randn(1, 1 + depth, Z, Y, X, device=dev)

    # undecomposed reference with the same kernels
    res = torch.empty(1, 1 + depth, Z, Y, X, device=dev)
    res[:, :1] = x
    block_forward_(res, 1, dil, bias, ws)
    g = gout.clone()
    gw = [torch.zeros_like(w) for w in ws]
    gb = torch.zeros_like(bias)
    block_backward_(res, g, 1, dil, ws, gw, gb)

    plan = SlabPlan(Z, world, halo)
    comm = VirtualRanks(world)
    blocks = {r: SlabBlock(plan, r, 1, depth, (Y, X), dev) for r in range(world)}
    for r, b in blocks.items():
        b.set_input(x[0, :, b.loc["g0"]:b.loc["g1"]])
    slab_forward(comm, plan, blocks, ws, bias, dil)
    for r, b in blocks.items():
        assert torch.equal(b.result[0, :, b.owned], res[0, :, b.loc["g0"]:b.loc["g1"]]), "forward differs on rank %d" % r
    for r, b in blocks.items():
        b.gradients = torch.zeros_like(b.result)
        b.gradients[0, :, b.owned] = gout[0, :, b.loc["g0"]:b.loc["g1"]]
    gws, gbs = slab_backward(comm, plan, blocks, ws, dil)
    assert _lib.device_status(dev) == 0
    for r, b in blocks.items():
        assert torch.equal(b.gradients[0, :1, b.owned], g[0, :1, b.loc["g0"]:b.loc["g1"]]), "input gradient differs on rank %d" % r
        assert_close(gbs[r], gb, 1e-4, "grad_bias")
        for a, e in zip(gws[r], gw):
            assert_close(a, e, 1e-4, "grad_weight")
