"""Size-independent properties of the CUDA path at the benchmark's full sizes, where the CPU
oracle would take minutes: adjointness of backward_x, linearity in the kernel (backward_k),
bias sums, batch additivity of the gradients (what batch data-parallelism relies on) and
run-to-run determinism.  Dot products are accumulated in float64."""
import pytest
import torch

pytestmark = pytest.mark.gpu


def _dot(a, b):
    return float((a.double() * b.double()).sum())


FULL_SHAPES = [
    (8, 6, (512, 512), 10),      # config 2 geometry
    (8, 6, (512, 512), 3),
    (2, 3, (1024, 1024), 7),     # config 3 geometry
    (2, 3, (128, 128, 128), 10),  # config 4 geometry
    (1, 2, (128, 128, 128), 4),
]


@pytest.mark.parametrize("B,C,sp,d", FULL_SHAPES, ids=lambda v: str(v).replace(" ", ""))
def test_adjoint_identities_at_full_size(cuda_device, B, C, sp, d):
    """<A f, g> == <f, A^T g> (test_conv2d.py:218-260 of the reference, at full size) and
    <A_k f, g> == <k, grad_k> (test_conv2d.py:263-311), for the linear ops."""
    from msd_pytorch_b200 import _lib
    from msd_pytorch_b200 import msd_custom_convolutions as cc

    dev = cuda_device
    gen = torch.Generator(device=dev).manual_seed(5)
    nd = len(sp)
    f = torch.randn(B, C, *sp, device=dev, generator=gen)
    g = torch.randn(B, 1, *sp, device=dev, generator=gen)
    k = torch.randn(1, C, *([3] * nd), device=dev, generator=gen)
    zero_bias = torch.zeros(1, device=dev)
    before = _lib.launch_counts()
    Af = torch.empty_like(g)
    cc.conv_forward(f, k, zero_bias, Af, d)
    ATg = torch.zeros_like(f)
    cc.conv_backward_x(g, k, ATg, d)
    gk = torch.zeros_like(k)
    cc.conv_backward_k(g, f, gk, d)
    gb = torch.zeros(1, device=dev)
    cc.conv_backward_bias(g, gb)
    assert _lib.device_status(dev) == 0
    assert _lib.launch_counts()[1] - before[1] >= 3, "the tuned kernels must be the ones under test"
    lhs = _dot(Af, g)
    scale = (float(Af.double().pow(2).sum()) * float(g.double().pow(2).sum())) ** 0.5
    assert abs(lhs - _dot(f, ATg)) <= 1e-5 * scale, "backward_x is not the adjoint of forward"
    assert abs(lhs - _dot(k, gk)) <= 1e-5 * scale, "backward_k is not the derivative in the kernel"
    assert abs(float(gb) - float(g.double().sum())) <= 1e-5 * float(g.double().abs().sum())


def test_gradients_are_additive_over_the_batch(cuda_device):
    """grad(batch) == sum of grad(halves): the identity behind the data-parallel all-reduce."""
    from msd_pytorch_b200.msd_block import msd_block

    dev = cuda_device
    torch.manual_seed(9)
    depth, sp = 12, (256, 384)
    dil = [1 + (i % 10) for i in range(depth)]
    ws = [(torch.randn(1, 1 + i, 3, 3, device=dev) * (2.0 / (9 * (1 + i))) ** 0.5).requires_grad_(True) for i in range(depth)]
    bias = (0.05 * torch.randn(depth, device=dev)).requires_grad_(True)
    x = torch.randn(4, 1, *sp, device=dev)
    go = torch.randn(4, 1 + depth, *sp, device=dev)

    def grads(sl):
        for p in ws + [bias]:
            p.grad = None
        msd_block(x[sl], dil, bias, *ws).backward(go[sl])
        return [p.grad.clone() for p in ws + [bias]]

    full = grads(slice(0, 4))
    a, b = grads(slice(0, 2)), grads(slice(2, 4))
    for gf, ga, gb_ in zip(full, a, b):
        ref = (ga.double() + gb_.double())
        err = (gf.double() - ref).abs().max()
        assert err <= 1e-4 * (ref.abs().max() + 1e-12), "batch additivity violated"
    again = grads(slice(0, 4))
    assert all(torch.equal(p, q) for p, q in zip(full, again)), "gradients are not run-to-run deterministic"


def test_block_forward_is_idempotent_on_its_buffer(cuda_device):
    """Re-running the forward over the same buffer reproduces every channel bit for bit
    (each layer only reads channels below the one it writes)."""
    from msd_pytorch_b200.msd_block import block_forward_

    dev = cuda_device
    torch.manual_seed(10)
    depth, sp = 20, (64, 64, 128)
    dil = [1 + (i % 10) for i in range(depth)]
    ws = [torch.randn(1, 1 + i, 3, 3, 3, device=dev) * (2.0 / (27 * (1 + i))) ** 0.5 for i in range(depth)]
    bias = 0.05 * torch.randn(depth, device=dev)
    res = torch.empty(1, 1 + depth, *sp, device=dev)
    res[:, :1] = torch.randn(1, 1, *sp, device=dev)
    block_forward_(res, 1, dil, bias, ws)
    first = res.clone()
    block_forward_(res, 1, dil, bias, ws)
    torch.cuda.synchronize()
    assert torch.equal(first, res)
    assert float(res[:, 1:].min()) >= 0.0  # ReLU outputs
