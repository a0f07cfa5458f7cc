"""CPU tests of the multi-GPU host logic with world_size-2 gloo process groups: the flat
gradient bucket of the batch data-parallel path and the halo-exchange schedule of the
z-slab path (on CPU tensors; the schedule is device-agnostic)."""
import os
import socket

import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp


def _free_port():
    s = socket.socket()
    s.bind(("127.0.0.1", 0))
    p = s.getsockname()[1]
    s.close()
    return p


def _worker(rank, world, port, fn_name, out_dir):
    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        globals()[fn_name](rank, world, out_dir)
    finally:
        dist.destroy_process_group()


def _run(fn_name, world, tmp_path):
    mp.spawn(_worker, args=(world, _free_port(), fn_name, str(tmp_path)), nprocs=world, join=True)


def _bucket_case(rank, world, out_dir):
    from msd_pytorch_b200.distributed import GradientBucket, split_batch

    torch.manual_seed(0)
    params = [torch.nn.Parameter(torch.zeros(3, 4)), torch.nn.Parameter(torch.zeros(7)), torch.nn.Parameter(torch.zeros(1, 2, 3, 3))]
    frozen = torch.nn.Parameter(torch.zeros(2), requires_grad=False)
    for k, p in enumerate(params):
        p.grad = torch.full_like(p, float(rank + 1) * (k + 1))
    bucket = GradientBucket(params + [frozen])
    assert bucket.numel == 12 + 7 + 18
    bucket.allreduce_()
    mean = sum(range(1, world + 1)) / world
    for k, p in enumerate(params):
        assert torch.allclose(p.grad, torch.full_like(p, mean * (k + 1)))
    assert split_batch(16, rank, world) == (rank * 16 // world, (rank + 1) * 16 // world)
    with pytest.raises(ValueError):
        split_batch(3, rank, 2)


def _halo_case(rank, world, out_dir):
    from msd_pytorch_b200.distributed import SlabPlan, TorchRanks

    Z, H = 20, 3
    plan = SlabPlan(Z, world, H)
    loc = plan.local(rank)
    vol = torch.full((loc["planes"], 2, 4), -1.0)
    for z in range(loc["g0"], loc["g1"]):
        vol[loc["z_begin"] + z - loc["g0"]] = float(z)           # owned planes hold their global index
    TorchRanks().exchange(plan, {rank: vol})
    first_global = loc["g0"] - loc["lo"]
    for k in range(loc["planes"]):
        assert torch.all(vol[k] == float(first_global + k)), (rank, k, vol[k, 0, 0].item())


def test_gradient_bucket_allreduce_gloo(tmp_path):
    _run("_bucket_case", 2, tmp_path)


def test_halo_exchange_gloo(tmp_path):
    _run("_halo_case", 2, tmp_path)


def test_slab_plan_and_virtual_exchange():
    from msd_pytorch_b200.distributed import SlabPlan, VirtualRanks, halo_transfers

    plan = SlabPlan(50, 3, 5)
    assert plan.bounds == [(0, 16), (16, 33), (33, 50)]
    assert plan.local(0) == dict(g0=0, g1=16, lo=0, hi=5, planes=21, z_begin=0, z_end=16)
    assert plan.local(1)["planes"] == 17 + 10 and plan.local(2)["hi"] == 0
    assert halo_transfers(plan, 0) == [("send", 1, 11, 16), ("recv", 1, 16, 21)]
    with pytest.raises(ValueError):
        SlabPlan(16, 4, 10)
    vols = {}
    for r in range(3):
        loc = plan.local(r)
        v = torch.full((loc["planes"], 1, 1), -1.0)
        v[loc["z_begin"]:loc["z_end"], 0, 0] = torch.arange(loc["g0"], loc["g1"], dtype=torch.float32)
        vols[r] = v
    VirtualRanks(3).exchange(plan, vols)
    for r in range(3):
        loc = plan.local(r)
        want = torch.arange(loc["g0"] - loc["lo"], loc["g1"] + loc["hi"], dtype=torch.float32)
        assert torch.equal(vols[r][:, 0, 0], want)
