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
    # the gradients now ARE slices of the flat buffer: accumulating in place and reducing again needs no gather
    for k, p in enumerate(params):
        assert p.grad.data_ptr() == bucket.views[k].data_ptr()
        p.grad.fill_(float(rank + 1))
    bucket.allreduce_(average=False)
    for p in params:
        assert torch.allclose(p.grad, torch.full_like(p, float(sum(range(1, world + 1)))))
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


def _partial_sum_case(rank, world, out_dir):
    """The forward's hand-over of z-tap partial sums and the backward's of gradient planes,
    started asynchronously like the slab schedule does, on CPU tensors."""
    from msd_pytorch_b200.distributed import SlabPlan, TorchRanks, halo_transfers, partial_sum_transfers

    Z, H, d = 24, 5, 3
    plan = SlabPlan(Z, world, H)
    loc = plan.local(rank)
    comm = TorchRanks()
    # u[tap][z] = 100 * tap + global plane index on the owned planes, -1 elsewhere
    u = torch.full((3, loc["planes"], 2, 2), -1.0)
    for tap in range(3):
        for z in range(loc["g0"], loc["g1"]):
            u[tap, loc["z_begin"] + z - loc["g0"]] = 100.0 * tap + z
    work = comm.start({rank: [(k, peer, tap, u[tap, a:b]) for k, peer, tap, a, b in partial_sum_transfers(plan, rank, d)]})
    work.wait()
    zb, ze = loc["z_begin"], loc["z_end"]
    if rank > 0:       # u_0 of the d planes below my first owned one
        for j in range(d):
            assert torch.all(u[0, zb - d + j] == float(loc["g0"] - d + j))
        assert torch.all(u[2, zb - 1] == -1.0) and torch.all(u[1, zb - 1] == -1.0)
    if rank < world - 1:  # u_2 of the d planes above my last owned one
        for j in range(d):
            assert torch.all(u[2, ze + j] == 200.0 + loc["g1"] + j)
        assert torch.all(u[0, ze] == -1.0)
    # gradient channel: only d planes per face travel
    g = torch.full((loc["planes"], 2, 2), -1.0)
    g[zb:ze] = torch.arange(loc["g0"], loc["g1"], dtype=torch.float32).view(-1, 1, 1).expand(-1, 2, 2)
    comm.start({rank: [(k, peer, 0, g[a:b]) for k, peer, a, b in halo_transfers(plan, rank, d)]}).wait()
    first = loc["g0"] - loc["lo"]
    for k in range(loc["planes"]):
        inside = (zb - (d if rank > 0 else 0)) <= k < (ze + (d if rank < world - 1 else 0))
        assert torch.all(g[k] == (float(first + k) if inside else -1.0)), (rank, k)


def test_partial_sum_and_gradient_handover_gloo(tmp_path):
    _run("_partial_sum_case", 3, tmp_path)


def test_boundary_windows_and_partial_sum_schedule():
    from msd_pytorch_b200.distributed import SlabPlan, VirtualRanks, boundary_windows, partial_sum_transfers

    plan = SlabPlan(60, 3, 10)
    assert boundary_windows(plan, 0, 4) == ([(16, 20)], [(0, 16)])
    assert boundary_windows(plan, 1, 4) == ([(10, 14), (26, 30)], [(14, 26)])
    assert boundary_windows(plan, 2, 10) == ([(10, 20)], [(20, 30)])
    assert boundary_windows(SlabPlan(60, 1, 0), 0, 7) == ([], [(0, 60)])
    assert boundary_windows(SlabPlan(36, 3, 10), 1, 6) == ([(10, 22)], [])   # 12 planes cannot be split 6 + interior + 6
    assert partial_sum_transfers(plan, 1, 3) == [("send", 0, 2, 10, 13), ("recv", 0, 0, 7, 10), ("send", 2, 0, 27, 30), ("recv", 2, 2, 30, 33)]
    with pytest.raises(ValueError):
        partial_sum_transfers(plan, 1, 11)
    # every send has exactly one matching receive of the same size
    bufs = {r: torch.zeros(3, plan.local(r)["planes"]) for r in range(3)}
    for r in range(3):
        loc = plan.local(r)
        bufs[r][:, loc["z_begin"]:loc["z_end"]] = torch.arange(loc["g0"], loc["g1"], dtype=torch.float32) + 1000.0 * torch.arange(3).view(3, 1)
    VirtualRanks(3).start({r: [(k, p, tap, bufs[r][tap, a:b]) for k, p, tap, a, b in partial_sum_transfers(plan, r, 3)] for r in range(3)})
    assert bufs[1][0, 7:10].tolist() == [17.0, 18.0, 19.0] and bufs[1][2, 30:33].tolist() == [2040.0, 2041.0, 2042.0]
    assert bufs[0][2, 20:23].tolist() == [2020.0, 2021.0, 2022.0] and bufs[2][0, 7:10].tolist() == [37.0, 38.0, 39.0]


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
