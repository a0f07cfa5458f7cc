"""fwd+bwd of ONE large 3D volume decomposed into z-slabs over the ranks (benchmark config
'c5': depth 80, 512^3, MSE), used by ``bench.py --config c5``.

Per step and rank: slab forward of all layers with a per-layer halo exchange, final 1x1
layer + MSE on the owned planes (two matrix-vector products, no copy of the channel
buffer), slab backward with a per-layer exchange of the gradient channel's halo, one sum of
the weight/bias gradients over the ranks.
"""
import json
import os
import time

import torch
import torch.distributed as dist

from . import _lib
from .distributed import SlabBlock, SlabPlan, TorchRanks, VirtualRanks, slab_backward, slab_forward


def algorithmic_bytes(depth, voxels):
    s1 = depth * (depth + 1) // 2
    return 4 * voxels * (s1 + depth), 4 * voxels * (3 * s1 + 2 * depth)


class SlabStep:
    def __init__(self, cfg, rank, world, device, size=None):
        Z, Y, X = cfg["spatial"] if size is None else (size, size, size)
        self.Z, self.Y, self.X = Z, Y, X
        self.depth = cfg["depth"]
        self.dil = [1 + (i % 10) for i in range(self.depth)]
        self.rank, self.world, self.device = rank, world, device
        self.plan = SlabPlan(Z, world, 10 if world > 1 else 0)
        self.comm = TorchRanks() if world > 1 else VirtualRanks(1)
        self.block = SlabBlock(self.plan, rank, 1, self.depth, (Y, X), device)
        loc = self.block.loc
        g = torch.Generator(device="cpu").manual_seed(4242)
        taps = 27
        self.ws = [(torch.randn(1, 1 + i, 3, 3, 3, generator=g) * (2.0 / (taps * (1 + i))) ** 0.5).to(device) for i in range(self.depth)]
        self.bias = torch.zeros(self.depth, device=device)
        self.fw = (torch.randn(1, 1 + self.depth, generator=g) / (1 + self.depth) ** 0.5).to(device)
        self.fb = (0.1 * torch.randn(1, generator=g)).to(device)
        # owned planes of input and target, U(0,1), seeded by global plane index range
        gd = torch.Generator(device=device).manual_seed(1000 + rank)
        zo = loc["g1"] - loc["g0"]
        self.x = torch.rand(1, zo, Y, X, device=device, generator=gd)
        self.t = torch.rand(zo * Y * X, device=device, generator=gd)
        self.block.gradients = torch.empty_like(self.block.result)
        self.vox_rank = zo * Y * X
        self.vox_total = Z * Y * X

    def forward(self):
        b = self.block
        b.set_input(self.x)
        slab_forward(self.comm, self.plan, {self.rank: b}, self.ws, self.bias, self.dil)

    def head(self):
        """Final 1x1 layer + MSE on the owned planes; fills the gradient buffer's owned planes."""
        b = self.block
        C = 1 + self.depth
        r2 = b.result[0, :, b.owned].reshape(C, -1)          # strided [C, Vo] view, no copy
        out = torch.matmul(self.fw, r2).view(-1) + self.fb
        diff = out - self.t
        loss = (diff * diff).sum() / self.vox_total
        gout = diff * (2.0 / self.vox_total)
        g2 = b.gradients[0, :, b.owned].reshape(C, -1)
        torch.mul(self.fw.view(C, 1), gout.view(1, -1), out=g2)
        self.gfw = torch.matmul(r2, gout)
        self.gfb = gout.sum()
        return loss

    def backward(self):
        b = self.block
        gws, gbs = slab_backward(self.comm, self.plan, {self.rank: b}, self.ws, self.dil)
        return gws[self.rank], gbs[self.rank]

    def step(self):
        self.forward()
        loss = self.head()
        gw, gb = self.backward()
        if self.world > 1:
            tail = torch.cat([self.gfw.reshape(-1), self.gfb.reshape(1), loss.reshape(1)])
            dist.all_reduce(tail)
            loss = tail[-1]
        return loss


def main(args, cfg, rank, world, local, peak=(6650.0, "fallback")):
    if not torch.cuda.is_available():
        raise SystemExit("bench.py --config c5 needs CUDA devices")
    device = torch.device("cuda", local)
    torch.cuda.set_device(device)
    if world > 1:
        os.environ.setdefault("MASTER_ADDR", "127.0.0.1")
        dist.init_process_group("nccl", device_id=device)
    size = int(os.environ.get("MSD_SLAB_SIZE", "0")) or None
    st = SlabStep(cfg, rank, world, device, size)

    def sync():
        torch.cuda.synchronize()
        if world > 1:
            dist.barrier()
            torch.cuda.synchronize()

    def timed(fn, steps, warmup):
        for _ in range(warmup):
            fn()
        sync()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        l0 = _lib.launch_counts()
        e0.record()
        for _ in range(steps):
            fn()
        e1.record()
        torch.cuda.synchronize()
        ms = e0.elapsed_time(e1) / steps
        l1 = _lib.launch_counts()
        if world > 1:
            tt = torch.tensor([ms], device=device)
            dist.barrier()
            dist.all_reduce(tt, op=dist.ReduceOp.MAX)
            ms = float(tt.item())
        return ms, ((l1[0] - l0[0]) // max(steps, 1))

    steps, warmup = args.steps, max(args.warmup, 3)
    ms_step, launches = timed(st.step, steps, warmup)
    ms_fwd, _ = timed(st.forward, max(1, steps // 2), 1)
    st.head()
    ms_bwd, _ = timed(st.backward, max(1, steps // 2), 1)
    # end to end: input and target start in pinned host memory, the loss value comes back
    xh, th = st.x.cpu().pin_memory(), st.t.cpu().pin_memory()

    def e2e():
        st.x.copy_(xh, non_blocking=True)
        st.t.copy_(th, non_blocking=True)
        return float(st.step().item())

    ms_e2e, _ = timed(e2e, 2, 1)
    status = _lib.device_status(device)
    if rank == 0:
        peak, peak_src = peak
        a_fwd, a_bwd = algorithmic_bytes(st.depth, st.vox_rank)
        gbs_bwd = a_bwd / (ms_bwd * 1e-3) / 1e9
        gbs_fwd = a_fwd / (ms_fwd * 1e-3) / 1e9
        res = {
            "metric": "fwd+bwd voxels/s", "value": st.vox_total / (ms_step * 1e-3), "unit": "voxels/s", "n_gpus": world, "steps": steps,
            "warmup": warmup, "ms_per_step": ms_step, "higher_is_better": True, "scaling": "strong", "vs_baseline": None, "dtype": "f32",
            "data": "synthetic",
            "config": {"workload": "c5: MSD 3D depth %d, one 1x%dx%dx%d volume, MSE, fwd+bwd, z-slabs of %d planes + 10-plane halos per rank; "
                                   "inputs larger than L2" % (st.depth, st.Z, st.Y, st.X, st.Z // world),
                       "parallelism": "zslab%d" % world, "l2_policy": "inputs larger than L2"},
            "e2e": {"value": st.vox_total / (ms_e2e * 1e-3), "unit": "voxels/s", "ms_per_step": ms_e2e,
                    "h2d_bytes_per_step": int(2 * st.vox_rank * 4), "d2h_bytes_per_step": 4},
            "gpu_launches": launches, "device_status": status,
            "roofline": {"kernel": "fused_backward3d_split_kernel (per rank; halo exchanges inside the timed span)", "bound": "hbm",
                         "achieved": gbs_bwd, "peak": peak, "peak_source": peak_src, "unit": "GB/s", "frac": gbs_bwd / peak,
                         "algorithmic_bytes_per_launch": a_bwd / st.depth, "avg_launch_ms": ms_bwd / st.depth, "launches": st.depth,
                         "traffic": None},
            "roofline_forward": {"kernel": "forward2d_kernel<NT=3> + zgather_kernel", "bound": "hbm", "achieved": gbs_fwd, "peak": peak,
                                 "unit": "GB/s", "frac": gbs_fwd / peak},
            "block_only": {"fwd_ms": ms_fwd, "bwd_ms": ms_bwd},
        }
        print(json.dumps(res), flush=True)
    if world > 1:
        dist.destroy_process_group()
