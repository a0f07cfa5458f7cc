#!/usr/bin/env python
"""Benchmark of the MSD hot path: forward + backward voxels/s, HBM roofline fraction,
end-to-end figure through the public model API, and the CPU baseline.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--config c2] [--impl reference]

Prints ONE JSON line (rank 0).  The headline (`value`, `e2e`, `roofline`) is measured on
`--config` (default c2).  With the default config two compact records follow at the END of the
line: `c4` (depth-50 3D on one GPU; only when N = 1) and `c5_zslab` (the 512^3 volume cut into
z-slabs over the N ranks, strong scaling).  Workloads (synthetic, seeded; dilations 1..10
cycling, c_in = width = 1, float32, weights ~ N(0, 2/(taps*n_in)), zero bias, seeded non-zero
final 1x1 layer):
  c1  2D regression  depth 30,  batch 1 of 256x256,      MSE, fwd+bwd+Adam
  c2  2D regression  depth 100, batch 8 of 512x512,      MSE, fwd+bwd            (default)
  c3  2D segmentation depth 100, batch 16 of 1024x1024, 4 classes, NLL, fwd+bwd
  c4  3D regression  depth 50,  batch 2 of 128^3,        MSE, fwd+bwd
  c5  3D regression  depth 80,  one 512^3 volume,        MSE, fwd+bwd (z-slabs over the ranks)
With N > 1 ranks (torchrun) c1-c4 run batch data-parallel, the per-rank batch fixed (weak
scaling) with one flat NCCL all-reduce of the parameter gradients per step; c3 can also be
run with its global batch of 16 split over the ranks (--strong).

`--impl reference` times the reference path on the host cores instead: the reference has
no CPU implementation, so this is its PyTorch-equivalent composition (edge-inclusive
reflection gather + unpadded dilated convolution + ReLU, dense block in place) from
oracle/msd_oracle.py, on a bounded sample of the same workload (one image / a cropped
volume per step at full depth), after a ladder of sizes that shows how the per-voxel cost
depends on the sample size.

`--one-layer c4:50:2` runs a few launches of ONE layer's forward and fused backward on the
named configuration's shape (here: 50 input channels, dilation 2) and prints their times;
it is the command the ncu summaries under profiles/ are captured from.

`--layer-table c2` times single layers of the configuration's shape over a grid of channel
counts and dilations, each as a CUDA graph of ten launches (device time only, no host gaps),
and prints one JSON line per dilation: what a layer costs per input channel and per launch.
"""
import argparse
import json
import os
import statistics
import subprocess
import sys
import threading
import time

ROOT = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, ROOT)

import torch  # noqa: E402

CONFIGS = {
    # name: ndim, depth, batch, spatial, c_out, loss, adam
    "c1": dict(ndim=2, depth=30, batch=1, spatial=(256, 256), c_out=1, loss="mse", adam=True, dist="normal"),
    "c2": dict(ndim=2, depth=100, batch=8, spatial=(512, 512), c_out=1, loss="mse", adam=False, dist="uniform"),
    "c3": dict(ndim=2, depth=100, batch=16, spatial=(1024, 1024), c_out=4, loss="nll", adam=False, dist="normal"),
    "c4": dict(ndim=3, depth=50, batch=2, spatial=(128, 128, 128), c_out=1, loss="mse", adam=False, dist="normal"),
    "c5": dict(ndim=3, depth=80, batch=1, spatial=(512, 512, 512), c_out=1, loss="mse", adam=False, dist="uniform"),
}


def algorithmic_bytes(depth, voxels):
    """Forward layer i reads n_i = 1+i channels and writes 1; the fused backward reads n_i
    activation channels, reads and writes n_i gradient channels, reads the output and its
    gradient: 4V(S1 + D) and 4V(3 S1 + 2 D) bytes, S1 = D(D+1)/2."""
    s1 = depth * (depth + 1) // 2
    return 4 * voxels * (s1 + depth), 4 * voxels * (3 * s1 + 2 * depth)


# DRAM traffic per launch measured by ncu (dram__bytes_read.sum + dram__bytes_write.sum) divided
# by the algorithmic bytes of the captured launch (`--one-layer` captures summarised in profiles/):
# 2D backward 1226.2 / 1275.1 MB and 2D forward 430.1 / 427.8 MB (c2:50:10); 3D backward
# 2495.0 / 2550.1 MB (c4:50:2) and 3D forward 509.8 / 436.2 MB (c4:25:4, both forward kernels).
# Traffic grows with the channel count like the algorithmic bytes do, so the ratio is applied to
# the average launch.
NCU_TRAFFIC_RATIO = {("bwd", 2): 1226.2 / 1275.1, ("fwd", 2): 430.1 / 427.8, ("bwd", 3): 2495.0 / 2550.1, ("fwd", 3): 509.8 / 436.2}


def measured_peak():
    p = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.exists(p):
        try:
            return float(json.load(open(p))["hbm_gbs"]), "measured"
        except Exception:
            pass
    return 6650.0, "fallback"


def make_data(cfg, batch, seed, generator_device="cpu"):
    g = torch.Generator().manual_seed(seed)
    shape = (batch, 1) + tuple(cfg["spatial"])
    rnd = torch.rand if cfg["dist"] == "uniform" else torch.randn
    x = rnd(shape, generator=g)
    if cfg["loss"] == "nll":
        y = torch.randint(0, cfg["c_out"], shape, generator=g)
    else:
        y = rnd(shape, generator=g)
    return x, y


def make_weights(cfg, seed):
    g = torch.Generator().manual_seed(seed)
    nd, depth = cfg["ndim"], cfg["depth"]
    taps = 3 ** nd
    ws = [torch.randn(1, 1 + i, *([3] * nd), generator=g) * (2.0 / (taps * (1 + i))) ** 0.5 for i in range(depth)]
    fw = torch.randn(cfg["c_out"], 1 + depth, 1, generator=g) / (1 + depth) ** 0.5
    fb = 0.1 * torch.randn(cfg["c_out"], generator=g)
    return ws, fw, fb


def voxels_of(batch, spatial):
    v = batch
    for s in spatial:
        v *= s
    return v


def describe_config(name, cfg, world, strong):
    """The `config` object of the JSON line; identical for both arms (`--impl`)."""
    batch = cfg["batch"] // world if strong else cfg["batch"]
    if name == "c5":
        workload = ("c5: MSD 3D depth %d, one 1x%s volume, mse loss, fwd+bwd, z-slabs over the ranks (partial-sum / gradient "
                    "hand-over of `dilation` planes per layer and face); inputs larger than L2" % (cfg["depth"], "x".join(map(str, cfg["spatial"]))))
        return {"workload": workload, "parallelism": "zslab%d" % world if world > 1 else "single", "l2_policy": "inputs larger than L2"}
    workload = "%s: MSD %dD depth %d, batch %d/GPU of 1x%s, c_out %d, %s loss, fwd+bwd%s; block + final 1x1 layer + loss; " \
               "inputs larger than L2 (%.2f GB channel buffer)" % (
                   name, cfg["ndim"], cfg["depth"], batch, "x".join(map(str, cfg["spatial"])), cfg["c_out"], cfg["loss"],
                   "+Adam" if cfg["adam"] else "", 4 * voxels_of(batch, cfg["spatial"]) * (1 + cfg["depth"]) / 1e9)
    return {"workload": workload, "parallelism": "dp%d" % world if world > 1 else "single", "l2_policy": "inputs larger than L2"}


class ClockSampler:
    """Samples nvidia-smi clocks and throttle reasons while the timed region runs."""

    Q = ("clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.hw_slowdown,clocks_event_reasons.hw_thermal_slowdown,"
         "clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap")

    def __init__(self, index):
        self.index = index
        self.rows = []
        self.proc = None

    def start(self):
        try:
            self.proc = subprocess.Popen(["nvidia-smi", "-i", str(self.index), "--query-gpu=" + self.Q, "--format=csv,noheader,nounits", "-lms", "100"],
                                         stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True)
            self.thread = threading.Thread(target=self._read, daemon=True)
            self.thread.start()
        except Exception:
            self.proc = None

    def _read(self):
        for line in self.proc.stdout:
            self.rows.append((time.time(), line.strip()))

    def stop(self, t0, t1):
        if not self.proc:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["nvidia-smi unavailable"]}
        time.sleep(0.15)
        self.proc.terminate()
        try:
            self.proc.wait(timeout=2)
        except Exception:
            pass
        sm, mx, reasons, power = [], [], set(), []
        names = ["hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"]
        rows = [r for (t, r) in self.rows if t0 - 0.05 <= t <= t1 + 0.15] or [r for (_, r) in self.rows]
        for r in rows:
            f = [x.strip() for x in r.split(",")]
            try:
                sm.append(float(f[0]))
                mx.append(float(f[1]))
                power.append(float(f[2]))
            except Exception:
                continue
            for n, v in zip(names, f[3:7]):
                if v.lower().startswith("active"):
                    reasons.add(n)
        return {"sm_mhz": statistics.median(sm) if sm else None, "sm_max_mhz": max(mx) if mx else None,
                "power_w_max": max(power) if power else None, "samples": len(sm), "reasons": sorted(reasons)}


class Timer:
    """Times `steps` calls of a function with CUDA events on the current stream, after
    `warmup` untimed calls, bracketed by a barrier and a device synchronisation; over several
    ranks the result is the maximum."""

    def __init__(self, device, world):
        self.device, self.world = device, world

    def sync(self):
        torch.cuda.synchronize()
        if self.world > 1:
            import torch.distributed as dist

            dist.barrier()
            torch.cuda.synchronize()

    def __call__(self, fn, steps, warmup, sample_clocks=False):
        from msd_pytorch_b200 import _lib

        for _ in range(warmup):
            fn()
        self.sync()
        sampler = ClockSampler(self.device.index) if sample_clocks else None
        if sampler:
            sampler.start()
            time.sleep(0.25)
        l0 = _lib.launch_counts()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        t0 = time.time()
        e0.record()
        for _ in range(steps):
            fn()
        e1.record()
        torch.cuda.synchronize()
        t1 = time.time()
        ms = e0.elapsed_time(e1)
        l1 = _lib.launch_counts()
        if self.world > 1:
            import torch.distributed as dist

            dist.barrier()
            torch.cuda.synchronize()
            tt = torch.tensor([ms], device=self.device)
            dist.all_reduce(tt, op=dist.ReduceOp.MAX)
            ms = float(tt.item())
        clocks = sampler.stop(t0, t1) if sampler else None
        return ms / steps, (l1[0] - l0[0], l1[1] - l0[1]), clocks


def build_model(cfg, device):
    """The public model API with the benchmark's seeded weights."""
    from msd_pytorch_b200 import MSDRegressionModel, MSDSegmentationModel

    if cfg["loss"] == "nll":
        model = MSDSegmentationModel(1, cfg["c_out"], cfg["depth"], 1, ndim=cfg["ndim"])
    else:
        model = MSDRegressionModel(1, cfg["c_out"], cfg["depth"], 1, loss="L2", ndim=cfg["ndim"])
    ws, fw, fb = make_weights(cfg, 4242)
    with torch.no_grad():
        for i, w in enumerate(ws):
            getattr(model.msd.msd_block, "weight%d" % i).copy_(w)
        model.msd.msd_block.bias.zero_()
        model.msd.final_layer.linear.weight.copy_(fw)
        model.msd.final_layer.linear.bias.copy_(fb)
    return model


def run_ours(args, name, cfg, rank, world, device, steps, warmup, full=True):
    """fwd+bwd of one configuration (batch data-parallel over the ranks).  `full` adds the
    end-to-end figure and the complete roofline objects; otherwise a compact record."""
    from msd_pytorch_b200 import _lib, autotune
    from msd_pytorch_b200.distributed import GradientBucket
    from msd_pytorch_b200.msd_block import block_backward_, block_forward_

    batch = cfg["batch"]
    if args.strong:
        assert batch % world == 0
        batch //= world
    tuned = None
    if not args.no_autotune:
        # per-shape launch autotuning (untimed set-up; winners are cached on disk)
        tuned = autotune.tune(batch, cfg["spatial"], max(2, cfg["depth"] // 2), range(1, 11), device=device, reps=3)
    model = build_model(cfg, device)
    bucket = GradientBucket(list(model.msd.parameters()))
    params = bucket.params
    x, y = make_data(cfg, batch, 1000 + rank)
    xd, yd = x.to(device), (y.squeeze(1) if cfg["loss"] == "nll" else y).to(device)
    xp, yp = x.pin_memory(), y.pin_memory()
    voxels_rank = voxels_of(batch, cfg["spatial"])
    timed = Timer(device, world)

    def step_device():
        for p in params:
            p.grad = None
        out = model.net(xd)
        loss = model.criterion(out, yd)
        loss.backward()
        bucket.allreduce_()
        if cfg["adam"]:
            model.optimizer.step()
        return loss

    def step_e2e():
        # the call a user makes: host tensors in, loss value out (H2D + D2H inside)
        val = model.forward(xp, yp)
        model.optimizer.zero_grad(set_to_none=True)
        model.loss.backward()
        bucket.allreduce_()
        if cfg["adam"]:
            model.optimizer.step()
        return val

    ms_step, launches, clocks = timed(step_device, steps, warmup, sample_clocks=True)
    ms_e2e = None
    if full:
        ms_e2e, _, _ = timed(step_e2e, max(2, steps // 2), max(3, warmup // 2))
    status = _lib.device_status(device)

    # ---- the block alone (the hot path proper), forward and backward timed separately ----
    depth, nd = cfg["depth"], cfg["ndim"]
    blk = model.msd.msd_block
    ws = [getattr(blk, "weight%d" % i).detach() for i in range(depth)]
    bias = blk.bias.detach()
    dil = model.msd.dilations
    res = torch.empty((batch, 1 + depth) + tuple(cfg["spatial"]), device=device)
    res[:, :1] = xd
    gbuf = torch.empty_like(res)
    gsrc = torch.randn_like(res)
    gws = [torch.zeros_like(w) for w in ws]
    gb = torch.zeros_like(bias)

    def fwd_only():
        block_forward_(res, 1, dil, bias, ws)

    def bwd_only():
        block_backward_(res, gbuf, 1, dil, ws, gws, gb)

    fwd_only()
    ms_fwd, lf, _ = timed(fwd_only, steps, warmup)
    gbuf.copy_(gsrc)
    ms_bwd, lb, _ = timed(bwd_only, steps, warmup)
    h2d = int(xp.numel() * xp.element_size() + yp.numel() * yp.element_size())
    del gbuf, gsrc, res, model, bucket, params, xd, yd, blk, ws, bias, gws, gb
    torch.cuda.empty_cache()
    a_fwd, a_bwd = algorithmic_bytes(depth, voxels_rank)
    peak, peak_src = measured_peak()
    gbs_fwd = a_fwd / (ms_fwd * 1e-3) / 1e9
    gbs_bwd = a_bwd / (ms_bwd * 1e-3) / 1e9
    if rank != 0:
        return None
    total_vox = voxels_rank * world
    if not full:
        return {"workload": describe_config(name, cfg, world, args.strong)["workload"], "ms_per_step": round(ms_step, 3),
                "voxels_per_s": total_vox / (ms_step * 1e-3), "steps": steps, "warmup": warmup,
                "fwd_ms": round(ms_fwd, 3), "bwd_ms": round(ms_bwd, 3),
                "roofline_frac_fwd": round(gbs_fwd / peak, 4), "roofline_frac_bwd": round(gbs_bwd / peak, 4),
                "roofline_frac_step": round((a_fwd + a_bwd) / (ms_step * 1e-3) / 1e9 / peak, 4),
                "gpu_launches": launches[0], "device_status": status, "clocks": clocks}
    return {
        "metric": "fwd+bwd voxels/s",
        "value": total_vox / (ms_step * 1e-3),
        "unit": "voxels/s",
        "n_gpus": world,
        "steps": steps,
        "warmup": warmup,
        "ms_per_step": ms_step,
        "higher_is_better": True,
        "scaling": "strong" if args.strong else "weak",
        "vs_baseline": None,
        "dtype": "f32",
        "data": "synthetic",
        "config": describe_config(name, cfg, world, args.strong),
        "launch_variants": {k: [v[d] for d in sorted(v)] for k, v in tuned.items()} if tuned else "library defaults",
        "e2e": {"value": total_vox / (ms_e2e * 1e-3), "unit": "voxels/s", "ms_per_step": ms_e2e,
                "h2d_bytes_per_step": h2d, "d2h_bytes_per_step": 4},
        "gpu_launches": launches[0],
        "gpu_launches_tuned_path": launches[1],
        "device_status": status,
        "clocks": clocks,
        "roofline": {
            "kernel": ("fused_backward_kernel" if nd == 2 else "fused_backward_split_kernel<3> (fused_backward_kernel<3> below 8 input channels)")
            + " (one launch per layer; the small second-pass reductions are inside the timed span)",
            "bound": "hbm", "achieved": gbs_bwd, "peak": peak, "peak_source": peak_src, "unit": "GB/s", "frac": gbs_bwd / peak,
            "frac_of_nominal_8TBs": gbs_bwd / 8000.0,
            "algorithmic_bytes_per_launch": a_bwd / depth, "avg_launch_ms": ms_bwd / depth, "launches": depth,
            "traffic": NCU_TRAFFIC_RATIO[("bwd", nd)] * a_bwd / depth,
            "traffic_source": "ncu capture of one mid-depth layer, scaled by algorithmic bytes",
        },
        "roofline_forward": {
            "kernel": "forward2d_kernel" if nd == 2 else "forward2d_kernel<NT=3> + zgather_kernel",
            "bound": "hbm", "achieved": gbs_fwd, "peak": peak, "unit": "GB/s", "frac": gbs_fwd / peak,
            "algorithmic_bytes_per_launch": a_fwd / depth, "avg_launch_ms": ms_fwd / depth, "launches": depth,
            "traffic": NCU_TRAFFIC_RATIO[("fwd", nd)] * a_fwd / depth,
        },
        "block_only": {"fwd_ms": ms_fwd, "bwd_ms": ms_bwd, "voxels_per_s": total_vox / ((ms_fwd + ms_bwd) * 1e-3),
                       "roofline_frac": (a_fwd + a_bwd) / ((ms_fwd + ms_bwd) * 1e-3) / 1e9 / peak},
    }


# --------------------------------------------------------------------------------------- #
# c5: ONE large 3D volume decomposed into z-slabs over the ranks                            #
# --------------------------------------------------------------------------------------- #
class NoTransfers:
    """Stands in for the communicator to time a rank's kernels without any hand-over."""

    def start(self, transfers):
        from msd_pytorch_b200.distributed import _Done

        return _Done()

    def allreduce_sum(self, tensors):
        pass


class SlabStep:
    """Per step and rank: slab forward of all layers (per-layer hand-over of z-tap partial
    sums), final 1x1 layer + MSE on the owned planes (two matrix-vector products, no copy of
    the channel buffer), slab backward (per-layer hand-over of the gradient channel's
    boundary planes), one sum of the weight/bias gradients over the ranks."""

    def __init__(self, cfg, rank, world, device, size=None):
        from msd_pytorch_b200.distributed import SlabBlock, SlabPlan, TorchRanks, VirtualRanks

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
        # owned planes of input and target, U(0,1), seeded per GLOBAL plane: the data (and so the
        # loss) are the same however many ranks share the volume
        zo = loc["g1"] - loc["g0"]
        self.x = torch.empty(1, zo, Y, X, device=device)
        self.t = torch.empty(zo, Y, X, device=device)
        gd = torch.Generator(device=device)
        for k in range(zo):
            gd.manual_seed(100000 + loc["g0"] + k)
            self.x[0, k].copy_(torch.rand(Y, X, device=device, generator=gd))
            self.t[k].copy_(torch.rand(Y, X, device=device, generator=gd))
        self.t = self.t.view(-1)
        self.block.gradients = torch.empty_like(self.block.result)
        self.vox_rank = zo * Y * X
        self.vox_total = Z * Y * X

    def forward(self, comm=None):
        from msd_pytorch_b200.distributed import slab_forward

        b = self.block
        b.set_input(self.x)
        slab_forward(comm or self.comm, self.plan, {self.rank: b}, self.ws, self.bias, self.dil)

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

    def backward(self, comm=None):
        from msd_pytorch_b200.distributed import slab_backward

        b = self.block
        gws, gbs = slab_backward(comm or self.comm, self.plan, {self.rank: b}, self.ws, self.dil)
        return gws[self.rank], gbs[self.rank]

    def transfers_only(self):
        """Every hand-over of one step, back to back, without the kernels between them."""
        from msd_pytorch_b200.distributed import halo_transfers, partial_sum_transfers

        b = self.block
        for d in self.dil:
            self.comm.start({self.rank: [(k, p, tap, b.u[tap, a:z]) for k, p, tap, a, z in partial_sum_transfers(self.plan, self.rank, d)]}).wait()
        for i in range(self.depth - 1, -1, -1):
            self.comm.start({self.rank: [(k, p, 0, b.gradients[0, 1 + i, a:z]) for k, p, a, z in halo_transfers(self.plan, self.rank, self.dil[i])]}).wait()

    def step(self, comm=None):
        import torch.distributed as dist

        self.forward(comm)
        loss = self.head()
        self.backward(comm)
        if self.world > 1 and comm is None:
            tail = torch.cat([self.gfw.reshape(-1), self.gfb.reshape(1), loss.reshape(1)])
            dist.all_reduce(tail)
            loss = tail[-1]
        return loss


def run_slab(args, cfg, rank, world, device, steps, warmup, full=True):
    from msd_pytorch_b200 import _lib, autotune

    size = int(os.environ.get("MSD_SLAB_SIZE", "0")) or None
    if not args.no_autotune:
        sp = cfg["spatial"] if size is None else (size, size, size)
        autotune.tune(1, (min(32, sp[0]), sp[1], sp[2]), 40, range(1, 11), device=device, reps=3)
    st = SlabStep(cfg, rank, world, device, size)
    timed = Timer(device, world)
    ms_step, launches, clocks = timed(st.step, steps, warmup, sample_clocks=True)
    loss_value = float(st.step().item())
    ms_fwd, _, _ = timed(st.forward, max(1, steps // 2), 1)
    st.head()
    ms_bwd, _, _ = timed(st.backward, max(1, steps // 2), 1)
    ms_alone = ms_quiet = None
    if world > 1:
        quiet = NoTransfers()
        ms_quiet, _, _ = timed(lambda: st.step(quiet), max(1, steps // 2), 1)   # the same kernels, nothing handed over
        ms_alone, _, _ = timed(st.transfers_only, max(1, steps // 2), 1)       # the hand-overs alone, serialised
    ms_e2e = None
    if full:
        # end to end: input and target start in pinned host memory, the loss value comes back
        xh, th = st.x.cpu().pin_memory(), st.t.cpu().pin_memory()

        def e2e():
            st.x.copy_(xh, non_blocking=True)
            st.t.copy_(th, non_blocking=True)
            return float(st.step().item())

        ms_e2e, _, _ = timed(e2e, 2, 1)
    status = _lib.device_status(device)
    vox_rank, vox_total, depth = st.vox_rank, st.vox_total, st.depth
    zs = (st.Z, st.Y, st.X)
    del st
    torch.cuda.empty_cache()
    if rank != 0:
        return None
    peak, peak_src = measured_peak()
    a_fwd, a_bwd = algorithmic_bytes(depth, vox_rank)
    gbs_bwd = a_bwd / (ms_bwd * 1e-3) / 1e9
    gbs_fwd = a_fwd / (ms_fwd * 1e-3) / 1e9
    exchange = None
    if world > 1:
        exchange = {"exposed_ms": round(ms_step - ms_quiet, 3), "step_without_transfers_ms": round(ms_quiet, 3),
                    "transfers_alone_ms": round(ms_alone, 3),
                    "what": "exposed = step - the same step with every hand-over skipped; transfers_alone = all hand-overs of a step back to back"}
    if not full:
        return {"workload": "c5: MSD 3D depth %d, one 1x%dx%dx%d volume, mse, fwd+bwd, z-slabs of %d planes per rank" % (depth, *zs, zs[0] // world),
                "scaling": "strong", "n_gpus": world, "ms_per_step": round(ms_step, 3), "voxels_per_s": vox_total / (ms_step * 1e-3),
                "steps": steps, "warmup": warmup, "fwd_ms": round(ms_fwd, 3), "bwd_ms": round(ms_bwd, 3), "exchange": exchange, "loss": loss_value,
                "roofline_frac_fwd": round(gbs_fwd / peak, 4), "roofline_frac_bwd": round(gbs_bwd / peak, 4),
                "roofline_frac_step": round((a_fwd + a_bwd) / (ms_step * 1e-3) / 1e9 / peak, 4),
                "gpu_launches": launches[0], "device_status": status, "clocks": clocks}
    return {
        "metric": "fwd+bwd voxels/s", "value": vox_total / (ms_step * 1e-3), "unit": "voxels/s", "n_gpus": world, "steps": steps,
        "warmup": warmup, "ms_per_step": ms_step, "higher_is_better": True, "scaling": "strong", "vs_baseline": None, "dtype": "f32",
        "data": "synthetic",
        "config": describe_config("c5", cfg, world, False),
        "e2e": {"value": vox_total / (ms_e2e * 1e-3), "unit": "voxels/s", "ms_per_step": ms_e2e,
                "h2d_bytes_per_step": int(2 * vox_rank * 4), "d2h_bytes_per_step": 4},
        "gpu_launches": launches[0], "device_status": status, "clocks": clocks,
        "roofline": {"kernel": "fused_backward_split_kernel<3> (per rank; gradient hand-overs inside the timed span)", "bound": "hbm",
                     "achieved": gbs_bwd, "peak": peak, "peak_source": peak_src, "unit": "GB/s", "frac": gbs_bwd / peak,
                     "algorithmic_bytes_per_launch": a_bwd / depth, "avg_launch_ms": ms_bwd / depth, "launches": depth,
                     "traffic": NCU_TRAFFIC_RATIO[("bwd", 3)] * a_bwd / depth,
                     "traffic_source": "ncu capture of one 128^3 layer, scaled by algorithmic bytes"},
        "roofline_forward": {"kernel": "forward2d_kernel<NT=3> + zgather_kernel", "bound": "hbm", "achieved": gbs_fwd, "peak": peak,
                             "unit": "GB/s", "frac": gbs_fwd / peak},
        "block_only": {"fwd_ms": ms_fwd, "bwd_ms": ms_bwd},
        "exchange": exchange, "loss": loss_value,
    }


# --------------------------------------------------------------------------------------- #
# CPU arm                                                                                   #
# --------------------------------------------------------------------------------------- #
def oracle_step_seconds(cfg, batch, spatial, threads, steps, warmup):
    """Seconds per fwd+bwd step of the CPU restatement (float32, in-place dense block)."""
    from oracle import msd_oracle as O

    torch.set_num_threads(threads)
    c = dict(cfg)
    c["spatial"] = spatial
    x, y = make_data(c, batch, 1000)
    if cfg["loss"] == "nll":
        y = y.squeeze(1)
    ws, fw, fb = make_weights(cfg, 4242)
    bias = torch.zeros(cfg["depth"])
    dil = [1 + (i % 10) for i in range(cfg["depth"])]
    times = []
    for i in range(warmup + steps):
        t0 = time.time()
        O.msd_network_step(x, y, dil, bias, ws, fw.squeeze(-1), fb, cfg["loss"])
        if i >= warmup:
            times.append(time.time() - t0)
    return statistics.median(times)


def cpu_ladder(cfg):
    """Sample sizes for the CPU, smallest to largest: one image / one cropped cube at full
    depth.  The largest is what a timed step uses; the smaller ones show how the per-voxel
    cost changes once the channel buffer no longer fits the host's caches."""
    if cfg["ndim"] == 2:
        return [tuple(min(s, e) for s in cfg["spatial"]) for e in (96, 192, 384, 512)]
    return [tuple(min(s, e) for s in cfg["spatial"]) for e in (24, 40, 56)]


CPU_ARM_BUDGET_S = 200.0  # the timed steps of `--impl reference` use the largest ladder size that fits this


def run_reference(args, name, cfg):
    threads = os.cpu_count() or 1
    ladder, chosen = [], None
    for sp in cpu_ladder(cfg):
        sec = oracle_step_seconds(cfg, 1, sp, threads, 1, 1 if not ladder else 0)
        ladder.append({"sample": "1x" + "x".join(map(str, sp)), "seconds_per_step": round(sec, 3), "voxels_per_s": round(voxels_of(1, sp) / sec, 1)})
        if chosen is None or sec * (args.steps + args.warmup) <= CPU_ARM_BUDGET_S:
            chosen = sp
    sp = chosen
    sec = oracle_step_seconds(cfg, 1, sp, threads, args.steps, args.warmup)
    vox = voxels_of(1, sp)
    v = vox / sec
    sample = ("one 1x%s sample at full depth %d per step (the largest size of `size_ladder` whose %d steps fit %d s)"
              % ("x".join(map(str, sp)), cfg["depth"], args.steps + args.warmup, int(CPU_ARM_BUDGET_S)))
    return {
        "impl": "reference", "metric": "fwd+bwd voxels/s", "value": v, "unit": "voxels/s", "n_gpus": args.gpus, "steps": args.steps,
        "warmup": args.warmup, "ms_per_step": sec * 1e3, "higher_is_better": True, "scaling": "strong" if args.strong else "weak",
        "vs_baseline": None, "dtype": "f32", "data": "synthetic",
        "config": describe_config(name, cfg, max(args.gpus, 1), args.strong),
        "cpu_baseline": {"value": v, "unit": "voxels/s", "cores": threads, "kind": "port", "sample": sample},
        "size_ladder": ladder,
        "e2e": {"value": v, "unit": "voxels/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
        "note": "the reference has no CPU implementation; this is its PyTorch-equivalent composition (oracle/msd_oracle.py) on the host cores",
    }


def ref_cuda_seconds(cfg, device, steps=2):
    """fwd+bwd of the dense block with the REFERENCE's own CUDA kernels (oracle/_ref, built
    unmodified), replaying msd_block.py's op sequence with its default block sizes."""
    from oracle import build_ref

    cc = build_ref.load()
    nd, depth, batch = cfg["ndim"], cfg["depth"], cfg["batch"]
    bs = {"f": (0, 16, 16), "x": (0, 16, 16), "k": (0, 16, 16), "b": (0, 16, 16)} if nd == 2 else \
        {"f": (2, 2, 32), "x": (2, 4, 16), "k": (2, 8, 16), "b": (8, 8, 8)}
    ws, _, _ = make_weights(cfg, 4242)
    ws = [w.to(device) for w in ws]
    bias = torch.zeros(depth, device=device)
    x, _ = make_data(cfg, batch, 1000)
    res = torch.empty((batch, 1 + depth) + tuple(cfg["spatial"]), device=device)
    res[:, :1] = x.to(device)
    grads = torch.randn_like(res)
    times = []
    for it in range(steps + 1):
        torch.cuda.synchronize()
        t0 = time.time()
        for i in range(depth):
            cc.conv_relu_forward(res[:, :1 + i], ws[i], bias[i:i + 1], res[:, 1 + i:2 + i], 1 + (i % 10), block_size=bs["f"])
        gb = torch.zeros_like(bias)
        for i in range(depth - 1, -1, -1):
            n = 1 + i
            d = 1 + (i % 10)
            cc.conv_relu_backward_x(res[:, n:n + 1], grads[:, n:n + 1], ws[i], grads[:, :n], d, block_size=bs["x"])
            gw = torch.zeros_like(ws[i])
            cc.conv_relu_backward_k(res[:, n:n + 1], grads[:, n:n + 1], res[:, :n], gw, d, block_size=bs["k"])
            cc.conv_relu_backward_bias(res[:, n:n + 1], grads[:, n:n + 1], gb[i:i + 1], block_size=bs["b"])
        torch.cuda.synchronize()
        if it > 0:
            times.append(time.time() - t0)
    return statistics.median(times)


def run_one_layer(spec, device, reps=10):
    """`--one-layer cfg:channels:dilation`: a few launches of one layer's forward and fused
    backward on the configuration's shape, timed with CUDA events (the profiling target)."""
    from msd_pytorch_b200 import msd_custom_convolutions as cc
    from msd_pytorch_b200.msd_block import block_backward_

    name, channels, d = spec.split(":")
    cfg, channels, d = CONFIGS[name], int(channels), int(d)
    nd = cfg["ndim"]
    batch, sp = cfg["batch"], cfg["spatial"]
    if name == "c5":  # one rank's slab of an 8-way split stands in for the 43 GB volume
        sp = (64,) + tuple(sp[1:])
    g = torch.Generator(device=device).manual_seed(0)
    res = torch.rand(batch, channels + 1, *sp, device=device, generator=g)
    grad = torch.randn(batch, channels + 1, *sp, device=device, generator=g)
    w = torch.randn(1, channels, *([3] * nd), device=device, generator=g) * (2.0 / (3 ** nd * channels)) ** 0.5
    b = torch.zeros(1, device=device)
    gw, gb = torch.zeros_like(w), torch.zeros(1, device=device)
    vox = voxels_of(batch, sp)
    out = {"layer": spec, "shape": [batch, channels + 1] + list(sp)}
    for what, fn, nbytes in (("forward", lambda: cc.conv_relu_forward(res[:, :channels], w, b, res[:, channels:channels + 1], d), 4 * vox * (channels + 1)),
                             ("backward", lambda: block_backward_(res, grad, channels, [d], [w], [gw], gb), 4 * vox * (3 * channels + 2))):
        fn()
        torch.cuda.synchronize()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        for _ in range(reps):
            fn()
        e1.record()
        torch.cuda.synchronize()
        ms = e0.elapsed_time(e1) / reps
        out[what] = {"ms": round(ms, 4), "algorithmic_GBps": round(nbytes / ms / 1e6, 1)}
    print(json.dumps(out), flush=True)


def run_layer_table(name, device, reps=10):
    """`--layer-table cfg`: microseconds of one layer's forward and of its fused backward (with
    the small reduction kernels of a one-layer block backward) against the number of input
    channels, for four dilations; each figure is a CUDA graph of `reps` launches replayed twice."""
    from msd_pytorch_b200 import msd_custom_convolutions as cc
    from msd_pytorch_b200.msd_block import block_backward_

    cfg = CONFIGS[name]
    nd, batch, sp = cfg["ndim"], cfg["batch"], cfg["spatial"]
    if name == "c5":
        sp = (64,) + tuple(sp[1:])
    channels = [c for c in (1, 4, 10, 25, 50, 100) if c <= cfg["depth"]]
    g = torch.Generator(device=device).manual_seed(0)
    top = max(channels)
    res = torch.rand(batch, top + 1, *sp, device=device, generator=g)
    grad = torch.randn(batch, top + 1, *sp, device=device, generator=g)
    b = torch.zeros(1, device=device)
    vox = voxels_of(batch, sp)
    peak, _ = measured_peak()

    def graph_us(fn):
        fn()
        torch.cuda.synchronize()
        gr = torch.cuda.CUDAGraph()
        with torch.cuda.graph(gr):
            for _ in range(reps):
                fn()
        gr.replay()
        torch.cuda.synchronize()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        gr.replay()
        gr.replay()
        e1.record()
        torch.cuda.synchronize()
        return e0.elapsed_time(e1) / (2 * reps) * 1e3

    for d in (1, 3, 6, 10):
        row = {"config": name, "dilation": d, "channels": channels, "forward_us": [], "forward_frac": [], "backward_us": [], "backward_frac": []}
        for c in channels:
            w = torch.randn(1, c, *([3] * nd), device=device, generator=g) * 0.1
            gw, gb = torch.zeros_like(w), torch.zeros(1, device=device)
            r, gr_ = res[:, :c + 1], grad[:, :c + 1]
            us = graph_us(lambda: cc.conv_relu_forward(res[:, :c], w, b, res[:, top:top + 1], d))
            row["forward_us"].append(round(us, 1))
            row["forward_frac"].append(round(4 * vox * (c + 1) / us / 1e3 / peak, 3))
            us = graph_us(lambda: block_backward_(r, gr_, c, [d], [w], [gw], gb))
            row["backward_us"].append(round(us, 1))
            row["backward_frac"].append(round(4 * vox * (3 * c + 2) / us / 1e3 / peak, 3))
        print(json.dumps(row), flush=True)


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=10)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--config", default="c2", choices=sorted(CONFIGS))
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--strong", action="store_true", help="split the config's global batch over the ranks instead of fixing the per-rank batch")
    ap.add_argument("--no-cpu-baseline", action="store_true")
    ap.add_argument("--no-ref-cuda", action="store_true")
    ap.add_argument("--no-autotune", action="store_true", help="use the library's default launch variants")
    ap.add_argument("--no-extra-configs", action="store_true", help="skip the c4 / c5_zslab records that follow the default config's line")
    ap.add_argument("--one-layer", default=None, metavar="CFG:CHANNELS:DILATION", help="time one layer's kernels (profiling target) and exit")
    ap.add_argument("--layer-table", default=None, metavar="CFG", choices=sorted(CONFIGS), help="time single layers over channel counts and dilations (CUDA graphs) and exit")
    ap.add_argument("--force-variant", default=None, metavar="FAMILY=V[,FAMILY=V]",
                    help="force a launch variant for all dilations (families: fwd2d, bwd2d, fwd3d, bwd3d); implies --no-autotune")
    args = ap.parse_args()
    args.warmup = max(args.warmup, 3) if args.impl == "ours" else args.warmup
    cfg = CONFIGS[args.config]
    rank = int(os.environ.get("RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    local = int(os.environ.get("LOCAL_RANK", "0"))

    if args.impl == "reference":
        if rank == 0:
            print(json.dumps(run_reference(args, args.config, cfg)), flush=True)
        return

    if not torch.cuda.is_available():
        raise SystemExit("bench.py needs a CUDA device (there is no CPU fallback); use --impl reference for the CPU baseline")
    device = torch.device("cuda", local)
    torch.cuda.set_device(device)
    torch.backends.cudnn.allow_tf32 = False
    torch.backends.cuda.matmul.allow_tf32 = False
    if args.force_variant:
        from msd_pytorch_b200 import _lib

        args.no_autotune = True
        fam = {"fwd2d": _lib.FAMILY_FWD2D, "bwd2d": _lib.FAMILY_BWD2D, "fwd3d": _lib.FAMILY_FWD3D, "bwd3d": _lib.FAMILY_BWD3D}
        for item in args.force_variant.split(","):
            name, v = item.split("=")
            for d in range(0, 33):
                _lib.check(_lib.lib.msd_tuning_set(fam[name], d, int(v)))
    if args.one_layer:
        run_one_layer(args.one_layer, device)
        return
    if args.layer_table:
        if not args.no_autotune:
            from msd_pytorch_b200 import autotune

            c = CONFIGS[args.layer_table]
            sp = c["spatial"] if args.layer_table != "c5" else (32,) + tuple(c["spatial"][1:])
            autotune.tune(c["batch"], sp, max(2, c["depth"] // 2), range(1, 11), device=device, reps=3)
        run_layer_table(args.layer_table, device)
        return
    if world > 1:
        import torch.distributed as dist

        os.environ.setdefault("MASTER_ADDR", "127.0.0.1")
        dist.init_process_group("nccl", device_id=device)
    if args.config == "c5":
        result = run_slab(args, cfg, rank, world, device, args.steps, args.warmup)
    else:
        result = run_ours(args, args.config, cfg, rank, world, device, args.steps, args.warmup)
    if rank == 0 and world == 1:
        if not args.no_cpu_baseline:
            threads = os.cpu_count() or 1
            sp = cpu_ladder(cfg)[-1]
            oracle_step_seconds(cfg, 1, cpu_ladder(cfg)[0], threads, 1, 0)  # warms the thread pool up
            sec = oracle_step_seconds(cfg, 1, sp, threads, 2, 0)
            result["cpu_baseline"] = {
                "value": voxels_of(1, sp) / sec, "unit": "voxels/s", "cores": threads, "kind": "port",
                "sample": "one 1x%s sample at full depth %d, median of 2 steps (%.1f s per step)" % ("x".join(map(str, sp)), cfg["depth"], sec)}
        if not args.no_ref_cuda and args.config != "c5":
            try:
                sec = ref_cuda_seconds(cfg, device)
                result["reference_cuda_kernels_on_this_gpu"] = {
                    "value": voxels_of(cfg["batch"], cfg["spatial"]) / sec, "unit": "voxels/s", "ms_per_step": sec * 1e3,
                    "what": "dense block fwd+bwd with the reference's own kernels compiled unmodified for sm_100a (no final layer / loss)"}
            except Exception as e:  # optional extra: the checker may not be built
                result["reference_cuda_kernels_on_this_gpu"] = {"unavailable": str(e)[:200]}
            torch.cuda.empty_cache()
    # ---- the 3D half of the target, as compact records at the end of the line ----
    if args.config == "c2" and not args.no_extra_configs and not args.strong:
        extra = {}
        if world == 1:
            extra["c4"] = run_ours(args, "c4", CONFIGS["c4"], rank, world, device, 5, 3, full=False)
        extra["c5_zslab"] = run_slab(args, CONFIGS["c5"], rank, world, device, 3, 3, full=False)
        if rank == 0:
            result.update(extra)
    if rank == 0:
        print(json.dumps(result), flush=True)
    if world > 1:
        import torch.distributed as dist

        dist.destroy_process_group()


if __name__ == "__main__":
    main()
