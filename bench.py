#!/usr/bin/env python
"""Benchmark of the MSD hot path: forward + backward voxels/s, HBM roofline fraction,
end-to-end figure through the public model API, and the CPU baseline.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--config c2] [--impl reference]

Prints ONE JSON line (rank 0).  Workloads (synthetic, seeded; dilations 1..10 cycling,
c_in = width = 1, float32, weights ~ N(0, 2/(taps*n_in)), zero bias, seeded non-zero
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
oracle/msd_oracle.py, on a bounded sample of the same workload.
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
# by the algorithmic bytes of the captured launch: 2D backward 1224.7 / 1275.1 MB and 2D forward
# 429.6 / 427.8 MB (batch 8 of 512x512, 50 input channels, dilation 10); 3D backward
# 2495.1 / 2550.1 MB (batch 2 of 128^3, 50 input channels, dilation 2) and 3D forward
# 509.6 / 436.2 MB (batch 2 of 128^3, 25 input channels, dilation 4).  Traffic grows with the channel count like the algorithmic bytes do, so the ratio
# is applied to the average launch.
NCU_TRAFFIC_RATIO = {("bwd", 2): 1224.7 / 1275.1, ("fwd", 2): 429.6 / 427.8, ("bwd", 3): 2495.1 / 2550.1, ("fwd", 3): 509.6 / 436.2}


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


def grads_bucket(model):
    return [p for p in model.msd.parameters() if p.requires_grad]


def run_ours(args, cfg, rank, world, device):
    import torch.distributed as dist
    from msd_pytorch_b200 import _lib
    from msd_pytorch_b200.msd_block import block_backward_, block_forward_

    batch = cfg["batch"]
    if args.strong:
        assert batch % world == 0
        batch //= world
    tuned = None
    if not args.no_autotune:
        # per-shape launch autotuning (untimed set-up; winners are cached on disk)
        from msd_pytorch_b200 import autotune

        tuned = autotune.tune(batch, cfg["spatial"], max(2, cfg["depth"] // 2), range(1, 11), device=device, reps=3)
    model = build_model(cfg, device)
    params = grads_bucket(model)
    x, y = make_data(cfg, batch, 1000 + rank)
    xd, yd = x.to(device), (y.squeeze(1) if cfg["loss"] == "nll" else y).to(device)
    xp, yp = x.pin_memory(), y.pin_memory()
    voxels_rank = batch
    for s in cfg["spatial"]:
        voxels_rank *= s
    flat = None

    def allreduce_grads():
        nonlocal flat
        if world == 1:
            return
        gs = [p.grad for p in params]
        flat = torch.cat([g.reshape(-1) for g in gs])
        dist.all_reduce(flat)
        flat /= world
        off = 0
        for g in gs:
            g.copy_(flat[off:off + g.numel()].view_as(g))
            off += g.numel()

    def step_device():
        for p in params:
            p.grad = None
        out = model.net(xd)
        loss = model.criterion(out, yd)
        loss.backward()
        allreduce_grads()
        if cfg["adam"]:
            model.optimizer.step()
        return loss

    def step_e2e():
        # the call a user makes: host tensors in, loss value out (H2D + D2H inside)
        val = model.forward(xp, yp)
        model.optimizer.zero_grad(set_to_none=True)
        model.loss.backward()
        allreduce_grads()
        if cfg["adam"]:
            model.optimizer.step()
        return val

    def timed(fn, steps, warmup, sample_clocks=False):
        for _ in range(warmup):
            fn()
        torch.cuda.synchronize()
        if world > 1:
            dist.barrier()
            torch.cuda.synchronize()
        sampler = ClockSampler(device.index) if sample_clocks else None
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
        if world > 1:
            dist.barrier()
            torch.cuda.synchronize()
            tt = torch.tensor([ms], device=device)
            dist.all_reduce(tt, op=dist.ReduceOp.MAX)
            ms = float(tt.item())
        clocks = sampler.stop(t0, t1) if sampler else None
        return ms / steps, (l1[0] - l0[0], l1[1] - l0[1]), clocks

    ms_step, launches, clocks = timed(step_device, args.steps, args.warmup, sample_clocks=True)
    ms_e2e, _, _ = timed(step_e2e, max(2, args.steps // 2), max(3, args.warmup // 2))
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
    ms_fwd, lf, _ = timed(fwd_only, args.steps, args.warmup)
    gbuf.copy_(gsrc)
    ms_bwd, lb, _ = timed(bwd_only, args.steps, args.warmup)
    del gbuf, gsrc, res
    a_fwd, a_bwd = algorithmic_bytes(depth, voxels_rank)
    peak, peak_src = measured_peak()
    gbs_fwd = a_fwd / (ms_fwd * 1e-3) / 1e9
    gbs_bwd = a_bwd / (ms_bwd * 1e-3) / 1e9

    result = None
    if rank == 0:
        total_vox = voxels_rank * world
        result = {
            "metric": "fwd+bwd voxels/s",
            "value": total_vox / (ms_step * 1e-3),
            "unit": "voxels/s",
            "n_gpus": world,
            "steps": args.steps,
            "warmup": args.warmup,
            "ms_per_step": ms_step,
            "higher_is_better": True,
            "scaling": "strong" if args.strong else "weak",
            "vs_baseline": None,
            "dtype": "f32",
            "data": "synthetic",
            "config": {
                "workload": "%s: MSD %dD depth %d, batch %d/GPU of 1x%s, c_out %d, %s loss, fwd+bwd%s; block + final 1x1 layer + loss; "
                            "inputs larger than L2 (%.2f GB channel buffer)" % (
                                args.config, nd, depth, batch, "x".join(map(str, cfg["spatial"])), cfg["c_out"], cfg["loss"],
                                "+Adam" if cfg["adam"] else "", 4 * voxels_rank * (1 + depth) / 1e9),
                "parallelism": "dp%d" % world if world > 1 else "single",
                "l2_policy": "inputs larger than L2",
                "launch_variants": {k: [v[d] for d in sorted(v)] for k, v in tuned.items()} if tuned else "library defaults",
            },
            "e2e": {"value": total_vox / (ms_e2e * 1e-3), "unit": "voxels/s", "ms_per_step": ms_e2e,
                    "h2d_bytes_per_step": int(xp.numel() * xp.element_size() + yp.numel() * yp.element_size()), "d2h_bytes_per_step": 4},
            "gpu_launches": launches[0],
            "gpu_launches_tuned_path": launches[1],
            "device_status": status,
            "clocks": clocks,
            "roofline": {
                "kernel": ("fused_backward_kernel" if nd == 2 else "fused_backward3d_split_kernel (fused_backward_kernel<3> below 8 input channels)")
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
    return result


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


def cpu_sample(cfg):
    """A bounded sample of the workload for the CPU: one image / a cropped volume."""
    if cfg["ndim"] == 2:
        return 1, tuple(min(s, 192) for s in cfg["spatial"])
    return 1, tuple(min(s, 40) for s in cfg["spatial"])


def run_reference(args, cfg):
    threads = os.cpu_count() or 1
    batch, sp = cpu_sample(cfg)
    sec = oracle_step_seconds(cfg, batch, sp, threads, args.steps, min(args.warmup, 1))
    vox = batch
    for s in sp:
        vox *= s
    v = vox / sec
    sample = "batch %d of 1x%s at full depth %d per step (per-voxel cost is size-independent)" % (batch, "x".join(map(str, sp)), cfg["depth"])
    return {
        "impl": "reference", "metric": "fwd+bwd voxels/s", "value": v, "unit": "voxels/s", "n_gpus": args.gpus, "steps": args.steps,
        "warmup": min(args.warmup, 1), "ms_per_step": sec * 1e3, "higher_is_better": True, "scaling": "weak", "vs_baseline": None,
        "dtype": "f32", "data": "synthetic",
        "config": {"workload": "%s (CPU sample: %s)" % (args.config, sample), "parallelism": "host threads"},
        "cpu_baseline": {"value": v, "unit": "voxels/s", "cores": threads, "kind": "port", "sample": sample},
        "e2e": {"value": v, "unit": "voxels/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
        "note": "the reference has no CPU implementation; this is its PyTorch-equivalent composition (oracle/msd_oracle.py)",
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
    args = ap.parse_args()
    args.warmup = max(args.warmup, 3) if args.impl == "ours" else args.warmup
    cfg = CONFIGS[args.config]
    rank = int(os.environ.get("RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    local = int(os.environ.get("LOCAL_RANK", "0"))

    if args.impl == "reference":
        if rank == 0:
            print(json.dumps(run_reference(args, cfg)), flush=True)
        return

    if args.config == "c5":
        from msd_pytorch_b200 import slab_bench

        slab_bench.main(args, cfg, rank, world, local, peak=measured_peak())
        return

    if not torch.cuda.is_available():
        raise SystemExit("bench.py needs a CUDA device (there is no CPU fallback); use --impl reference for the CPU baseline")
    device = torch.device("cuda", local)
    torch.cuda.set_device(device)
    if world > 1:
        import torch.distributed as dist

        os.environ.setdefault("MASTER_ADDR", "127.0.0.1")
        dist.init_process_group("nccl", device_id=device)
    torch.backends.cudnn.allow_tf32 = False
    torch.backends.cuda.matmul.allow_tf32 = False
    result = run_ours(args, cfg, rank, world, device)
    if rank == 0:
        if world == 1 and not args.no_cpu_baseline:
            threads = os.cpu_count() or 1
            batch, sp = cpu_sample(cfg)
            sec = oracle_step_seconds(cfg, batch, sp, threads, 2, 0)
            vox = batch
            for s in sp:
                vox *= s
            result["cpu_baseline"] = {
                "value": vox / sec, "unit": "voxels/s", "cores": threads, "kind": "port",
                "sample": "batch %d of 1x%s at full depth %d, median of 2 steps (%.1f s per step)" % (
                    batch, "x".join(map(str, sp)), cfg["depth"], sec)}
        if world == 1 and not args.no_ref_cuda:
            try:
                sec = ref_cuda_seconds(cfg, device)
                vox = cfg["batch"]
                for s in cfg["spatial"]:
                    vox *= s
                result["reference_cuda_kernels_on_this_gpu"] = {
                    "value": vox / sec, "unit": "voxels/s", "ms_per_step": sec * 1e3,
                    "what": "dense block fwd+bwd with the reference's own kernels compiled unmodified for sm_100a (no final layer / loss)"}
            except Exception as e:  # optional extra: the checker may not be built
                result["reference_cuda_kernels_on_this_gpu"] = {"unavailable": str(e)[:200]}
        print(json.dumps(result), flush=True)
    if world > 1:
        import torch.distributed as dist

        dist.destroy_process_group()


if __name__ == "__main__":
    main()
