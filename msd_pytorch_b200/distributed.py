"""Multi-GPU execution of the MSD hot path: one process per GPU.

Two partitionings, following the shapes of the workloads:

* **Batch data-parallel** (2D workloads): every rank runs the whole block on its share of
  the batch; the only exchange is ONE all-reduce per step over a flat bucket holding all
  parameter gradients (:class:`GradientBucket`).  The reference's counterpart is
  ``nn.DataParallel`` (msd_regression_model.py:78-79), a single-process scatter/gather.

* **z-slab decomposition** (one large 3D volume; no counterpart in the reference): the
  volume is cut into contiguous slabs of z-planes (:class:`SlabPlan`).  Each rank keeps its
  slab of the dense channel buffer plus ``halo`` planes of its neighbours on each interior
  side.  After a layer has produced its channel on the owned planes, the ``halo`` boundary
  planes of that ONE channel go to the neighbours (point-to-point, NVLink under NCCL);
  before a layer's backward the same happens for its gradient channel.  The edge-inclusive
  reflection applies only at the volume's real ends, where the local buffer ends too.
  Weight and bias gradients are summed over the ranks once, at the end of the backward.

The exchange schedule is written against a tiny communicator interface so that it runs
unchanged over ``torch.distributed`` (NCCL on GPUs, gloo on CPU tensors in the tests) and
over :class:`VirtualRanks`, which plays all ranks inside one process on one GPU.
"""
import ctypes

import torch
import torch.distributed as dist

from . import _lib


# --------------------------------------------------------------------------- #
# batch data-parallel                                                          #
# --------------------------------------------------------------------------- #
def split_batch(batch, rank, world):
    """Samples [lo, hi) of a global batch owned by ``rank`` (even split required)."""
    if batch % world:
        raise ValueError("batch %d is not divisible by the number of ranks %d" % (batch, world))
    per = batch // world
    return rank * per, (rank + 1) * per


class GradientBucket:
    """All gradients of ``params`` as ONE flat buffer, so that a step needs one all-reduce.

    ``allreduce_()`` averages (or sums) the ``.grad`` tensors over the ranks in place.  With a
    few tens of thousands of floats the collective is latency-bound; bucketing it is what
    keeps it to a single launch."""

    def __init__(self, params, group=None):
        self.params = [p for p in params if p.requires_grad]
        self.group = group
        self.numel = sum(p.numel() for p in self.params)
        self.flat = None

    def allreduce_(self, average=True):
        world = dist.get_world_size(self.group) if dist.is_initialized() else 1
        if world == 1:
            return
        grads = [p.grad for p in self.params]
        if any(g is None for g in grads):
            raise RuntimeError("GradientBucket.allreduce_: a parameter has no gradient")
        if self.flat is None or self.flat.device != grads[0].device or self.flat.dtype != grads[0].dtype:
            self.flat = torch.empty(self.numel, dtype=grads[0].dtype, device=grads[0].device)
        torch.cat([g.reshape(-1) for g in grads], out=self.flat)
        dist.all_reduce(self.flat, group=self.group)
        if average:
            self.flat /= world
        off = 0
        for g in grads:
            g.copy_(self.flat[off:off + g.numel()].view_as(g))
            off += g.numel()


# --------------------------------------------------------------------------- #
# z-slab decomposition                                                         #
# --------------------------------------------------------------------------- #
class SlabPlan:
    """Contiguous split of ``Z`` planes over ``world`` ranks with ``halo`` planes of overlap."""

    def __init__(self, Z, world, halo):
        if world < 1 or Z < world:
            raise ValueError("cannot split %d planes over %d ranks" % (Z, world))
        self.Z, self.world, self.halo = Z, world, halo
        self.bounds = [(r * Z // world, (r + 1) * Z // world) for r in range(world)]
        if world > 1 and min(b - a for a, b in self.bounds) < halo:
            raise ValueError("slabs of %d planes are thinner than the halo of %d" % (min(b - a for a, b in self.bounds), halo))

    def local(self, rank):
        """Geometry of ``rank``'s local buffer: global range, halo widths, owned window."""
        g0, g1 = self.bounds[rank]
        lo = self.halo if rank > 0 else 0
        hi = self.halo if rank < self.world - 1 else 0
        return dict(g0=g0, g1=g1, lo=lo, hi=hi, planes=(g1 - g0) + lo + hi, z_begin=lo, z_end=lo + (g1 - g0))


def halo_transfers(plan, rank):
    """The point-to-point transfers of one exchange, for ``rank``: a list of
    ``(kind, peer, z_from, z_to)`` in LOCAL plane indices, kind 'send' or 'recv'."""
    loc = plan.local(rank)
    H = plan.halo
    ops = []
    if rank > 0:  # lower neighbour: it needs my first H owned planes; I need its last H
        ops.append(("send", rank - 1, loc["z_begin"], loc["z_begin"] + H))
        ops.append(("recv", rank - 1, 0, H))
    if rank < plan.world - 1:
        ops.append(("send", rank + 1, loc["z_end"] - H, loc["z_end"]))
        ops.append(("recv", rank + 1, loc["z_end"], loc["z_end"] + H))
    return ops


class TorchRanks:
    """Communicator over ``torch.distributed`` (one process per rank)."""

    def __init__(self, group=None):
        self.group = group
        self.rank = dist.get_rank(group)
        self.world = dist.get_world_size(group)

    def exchange(self, plan, volumes):
        """``volumes``: {rank: tensor [Zl, Y, X]} holding this process's rank only."""
        vol = volumes[self.rank]
        ops = []
        for kind, peer, a, b in halo_transfers(plan, self.rank):
            fn = dist.isend if kind == "send" else dist.irecv
            ops.append(dist.P2POp(fn, vol[a:b], peer, self.group))
        if ops:
            for req in dist.batch_isend_irecv(ops):
                req.wait()

    def allreduce_sum(self, tensors):
        for t in tensors.values():
            dist.all_reduce(t, group=self.group)

    def ranks(self):
        return [self.rank]


class VirtualRanks:
    """All ranks played by one process (tests, single-GPU checks): the 'transfers' are copies."""

    def __init__(self, world):
        self.world = world

    def exchange(self, plan, volumes):
        for r in range(self.world):
            for kind, peer, a, b in halo_transfers(plan, r):
                if kind != "send":
                    continue
                # the matching receive of `peer`: planes of the same global indices
                dst = [op for op in halo_transfers(plan, peer) if op[0] == "recv" and op[1] == r][0]
                volumes[peer][dst[2]:dst[3]].copy_(volumes[r][a:b])

    def allreduce_sum(self, tensors):
        total = sum(tensors.values())
        for t in tensors.values():
            t.copy_(total)

    def ranks(self):
        return list(range(self.world))


class SlabBlock:
    """State of ONE rank of a z-slab decomposed MSD block (batch 1, c_in channels, width 1)."""

    def __init__(self, plan, rank, c_in, depth, spatial_yx, device):
        self.plan, self.rank, self.c_in, self.depth = plan, rank, c_in, depth
        self.loc = plan.local(rank)
        Y, X = spatial_yx
        self.device = device
        self.result = torch.zeros(1, c_in + depth, self.loc["planes"], Y, X, device=device)
        self.gradients = None
        n = _lib.lib.msd_forward_workspace_bytes(_lib.MSD_F32, 5, self.loc["planes"] * Y * X)
        n = max(n, _lib.lib.msd_workspace_bytes(_lib.MSD_F32, 5, self.loc["planes"] * Y * X, c_in + depth, 1))
        self.ws = torch.empty(int(n), dtype=torch.uint8, device=device)

    @property
    def owned(self):
        return slice(self.loc["z_begin"], self.loc["z_end"])

    def set_input(self, x_global_slab):
        """``x_global_slab``: the owned planes of the input ``[c_in, Zo, Y, X]``."""
        self.result[0, :self.c_in, self.owned] = x_global_slab

    def forward_layer(self, i, weight, bias_i, dilation):
        dev = self.device
        _lib.check(_lib.lib.msd_slab_layer_forward(_lib.describe(self.result), self.c_in + i, weight.data_ptr(), bias_i.data_ptr(), int(dilation),
                                                   self.loc["z_begin"], self.loc["z_end"], self.ws.data_ptr(), self.ws.numel(), dev.index,
                                                   _lib.stream_of(dev)))

    def gate_top_channel(self):
        """Multiply the gradient of the last channel by its ReLU gate on the owned planes (the
        layers below get theirs gated by the kernel of the layer above)."""
        g = self.gradients[0, -1, self.owned]
        g.mul_(self.result[0, -1, self.owned] > 0)

    def backward_layer(self, i, weight, dilation, grad_weight, grad_bias_i, flags=0):
        dev = self.device
        _lib.check(_lib.lib.msd_slab_layer_backward(_lib.describe(self.result), _lib.describe(self.gradients), self.c_in + i, weight.data_ptr(),
                                                    int(dilation), self.loc["z_begin"], self.loc["z_end"], grad_weight.data_ptr(),
                                                    grad_bias_i.data_ptr(), int(flags), self.ws.data_ptr(), self.ws.numel(), dev.index,
                                                    _lib.stream_of(dev)))


def slab_forward(comm, plan, blocks, weights, bias, dilations):
    """Forward of all layers on the ranks in ``blocks`` ({rank: SlabBlock}); exchanges the new
    channel's boundary planes after every layer (and the input channels' first)."""
    any_block = next(iter(blocks.values()))
    for c in range(any_block.c_in):
        comm.exchange(plan, {r: b.result[0, c] for r, b in blocks.items()})
    for i, (w, d) in enumerate(zip(weights, dilations)):
        for b in blocks.values():
            b.forward_layer(i, w, bias[i:i + 1], d)
        comm.exchange(plan, {r: b.result[0, b.c_in + i] for r, b in blocks.items()})


def slab_backward(comm, plan, blocks, weights, dilations):
    """Backward of all layers, last to first.  ``b.gradients`` must hold the gradient w.r.t.
    every channel on the owned planes.  Returns ({rank: [grad_weight_i]}, {rank: grad_bias})
    already summed over the ranks; the input gradient is ``b.gradients[:, :c_in]`` (owned planes)."""
    gws = {r: [torch.zeros_like(w) for w in weights] for r in blocks}
    gbs = {r: torch.zeros(len(weights), device=b.device) for r, b in blocks.items()}
    # Every layer reads an already gated gradient channel: the top one is gated here, each
    # other one by the kernel of the layer above when it stores that channel; the exchanged
    # halo planes therefore carry gated values and no activation halo is read.
    for b in blocks.values():
        b.gate_top_channel()
    for i in range(len(weights) - 1, -1, -1):
        comm.exchange(plan, {r: b.gradients[0, b.c_in + i] for r, b in blocks.items()})
        flags = _lib.SLAB_GRADIENT_IS_GATED | (_lib.SLAB_GATE_CHANNEL_BELOW if i > 0 else 0)
        for r, b in blocks.items():
            b.backward_layer(i, weights[i], dilations[i], gws[r][i], gbs[r][i:i + 1], flags)
    # one sum over the ranks for all weight gradients, one for the bias
    flat = {r: torch.cat([g.reshape(-1) for g in gws[r]] + [gbs[r]]) for r in blocks}
    comm.allreduce_sum(flat)
    for r in blocks:
        off = 0
        for g in gws[r]:
            g.copy_(flat[r][off:off + g.numel()].view_as(g))
            off += g.numel()
        gbs[r].copy_(flat[r][off:])
    return gws, gbs
