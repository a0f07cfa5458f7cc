"""Multi-GPU execution of the MSD hot path: one process per GPU.

Two partitionings, following the shapes of the workloads:

* **Batch data-parallel** (2D workloads): every rank runs the whole block on its share of
  the batch; the only exchange is ONE all-reduce per step over a flat bucket holding all
  parameter gradients (:class:`GradientBucket`).  The reference's counterpart is
  ``nn.DataParallel`` (msd_regression_model.py:78-79), a single-process scatter/gather.

* **z-slab decomposition** (one large 3D volume; no counterpart in the reference): the
  volume is cut into contiguous slabs of z-planes (:class:`SlabPlan`).  Each rank keeps its
  slab of the dense channel buffer plus ``halo`` planes of room on each interior side.
  A 3x3x3 layer couples planes only through its three z-taps, and the forward kernels
  already split the sum by z-tap (in-plane partial sums ``u_t``, then
  ``out[z] = relu(b + u_0[z-d] + u_1[z] + u_2[z+d])``).  So per forward layer every rank
  computes the partial sums of its OWN planes only, boundary planes first; ``d`` planes of
  ``u_0`` go to the upper neighbour and ``d`` planes of ``u_2`` to the lower one
  (point-to-point, NVLink under NCCL) while the interior planes are computed; then the
  gather step runs.  No activation halo is ever exchanged and no plane is computed twice.
  Per backward layer the ``d`` boundary planes of the (already gated) gradient channel the
  layer reads are needed from the neighbours; the layer above computes its boundary planes
  first and sends them while it works on its interior.  The edge-inclusive reflection
  applies only at the volume's real ends, where the local buffer ends too.  Weight and
  bias gradients are summed over the ranks once, at the end of the backward.

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

    ``allreduce_()`` averages (or sums) the ``.grad`` tensors over the ranks.  The gradients
    are gathered into the flat buffer with one multi-tensor copy, reduced with one collective
    (a few tens of thousands of floats: latency-bound, so a single launch is what matters),
    and every ``p.grad`` is then re-pointed at its slice of the buffer - nothing is copied
    back.  When the gradients already are those slices (the caller kept them and accumulated
    in place) the gather is skipped as well."""

    def __init__(self, params, group=None):
        self.params = [p for p in params if p.requires_grad]
        self.group = group
        self.numel = sum(p.numel() for p in self.params)
        self.flat = None
        self.views = None

    def _ensure(self, like):
        if self.flat is None or self.flat.device != like.device or self.flat.dtype != like.dtype:
            self.flat = torch.empty(self.numel, dtype=like.dtype, device=like.device)
            self.views, off = [], 0
            for p in self.params:
                self.views.append(self.flat[off:off + p.numel()].view_as(p))
                off += p.numel()

    def allreduce_(self, average=True):
        world = dist.get_world_size(self.group) if dist.is_initialized() else 1
        if world == 1:
            return
        grads = [p.grad for p in self.params]
        if any(g is None for g in grads):
            raise RuntimeError("GradientBucket.allreduce_: a parameter has no gradient")
        self._ensure(grads[0])
        in_place = all(g.data_ptr() == v.data_ptr() and g.is_contiguous() for g, v in zip(grads, self.views))
        if not in_place:
            torch.cat([g.reshape(-1) for g in grads], out=self.flat)
        if average and dist.get_backend(self.group) == "nccl":
            dist.all_reduce(self.flat, op=dist.ReduceOp.AVG, group=self.group)
        else:
            dist.all_reduce(self.flat, group=self.group)
            if average:
                self.flat /= world
        if not in_place:
            for p, v in zip(self.params, self.views):
                p.grad = v


# --------------------------------------------------------------------------- #
# z-slab decomposition                                                         #
# --------------------------------------------------------------------------- #
class SlabPlan:
    """Contiguous split of ``Z`` planes over ``world`` ranks with ``halo`` planes of room for
    the neighbours' data on each interior side (``halo`` >= the largest dilation)."""

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


def halo_transfers(plan, rank, width=None):
    """The point-to-point transfers that fill ``rank``'s halo planes of one channel with the
    neighbours' boundary planes, ``width`` planes per face (default: the whole halo): a list
    of ``(kind, peer, z_from, z_to)`` in LOCAL plane indices, kind 'send' or 'recv'."""
    loc = plan.local(rank)
    H = plan.halo if width is None else width
    if plan.world > 1 and H > plan.halo:
        raise ValueError("cannot exchange %d planes with a halo of %d" % (H, plan.halo))
    ops = []
    if rank > 0:  # lower neighbour: it needs my first H owned planes; I need its last H
        ops.append(("send", rank - 1, loc["z_begin"], loc["z_begin"] + H))
        ops.append(("recv", rank - 1, loc["z_begin"] - H, loc["z_begin"]))
    if rank < plan.world - 1:
        ops.append(("send", rank + 1, loc["z_end"] - H, loc["z_end"]))
        ops.append(("recv", rank + 1, loc["z_end"], loc["z_end"] + H))
    return ops


def partial_sum_transfers(plan, rank, d):
    """Transfers of one forward layer with dilation ``d``: ``(kind, peer, tap, z_from, z_to)``
    over the z-tap partial sums ``u[tap]`` in LOCAL plane indices.  Output plane z reads
    ``u_0[z-d]`` and ``u_2[z+d]``: the upper neighbour's lowest ``d`` outputs need ``u_0`` of
    my top ``d`` planes, the lower neighbour's highest ``d`` outputs need ``u_2`` of my bottom
    ``d`` planes, and I need the mirror images of both."""
    if plan.world > 1 and d > plan.halo:
        raise ValueError("dilation %d exceeds the halo of %d planes" % (d, plan.halo))
    loc = plan.local(rank)
    zb, ze = loc["z_begin"], loc["z_end"]
    ops = []
    if rank > 0:
        ops.append(("send", rank - 1, 2, zb, zb + d))
        ops.append(("recv", rank - 1, 0, zb - d, zb))
    if rank < plan.world - 1:
        ops.append(("send", rank + 1, 0, ze - d, ze))
        ops.append(("recv", rank + 1, 2, ze, ze + d))
    return ops


def boundary_windows(plan, rank, width):
    """Splits the owned planes into the windows next to interior faces (``width`` planes each,
    the ones a neighbour is waiting for) and the rest: ``(boundary, interior)``, lists of
    ``(z_begin, z_end)`` in local indices.  A slab too thin to split is all boundary."""
    loc = plan.local(rank)
    zb, ze = loc["z_begin"], loc["z_end"]
    lower, upper = rank > 0, rank < plan.world - 1
    if not (lower or upper):
        return [], [(zb, ze)]
    if (ze - zb) <= width * (int(lower) + int(upper)):
        return [(zb, ze)], []
    boundary = ([(zb, zb + width)] if lower else []) + ([(ze - width, ze)] if upper else [])
    return boundary, [(zb + (width if lower else 0), ze - (width if upper else 0))]


class _Done:
    def wait(self):
        pass


class _Works:
    def __init__(self, works):
        self.works = works

    def wait(self):
        """Makes the current stream wait for the transfers (the host does not block)."""
        for w in self.works:
            w.wait()


class TorchRanks:
    """Communicator over ``torch.distributed`` (one process per rank)."""

    def __init__(self, group=None):
        self.group = group
        self.rank = dist.get_rank(group)
        self.world = dist.get_world_size(group)

    def start(self, transfers):
        """``transfers``: {rank: [(kind, peer, tag, tensor)]} holding this process's rank only.
        Enqueues all of them as one group behind the work already on the current stream and
        returns a handle whose ``wait()`` orders the current stream after their completion."""
        ops = []
        for kind, peer, _tag, tensor in transfers.get(self.rank, []):
            fn = dist.isend if kind == "send" else dist.irecv
            ops.append(dist.P2POp(fn, tensor, peer, self.group))
        return _Works(dist.batch_isend_irecv(ops)) if ops else _Done()

    def exchange(self, plan, volumes, width=None):
        """``volumes``: {rank: tensor [Zl, Y, X]} holding this process's rank only."""
        vol = volumes[self.rank]
        self.start({self.rank: [(k, peer, 0, vol[a:b]) for k, peer, a, b in halo_transfers(plan, self.rank, width)]}).wait()

    def allreduce_sum(self, tensors):
        for t in tensors.values():
            dist.all_reduce(t, group=self.group)

    def ranks(self):
        return [self.rank]


class VirtualRanks:
    """All ranks played by one process (tests, single-GPU checks): the 'transfers' are copies."""

    def __init__(self, world):
        self.world = world

    def start(self, transfers):
        for r, ops in transfers.items():
            for kind, peer, tag, src in ops:
                if kind != "send":
                    continue
                dst = [t for (k, p, g, t) in transfers[peer] if k == "recv" and p == r and g == tag]
                if len(dst) != 1:
                    raise RuntimeError("send %d -> %d (tag %r) has %d matching receives" % (r, peer, tag, len(dst)))
                dst[0].copy_(src)
        return _Done()

    def exchange(self, plan, volumes, width=None):
        self.start({r: [(k, peer, 0, volumes[r][a:b]) for k, peer, a, b in halo_transfers(plan, r, width)] for r in range(self.world)})

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
        nvox = self.loc["planes"] * Y * X
        n = _lib.lib.msd_forward_workspace_bytes(_lib.MSD_F32, 5, nvox)
        n = max(n, _lib.lib.msd_workspace_bytes(_lib.MSD_F32, 5, nvox, c_in + depth, 1))
        self.ws = torch.empty(int(n), dtype=torch.uint8, device=device)
        # the forward's z-tap partial sums u[tap][z][y][x] live at the start of the workspace
        self.u = self.ws[:3 * nvox * 4].view(torch.float32).view(3, self.loc["planes"], Y, X)

    @property
    def owned(self):
        return slice(self.loc["z_begin"], self.loc["z_end"])

    def set_input(self, x_global_slab):
        """``x_global_slab``: the owned planes of the input ``[c_in, Zo, Y, X]``."""
        self.result[0, :self.c_in, self.owned] = x_global_slab

    def forward_layer(self, i, weight, bias_i, dilation, window=None, flags=0):
        dev = self.device
        z0, z1 = window or (self.loc["z_begin"], self.loc["z_end"])
        _lib.check(_lib.lib.msd_slab_layer_forward(_lib.describe(self.result), self.c_in + i, weight.data_ptr(), bias_i.data_ptr(), int(dilation),
                                                   int(z0), int(z1), int(flags), self.ws.data_ptr(), self.ws.numel(), dev.index,
                                                   _lib.stream_of(dev)))

    def gate_top_channel(self):
        """Multiply the gradient of the last channel by its ReLU gate on the owned planes (the
        layers below get theirs gated by the kernel of the layer above)."""
        g = self.gradients[0, -1, self.owned]
        g.mul_(self.result[0, -1, self.owned] > 0)

    def backward_layer(self, i, weight, dilation, grad_weight, grad_bias_i, flags=0, window=None):
        dev = self.device
        z0, z1 = window or (self.loc["z_begin"], self.loc["z_end"])
        _lib.check(_lib.lib.msd_slab_layer_backward(_lib.describe(self.result), _lib.describe(self.gradients), self.c_in + i, weight.data_ptr(),
                                                    int(dilation), int(z0), int(z1), grad_weight.data_ptr(),
                                                    grad_bias_i.data_ptr(), int(flags), self.ws.data_ptr(), self.ws.numel(), dev.index,
                                                    _lib.stream_of(dev)))


def slab_forward(comm, plan, blocks, weights, bias, dilations):
    """Forward of all layers on the ranks in ``blocks`` ({rank: SlabBlock}).  Per layer: the
    z-tap partial sums of the planes next to interior faces, their hand-over to the neighbours
    (in flight while the interior planes are computed), then the gather step."""
    S, G = _lib.SLAB_FORWARD_SUMS_ONLY, _lib.SLAB_FORWARD_GATHER_ONLY
    for i, (w, d) in enumerate(zip(weights, dilations)):
        split = {r: boundary_windows(plan, r, d) for r in blocks}
        for r, b in blocks.items():
            for win in split[r][0]:
                b.forward_layer(i, w, bias[i:i + 1], d, win, S)
        pending = comm.start({r: [(k, peer, tap, b.u[tap, a:z]) for k, peer, tap, a, z in partial_sum_transfers(plan, r, d)]
                              for r, b in blocks.items()})
        for r, b in blocks.items():
            for win in split[r][1]:
                b.forward_layer(i, w, bias[i:i + 1], d, win, S)
        pending.wait()
        for b in blocks.values():
            b.forward_layer(i, w, bias[i:i + 1], d, None, G)


def slab_backward(comm, plan, blocks, weights, dilations):
    """Backward of all layers, last to first.  ``b.gradients`` must hold the gradient w.r.t.
    every channel on the owned planes.  Returns ({rank: [grad_weight_i]}, {rank: grad_bias})
    already summed over the ranks; the input gradient is ``b.gradients[:, :c_in]`` (owned planes).

    Layer i reads channel c_in + i of the gradients ``d_i`` planes beyond its window.  That
    channel is final once layer i + 1 has run, so layer i + 1 computes the planes next to
    interior faces first and their hand-over travels while it computes its interior."""
    gws = {r: [torch.zeros_like(w) for w in weights] for r in blocks}
    gbs = {r: torch.zeros(len(weights), device=b.device) for r, b in blocks.items()}
    # Every layer reads an already gated gradient channel: the top one is gated here, each
    # other one by the kernel of the layer above when it stores that channel; the exchanged
    # halo planes therefore carry gated values and no activation halo is read.
    for b in blocks.values():
        b.gate_top_channel()
    depth = len(weights)

    def start_halo(i):
        return comm.start({r: [(k, peer, 0, b.gradients[0, b.c_in + i, a:z]) for k, peer, a, z in halo_transfers(plan, r, dilations[i])]
                           for r, b in blocks.items()})

    pending = start_halo(depth - 1)
    for i in range(depth - 1, -1, -1):
        pending.wait()
        flags = _lib.SLAB_GRADIENT_IS_GATED | (_lib.SLAB_GATE_CHANNEL_BELOW if i > 0 else 0)
        split = {r: boundary_windows(plan, r, dilations[i - 1]) if i > 0 else ([], [(b.loc["z_begin"], b.loc["z_end"])]) for r, b in blocks.items()}
        for r, b in blocks.items():
            for win in split[r][0]:
                b.backward_layer(i, weights[i], dilations[i], gws[r][i], gbs[r][i:i + 1], flags, win)
        if i > 0:
            pending = start_halo(i - 1)
        for r, b in blocks.items():
            for win in split[r][1]:
                b.backward_layer(i, weights[i], dilations[i], gws[r][i], gbs[r][i:i + 1], flags, win)
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
