"""Writes golden vectors produced by the REFERENCE's own CUDA kernels.

Needs a GPU and ``oracle/_ref/msd_custom_convolutions_ref.so`` (the reference's ten
native sources compiled unmodified by ``oracle/build_ref.py``).  The reference's op
sequence for the dense block (msd_pytorch/msd_block.py:40-58,88-130) is replayed
on top of its ops.  Output: ``<outdir>/ref_cuda_ops.npz`` and ``ref_cuda_block.npz``
(float64 computations by the reference's double instantiations, plus the same from its
float32 instantiations under ``*_f32_*`` keys), which are then committed under ``tests/golden/``.

Usage (on a machine with a GPU):  python tests/golden/make_golden_ref_cuda.py <outdir>
"""
import os
import sys

import numpy as np
import torch

HERE = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, os.path.join(HERE, "..", ".."))
sys.path.insert(0, HERE)

import cases  # noqa: E402
from oracle import build_ref  # noqa: E402


def blocks(nd):
    return (0, 16, 16) if nd == 2 else (4, 4, 8)


def main(outdir):
    cc = build_ref.load()
    dev = torch.device("cuda:0")
    out = {}
    for case in cases.OP_CASES:
        name = case[0]
        a = cases.op_inputs(case)
        nd = a["x"].ndim - 2
        bs = blocks(nd)
        for dt, dtag in ((torch.float64, ""), (torch.float32, "_f32")):
            x, k, b, g = (torch.from_numpy(a[n]).to(dev, dt) for n in ("x", "k", "b", "g"))
            d = a["d"]
            for relu in (False, True):
                tag = name + ("_relu" if relu else "_lin") + dtag
                y = torch.empty_like(g)
                (cc.conv_relu_forward if relu else cc.conv_forward)(x, k, b, y, d, block_size=bs)
                gx = torch.zeros_like(x)
                gk = torch.zeros_like(k)
                gb = torch.zeros_like(b)
                if relu:
                    cc.conv_relu_backward_x(y, g, k, gx, d, block_size=bs)
                    cc.conv_relu_backward_k(y, g, x, gk, d, block_size=bs)
                    cc.conv_relu_backward_bias(y, g, gb, block_size=bs)
                else:
                    cc.conv_backward_x(g, k, gx, d, block_size=bs)
                    cc.conv_backward_k(g, x, gk, d, block_size=bs)
                    cc.conv_backward_bias(g, gb, block_size=bs)
                torch.cuda.synchronize()
                out[tag + "_y"] = y.cpu().numpy()
                out[tag + "_gx"] = gx.cpu().numpy()
                out[tag + "_gk"] = gk.cpu().numpy()
                out[tag + "_gb"] = gb.cpu().numpy()
    np.savez_compressed(os.path.join(outdir, "ref_cuda_ops.npz"), **out)

    out = {}
    for case in cases.BLOCK_CASES:
        name, B, c_in, depth, width, sp, dil = case
        a = cases.block_inputs(case)
        nd = len(sp)
        bs = blocks(nd)
        for dt, dtag in ((torch.float64, ""), (torch.float32, "_f32")):
            x = torch.from_numpy(a["x"]).to(dev, dt)
            ws = [torch.from_numpy(w).to(dev, dt) for w in a["weights"]]
            bias = torch.from_numpy(a["bias"]).to(dev, dt)
            res = x.new_empty((B, c_in + depth * width) + tuple(sp))
            res[:, :c_in] = x
            for i in range(depth):
                n = c_in + i * width
                cc.conv_relu_forward(res[:, :n], ws[i], bias[i * width:(i + 1) * width], res[:, n:n + width], dil[i], block_size=bs)
            grads = torch.from_numpy(a["gout"]).to(dev, dt).clone()
            gb = torch.zeros_like(bias)
            for i in range(depth - 1, -1, -1):
                n = c_in + i * width
                so, sg = res[:, n:n + width], grads[:, n:n + width]
                cc.conv_relu_backward_x(so, sg, ws[i], grads[:, :n], dil[i], block_size=bs)
                gw = torch.zeros_like(ws[i])
                cc.conv_relu_backward_k(so, sg, res[:, :n], gw, dil[i], block_size=bs)
                cc.conv_relu_backward_bias(so, sg, gb[i * width:(i + 1) * width], block_size=bs)
                out[name + dtag + "_gw%d" % i] = gw.cpu().numpy()
            torch.cuda.synchronize()
            out[name + dtag + "_result"] = res.cpu().numpy()
            out[name + dtag + "_gi"] = grads[:, :c_in].cpu().numpy()
            out[name + dtag + "_gb"] = gb.cpu().numpy()
    np.savez_compressed(os.path.join(outdir, "ref_cuda_block.npz"), **out)
    print("written to", outdir)


if __name__ == "__main__":
    main(sys.argv[1] if len(sys.argv) > 1 else HERE)
