"""Writes ``tests/golden/oracle_*.npz``: outputs of the loop restatement of the reference's
kernels (oracle/msd_oracle.py ``loops_*``) in float64 on the seeded cases of ``cases.py``.

Run from the repository root:  python tests/golden/make_golden.py
"""
import os
import sys

import numpy as np
import torch

HERE = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, os.path.join(HERE, "..", ".."))
sys.path.insert(0, HERE)

import cases  # noqa: E402
from oracle import msd_oracle as O  # noqa: E402


def main():
    out = {}
    for case in cases.OP_CASES:
        name = case[0]
        a = cases.op_inputs(case)
        x, k, b, g, d = a["x"], a["k"], a["b"], a["g"], a["d"]
        for relu in (False, True):
            tag = name + ("_relu" if relu else "_lin")
            y = O.loops_conv_forward(x, k, b, d, relu)
            gate = y if relu else None
            out[tag + "_y"] = y
            out[tag + "_gx"] = O.loops_conv_backward_x(g, k, d, gate)
            out[tag + "_gk"] = O.loops_conv_backward_k(g, x, d, gate)
            out[tag + "_gb"] = O.loops_conv_backward_bias(g, gate)
    np.savez_compressed(os.path.join(HERE, "oracle_ops.npz"), **out)

    out = {}
    for case in cases.BLOCK_CASES:
        name = case[0]
        a = cases.block_inputs(case)
        x = torch.from_numpy(a["x"])
        ws = [torch.from_numpy(w) for w in a["weights"]]
        bias = torch.from_numpy(a["bias"])
        res = O.msd_block_forward(x, a["dilations"], bias, ws)
        gi, gb, gws = O.msd_block_backward(res, torch.from_numpy(a["gout"]), a["dilations"], bias, ws)
        out[name + "_result"] = res.numpy()
        out[name + "_gi"] = gi.numpy()
        out[name + "_gb"] = gb.numpy()
        for i, gw in enumerate(gws):
            out[name + "_gw%d" % i] = gw.numpy()
    np.savez_compressed(os.path.join(HERE, "oracle_block.npz"), **out)
    print("written")


if __name__ == "__main__":
    main()
