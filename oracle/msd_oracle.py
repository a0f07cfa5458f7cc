"""CPU restatement of the Mixed-Scale Dense convolution path of ahendriksen/msd_pytorch.

TEST INFRASTRUCTURE ONLY.  Only ``tests/``, ``__graft_entry__.smoke()`` and the
CPU-baseline legs of ``bench.py`` may import this file; the product package
(``msd_pytorch_b200``) never does and has no CPU path of its own.

The reference has no CPU implementation (every op rejects CPU tensors,
msd_pytorch/msd_custom_convolutions.cpp:98,131,161,226,261,296,328), so this file
restates the arithmetic of its CUDA kernels twice:

``loops_*``  plain Python/numpy loops that follow the kernels statement by
             statement (index map, tap order, the border tap flip of backward_x).
             Slow; used on small cases to pin the vectorised version.
``conv_*``   the same eight operations with the *signatures and in-place /
             accumulate semantics* of the reference's ``msd_custom_convolutions``
             module (msd_custom_convolutions.cpp:343-369), written with torch CPU
             ops: an index gather with the edge-inclusive reflection map, an
             unpadded dilated ``F.conv{2,3}d``, ReLU, and the explicit adjoints.
``msd_block_forward / msd_block_backward``
             the dense block over ONE in-place channel buffer
             (msd_pytorch/msd_block.py:8-134).

Parity pin: checked in ``tests/test_oracle.py`` against every invariant the
reference's own tests hold for this path (interior equals a zero-padded torch
convolution, adjoint identities, bias sums, gradcheck, all-zero known answers)
and against golden vectors produced by the reference's own CUDA kernels on a
B200 (``tests/golden/ref_cuda_*.npz``, made by ``tests/golden/make_golden_ref_cuda.py``).
"""
import numpy as np
import torch
import torch.nn.functional as F


# --------------------------------------------------------------------------- #
# Index map                                                                    #
# --------------------------------------------------------------------------- #
def reflect(i, n):
    """Edge-inclusive ("symmetric") reflection: -k -> k-1, n-1+k -> n-k.

    Follows msd_pytorch/msd_custom_convolutions/kernel_utils.cuh:30-38.  One
    reflection suffices because the ops require dilation <= size
    (msd_custom_convolutions.cpp:39-52).
    """
    if i < 0:
        return -i - 1
    if i >= n:
        return 2 * n - i - 1
    return i


def reflect_indices(n, d):
    """Source index of every position of the virtually padded axis [-d, n+d)."""
    return np.array([reflect(i, n) for i in range(-d, n + d)], dtype=np.int64)


# --------------------------------------------------------------------------- #
# Loop restatements (numpy, float64 unless told otherwise)                     #
# --------------------------------------------------------------------------- #
def _taps(ndim):
    r = (-1, 0, 1)
    if ndim == 2:
        return [(p, q) for p in r for q in r]
    return [(o, p, q) for o in r for p in r for q in r]


def loops_conv_forward(x, k, bias, d, relu):
    """out[b,o,pos] = bias[o] + sum_c sum_taps x[b,c,refl(pos+d*tap)] * k[o,c,tap].

    Follows conv2d_forward.cu:143-173 and conv3d_forward.cu:160-195 (channel-then-tap
    accumulation order starting from the bias; ReLU is ``max(0, o)``).
    """
    x = np.asarray(x)
    k = np.asarray(k)
    B, C = x.shape[:2]
    sp = x.shape[2:]
    nd = len(sp)
    O = k.shape[0]
    out = np.zeros((B, O) + sp, dtype=x.dtype)
    taps = _taps(nd)
    for b in range(B):
        for o in range(O):
            for pos in np.ndindex(*sp):
                acc = x.dtype.type(bias[o])
                for c in range(C):
                    for t in taps:
                        src = tuple(reflect(pos[a] + d * t[a], sp[a]) for a in range(nd))
                        kidx = tuple(ti + 1 for ti in t)
                        acc = acc + x[(b, c) + src] * k[(o, c) + kidx]
                out[(b, o) + pos] = max(x.dtype.type(0), acc) if relu else acc
    return out


def loops_conv_backward_x(gout, k, d, out=None):
    """Input gradient in the reference's gather form, including its border tap flip.

    gin[b,c,pos] = sum_o sum_taps gate * gout[b,o,refl(pos-d*tap)] * k[o,c,flip(tap)]
    where, per axis, tap index 2 becomes 0 when pos < d and tap index 0 becomes 2
    when size <= pos + d (conv2d_backward_x.cu:56-71,153-207;
    conv3d_backward_x.cu:60-82,171-240).  ``out`` (the ReLU output) enables the
    gate ``out[b,o,neighbour] > 0`` (conv2d_backward_x.cu:197).
    Returns the gradient (the caller adds it to its buffer).
    """
    gout = np.asarray(gout)
    k = np.asarray(k)
    B, O = gout.shape[:2]
    sp = gout.shape[2:]
    nd = len(sp)
    C = k.shape[1]
    gin = np.zeros((B, C) + sp, dtype=gout.dtype)
    taps = _taps(nd)
    for b in range(B):
        for c in range(C):
            for pos in np.ndindex(*sp):
                g = gout.dtype.type(0)
                for o in range(O):
                    for t in taps:
                        src = tuple(reflect(pos[a] - d * t[a], sp[a]) for a in range(nd))
                        kidx = []
                        for a in range(nd):
                            prog = [0, 1, 2]
                            if pos[a] < d:
                                prog[2] = 0
                            if sp[a] <= pos[a] + d:
                                prog[0] = 2
                            kidx.append(prog[t[a] + 1])
                        if out is None or out[(b, o) + src] > 0:
                            g = g + gout[(b, o) + src] * k[(o, c) + tuple(kidx)]
                gin[(b, c) + pos] = g
    return gin


def loops_conv_backward_k(gout, x, d, out=None):
    """gk[o,c,tap] = sum_{b,pos} x[b,c,refl(pos+d*tap)] * gout[b,o,pos] * gate(out[b,o,pos] > 0).

    Follows conv2d_backward_k.cu:89-111 and conv3d_backward_k.cu:96-121.
    """
    gout = np.asarray(gout)
    x = np.asarray(x)
    B, O = gout.shape[:2]
    sp = gout.shape[2:]
    nd = len(sp)
    C = x.shape[1]
    gk = np.zeros((O, C) + (3,) * nd, dtype=gout.dtype)
    for b in range(B):
        for c in range(C):
            for o in range(O):
                for t in _taps(nd):
                    s = gout.dtype.type(0)
                    for pos in np.ndindex(*sp):
                        if out is not None and not out[(b, o) + pos] > 0:
                            continue
                        src = tuple(reflect(pos[a] + d * t[a], sp[a]) for a in range(nd))
                        s = s + x[(b, c) + src] * gout[(b, o) + pos]
                    gk[(o, c) + tuple(ti + 1 for ti in t)] += s
    return gk


def loops_conv_backward_bias(gout, out=None):
    """gb[o] = sum_{b,pos} gout * gate (conv2d_backward_bias.cu:37-48; the non-ReLU
    form is ``grad_output.sum((0,2,3[,4]))``, msd_custom_convolutions.cpp:180-211)."""
    gout = np.asarray(gout)
    if out is not None:
        gout = gout * (np.asarray(out) > 0)
    axes = (0,) + tuple(range(2, gout.ndim))
    return gout.sum(axis=axes)


# --------------------------------------------------------------------------- #
# Vectorised torch-CPU restatement with the reference's op signatures          #
# --------------------------------------------------------------------------- #
def _index_vectors(spatial, d, device):
    return [torch.as_tensor(reflect_indices(n, d), device=device) for n in spatial]


def symmetric_pad(x, d):
    """Gather x on the virtually padded grid [-d, n+d) of every spatial axis."""
    for axis, idx in enumerate(_index_vectors(x.shape[2:], d, x.device)):
        x = x.index_select(2 + axis, idx)
    return x


def symmetric_pad_adjoint(gpad, spatial, d):
    """Adjoint of :func:`symmetric_pad`: fold the padded gradient back (index_add)."""
    for axis, idx in enumerate(_index_vectors(spatial, d, gpad.device)):
        shape = list(gpad.shape)
        shape[2 + axis] = spatial[axis]
        folded = gpad.new_zeros(shape)
        folded.index_add_(2 + axis, idx, gpad)
        gpad = folded
    return gpad


def _conv(nd):
    return F.conv2d if nd == 2 else F.conv3d


def _conv_t(nd):
    return F.conv_transpose2d if nd == 2 else F.conv_transpose3d


def _conv_weight_grad(xpad, kshape, gout, d):
    nd = gout.dim() - 2
    fn = torch.nn.grad.conv2d_weight if nd == 2 else torch.nn.grad.conv3d_weight
    return fn(xpad, kshape, gout, dilation=d)


def _check(input_like, d):
    if d <= 0 or any(d > n for n in input_like.shape[2:]):
        raise RuntimeError("Dilation must be >= 1 and not greater than the size of the image")


def conv_forward(input, kernel, bias, output, dilation, block_size=None):
    """msd_custom_convolutions.cpp:85-116; writes into ``output``."""
    _check(input, dilation)
    nd = input.dim() - 2
    output.copy_(_conv(nd)(symmetric_pad(input, dilation), kernel, bias, dilation=dilation))


def conv_relu_forward(input, kernel, bias, output, dilation, block_size=None):
    """msd_custom_convolutions.cpp:213-245; writes ``max(0, conv)`` into ``output``."""
    _check(input, dilation)
    nd = input.dim() - 2
    output.copy_(F.relu(_conv(nd)(symmetric_pad(input, dilation), kernel, bias, dilation=dilation)))


def conv_backward_x(grad_output, kernel, grad_input, dilation, block_size=None):
    """msd_custom_convolutions.cpp:118-148; ADDS to ``grad_input``
    (conv2d_backward_x.cu:103)."""
    _check(grad_output, dilation)
    nd = grad_output.dim() - 2
    gpad = _conv_t(nd)(grad_output, kernel, dilation=dilation)
    grad_input.add_(symmetric_pad_adjoint(gpad, grad_input.shape[2:], dilation))


def conv_relu_backward_x(output, grad_output, kernel, grad_input, dilation, block_size=None):
    """msd_custom_convolutions.cpp:247-281; gate is strictly ``output > 0``."""
    conv_backward_x(grad_output * (output > 0).to(grad_output.dtype), kernel, grad_input, dilation)


def conv_backward_k(grad_output, input, grad_kernel, dilation, block_size=None):
    """msd_custom_convolutions.cpp:150-178; ADDS to ``grad_kernel`` (conv2d_backward_k.cu:52)."""
    _check(input, dilation)
    grad_kernel.add_(_conv_weight_grad(symmetric_pad(input, dilation), grad_kernel.shape, grad_output.contiguous(), dilation))


def conv_relu_backward_k(output, grad_output, input, grad_kernel, dilation, block_size=None):
    """msd_custom_convolutions.cpp:283-316."""
    conv_backward_k(grad_output * (output > 0).to(grad_output.dtype), input, grad_kernel, dilation)


def conv_backward_bias(grad_output, grad_bias, block_size=None):
    """msd_custom_convolutions.cpp:180-211; ADDS the sum over batch and space."""
    axes = (0,) + tuple(range(2, grad_output.dim()))
    grad_bias.add_(grad_output.sum(axes))


def conv_relu_backward_bias(output, grad_output, grad_bias, block_size=None):
    """msd_custom_convolutions.cpp:318-338 / conv2d_backward_bias.cu:37-48."""
    conv_backward_bias(grad_output * (output > 0).to(grad_output.dtype), grad_bias)


# --------------------------------------------------------------------------- #
# The dense block (msd_pytorch/msd_block.py:8-134)                             #
# --------------------------------------------------------------------------- #
def msd_block_forward(input, dilations, bias, weights):
    """One buffer ``[B, c_in + sum(width), *spatial]``; layer i reads channels
    ``[0, n_i)`` and writes ``[n_i, n_i + width_i)`` in place (msd_block.py:30-58)."""
    widths = [w.shape[0] for w in weights]
    result = input.new_empty((input.shape[0], input.shape[1] + sum(widths)) + tuple(input.shape[2:]))
    result[:, : input.shape[1]] = input
    start, bstart = input.shape[1], 0
    for w, d in zip(weights, dilations):
        o = w.shape[0]
        conv_relu_forward(result[:, :start], w, bias[bstart : bstart + o], result[:, start : start + o], d)
        start += o
        bstart += o
    return result


def msd_block_backward(result, grad_output, dilations, bias, weights):
    """Layers in reverse over ONE gradient buffer (msd_block.py:64-134).
    Returns ``(grad_input, grad_bias, [grad_weight_i])``."""
    grad_bias = torch.zeros_like(bias)
    gradients = grad_output.clone()
    grad_weights = [None] * len(weights)
    end, bend = result.shape[1], bias.shape[0]
    for idx in range(len(weights) - 1, -1, -1):
        w = weights[idx]
        o = w.shape[0]
        start, bstart = end - o, bend - o
        sub_out, sub_gout = result[:, start:end], gradients[:, start:end]
        conv_relu_backward_x(sub_out, sub_gout, w, gradients[:, :start], dilations[idx])
        gw = torch.zeros_like(w)
        conv_relu_backward_k(sub_out, sub_gout, result[:, :start], gw, dilations[idx])
        grad_weights[idx] = gw
        conv_relu_backward_bias(sub_out, sub_gout, grad_bias[bstart:bend])
        end, bend = start, bstart
    return gradients[:, : weights[0].shape[1]], grad_bias, grad_weights


class MSDBlockOracleFunction(torch.autograd.Function):
    """Autograd wrapper so that a whole network (block + final 1x1 layer + loss)
    can be differentiated on the CPU with exactly the block arithmetic above."""

    @staticmethod
    def forward(ctx, input, dilations, bias, *weights):
        result = msd_block_forward(input, dilations, bias, weights)
        ctx.dilations = dilations
        ctx.save_for_backward(bias, result, *weights)
        return result

    @staticmethod
    def backward(ctx, grad_output):
        bias, result, *weights = ctx.saved_tensors
        gi, gb, gws = msd_block_backward(result, grad_output, ctx.dilations, bias, weights)
        return (gi, None, gb, *gws)


def msd_network_step(x, target, dilations, bias, weights, final_w, final_b, loss="mse"):
    """Forward + backward of block -> final 1x1 layer -> loss on the CPU.

    ``final_w`` is ``[c_out, C_total]``, ``final_b`` ``[c_out]`` (the reference's
    MSDFinalLayer is a Conv1d on the flattened view, msd_module.py:60-88).
    ``loss`` is "mse" (regression, msd_regression_model.py:5) or "nll"
    (LogSoftmax + NLLLoss, msd_segmentation_model.py:64-68).
    Returns ``(loss_value, result_buffer, grad_input, grad_bias, grad_weights, grad_final_w, grad_final_b)``.
    """
    bias = bias.detach().clone().requires_grad_(True)
    weights = [w.detach().clone().requires_grad_(True) for w in weights]
    final_w = final_w.detach().clone().requires_grad_(True)
    final_b = final_b.detach().clone().requires_grad_(True)
    x = x.detach().clone().requires_grad_(True)
    result = MSDBlockOracleFunction.apply(x, list(dilations), bias, *weights)
    B, C = result.shape[:2]
    flat = result.reshape(B, C, -1)
    out = torch.einsum("oc,bcv->bov", final_w, flat) + final_b[None, :, None]
    out = out.reshape((B, final_w.shape[0]) + tuple(result.shape[2:]))
    if loss == "mse":
        value = F.mse_loss(out, target)
    elif loss == "nll":
        value = F.nll_loss(F.log_softmax(out, dim=1), target)
    else:
        raise ValueError(loss)
    value.backward()
    return (
        value.detach(),
        result.detach(),
        x.grad,
        bias.grad,
        [w.grad for w in weights],
        final_w.grad,
        final_b.grad,
    )
