"""Differentiable wrappers of the block ops for torch.autograd.

The reference registers its gradients in Python as compositions of the same ops
(``benchmark/sparse_conv_lib.py:80-147``, ``sbnet_ops/tests/test_sparse_blocks.py:36-98``):

* d(sparse_gather)/dx      = sparse_scatter(grad, ..., zeros_like(x), add=True, atomic=True)
* d(sparse_scatter)/dx     = sparse_gather(grad, ...)
* d(sparse_scatter)/dybase = grad                       (add=True)
                           = grad with the scattered pixels stamped out   (add=False)

Two differences from the reference, both deliberate: the scatter gradient passes ``transpose`` on to
the gather (the reference drops it, so its gradient has the wrong layout for transposed stacks), and
the stamp-out for ``add=False`` overwrites the scattered pixels of a copy of ``grad`` with zeros
directly instead of building a ones/zeros mask and multiplying.
All heavy lifting happens in the CUDA library; nothing here computes on tensors itself except
allocating the zero base.
"""
from __future__ import annotations

import torch

from . import ops


class _SparseGather(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x, bin_counts, indices, bsize, bstride, boffset, transpose):
        ctx.save_for_backward(indices)
        ctx.meta = (int(bin_counts.reshape(-1)[0]), tuple(bsize), tuple(bstride), tuple(boffset),
                    bool(transpose), x.shape, x.dtype)
        return ops.sparse_gather(x, bin_counts, indices, bsize, bstride, boffset, transpose=transpose)

    @staticmethod
    def backward(ctx, grad):
        (indices,) = ctx.saved_tensors
        nb, bsize, bstride, boffset, transpose, shape, dtype = ctx.meta
        base = torch.zeros(shape, dtype=dtype, device=grad.device)
        gx = ops.sparse_scatter_var(grad.contiguous(), [nb], indices, base, bsize, bstride, boffset,
                                    add=True, atomic=True, transpose=transpose)
        return gx, None, None, None, None, None, None


class _SparseScatter(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x, bin_counts, indices, ybase, bsize, bstride, boffset, add, atomic, transpose):
        ctx.save_for_backward(indices)
        ctx.meta = (int(bin_counts.reshape(-1)[0]), tuple(bsize), tuple(bstride), tuple(boffset),
                    bool(add), bool(transpose), x.shape)
        return ops.sparse_scatter(x, bin_counts, indices, ybase, bsize, bstride, boffset, add=add,
                                  atomic=atomic, transpose=transpose)

    @staticmethod
    def backward(ctx, grad):
        (indices,) = ctx.saved_tensors
        nb, bsize, bstride, boffset, add, transpose, xshape = ctx.meta
        grad = grad.contiguous()
        gx = ops.sparse_gather(grad, [nb], indices, bsize, bstride, boffset, transpose=transpose)
        if add:
            gbase = grad
        else:   # scattered pixels do not depend on ybase: zero them in a copy of grad
            zeros = torch.zeros(xshape, dtype=grad.dtype, device=grad.device)
            gbase = ops.sparse_scatter(zeros, [nb], indices, grad, bsize, bstride, boffset, add=False,
                                       transpose=transpose)
        return gx, None, None, gbase, None, None, None, None, None, None


def sparse_gather(x, bin_counts, active_block_indices, dynamic_bsize, dynamic_bstride, dynamic_boffset,
                  transpose=False):
    """Differentiable ``SparseGather`` (gradient flows to ``x``)."""
    return _SparseGather.apply(x, bin_counts, active_block_indices, dynamic_bsize, dynamic_bstride,
                               dynamic_boffset, transpose)


def sparse_scatter(x, bin_counts, active_block_indices, ybase, dynamic_bsize, dynamic_bstride,
                   dynamic_boffset, add, atomic=False, transpose=False):
    """Differentiable ``SparseScatter`` (gradients flow to the block stack ``x`` and to ``ybase``)."""
    return _SparseScatter.apply(x, bin_counts, active_block_indices, ybase, dynamic_bsize,
                                dynamic_bstride, dynamic_boffset, add, atomic, transpose)
