"""Autograd wrappers that put the hand-written GEMM on the training path.

``linear(x, w, wt)``: forward ``x @ w^T`` with the tcgen05 GEMM; backward ``dx = dy @ w`` computed as a K-major GEMM
against ``wt = w^T`` (kept once per frozen weight — the base model takes no gradient, only activations do).  On CPU both
directions are plain matmuls, which makes the same module testable against torch autograd."""
from __future__ import annotations

import torch


class _LinearFrozen(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x, w, wt):
        ctx.save_for_backward(w, wt)
        shp = x.shape
        x2 = x.reshape(-1, shp[-1])
        if x2.is_cuda:
            from . import cuda as K
            y = K.gemm(x2.contiguous(), w)
        else:
            y = x2 @ w.t()
        return y.reshape(*shp[:-1], w.shape[0])

    @staticmethod
    def backward(ctx, dy):
        w, wt = ctx.saved_tensors
        shp = dy.shape
        d2 = dy.reshape(-1, shp[-1])
        if d2.is_cuda:
            from . import cuda as K
            dx = K.gemm(d2.contiguous(), wt)
        else:
            dx = d2 @ w
        return dx.reshape(*shp[:-1], w.shape[1]), None, None


def linear_frozen(x, w, wt=None):
    if wt is None:
        wt = w.t().contiguous()
    return _LinearFrozen.apply(x, w, wt)


def _own(t):
    """A group reduction may answer with a view of its communication buffer that the next reduction overwrites; autograd keeps
    results for the backward pass, so they get storage of their own."""
    return t.clone() if t._base is not None else t


class _CopyToTP(torch.autograd.Function):
    """Entry of a tensor-parallel region: the activation is the same on every rank and feeds every rank's weight shard, so its
    gradient is the SUM of the ranks' partial gradients (forward identity, backward all-reduce)."""

    @staticmethod
    def forward(ctx, x, tp):
        ctx.tp = tp
        return x

    @staticmethod
    def backward(ctx, dy):
        return _own(ctx.tp.all_reduce(dy.contiguous().clone())), None     # never reduce in place into autograd's buffer


class _ReduceFromTP(torch.autograd.Function):
    """Exit of a tensor-parallel region: the ranks' partial sums are reduced (forward all-reduce); the gradient of the reduced
    activation is the gradient of every partial sum (backward identity)."""

    @staticmethod
    def forward(ctx, x, tp):
        return _own(tp.all_reduce(x.contiguous().clone()))

    @staticmethod
    def backward(ctx, dy):
        return dy, None


def copy_to_tp(x, tp):
    return _CopyToTP.apply(x, tp) if tp is not None and tp.size > 1 else x


def reduce_from_tp(x, tp):
    return _ReduceFromTP.apply(x, tp) if tp is not None and tp.size > 1 else x
