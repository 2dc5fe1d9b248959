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
