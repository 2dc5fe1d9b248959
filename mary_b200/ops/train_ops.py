"""Differentiable building blocks of the LoRA fine-tuning step, each with a forward AND a backward kernel of this package
(``csrc/kernels/train.cu``) and a plain PyTorch branch for CPU tensors, so that the same modules are checked against torch
autograd without a GPU.

* ``rmsnorm(x, w, res=None, alpha=1.0)``      ``(res + x * rstd(x) * w) * alpha``; the gain is frozen (no gradient to it)
* ``geglu(gu)``                               ``gelu_tanh(gu[:, :F]) * gu[:, F:]``
* ``qkv_norm_rope(qkv, pos, ...)``            per-head RMS norm (q, k with gains, v without), split-half rotation of q and k
* ``LoraLinear``                              frozen base weight with rank-r adapters on row ranges, folded into the base GEMMs:
  ``y = [x | s u] [W | B]^T`` with ``u = x A^T`` (one GEMM with 16 extra K columns per adapter instead of a second full-width
  GEMM and an add), ``dx = [dy | s dy B] [W^T | A^T]^T`` likewise, and the weight gradients ``dA = (s dy B)^T x``,
  ``dB = dy^T (s u)`` by a kernel that streams the activations once.

Reference: the training loop ``src/bin/gemma_train_lora.rs:259-319`` and the adapter math ``src/models/gemma/lora.rs:413-428``
(there through burn's autodiff over separate ops in f32).

Wide buffers: ``wide(rows, cols, extra)`` allocates ``[rows, cols + extra]`` and returns the ``[:, :cols]`` view; an op that is
given ``out_extra=r`` writes its result into such a view, and ``LoraLinear`` recognises the view and uses the spare columns for
``s u`` (forward) or ``s dy B`` (backward) instead of copying its input."""
from __future__ import annotations

import torch

from ..utils.canary import empty as _empty
from .cuda import _p, _stream, check, declare, lib

declare("mary_rmsnorm_train_fwd", "plpplffplli" + "s")
declare("mary_rmsnorm_train_bwd", "plplpffplplli" + "s")
declare("mary_geglu_train_fwd", "plplli" + "s")
declare("mary_geglu_train_bwd", "plplplli" + "s")
declare("mary_qkv_norm_rope_train", "plplppppfpliiili" + "s")
declare("mary_lora_wgrad_splits", "iii")
declare("mary_lora_wgrad", "plpliiipp" + "s")
declare("mary_softcap_ce", "plpliffp" + "s")


def wide(rows: int, cols: int, extra: int, like) -> torch.Tensor:
    """``[rows, cols]`` view of a fresh ``[rows, cols + extra]`` buffer."""
    return _empty(rows, cols + extra, dtype=like.dtype, device=like.device)[:, :cols]


def _wide_base(t: torch.Tensor, extra: int):
    """The ``[rows, cols + extra]`` buffer that ``t`` is the leading-columns view of, or None."""
    b = t._base
    if extra and b is not None and b.dim() == 2 and t.dim() == 2 and t.storage_offset() == b.storage_offset() and t.stride(1) == 1 \
            and b.stride(1) == 1 and t.stride(0) == b.stride(0) and b.shape[0] == t.shape[0] and b.shape[1] == t.shape[1] + extra \
            and b.stride(0) == b.shape[1]:
        return b
    return None


def _rows(x):
    """2-D view with unit inner stride (a copy only when the layout demands one)."""
    x2 = x.reshape(-1, x.shape[-1])
    return x2 if x2.stride(1) == 1 else x2.contiguous()


# --------------------------------------------------------------------------------------------------------------- RMS norm
class _RmsNorm(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x, w, res, alpha, eps, out_extra):
        x2 = _rows(x)
        ctx.save_for_backward(x2, w)
        ctx.alpha, ctx.eps, ctx.shape, ctx.has_res = alpha, eps, x.shape, res is not None
        rows, H = x2.shape
        if x2.is_cuda:
            out = wide(rows, H, out_extra, x2)
            r2 = _rows(res) if res is not None else None
            check(lib().mary_rmsnorm_train_fwd(_p(x2), x2.stride(0), _p(w), _p(r2), r2.stride(0) if r2 is not None else 0, alpha, eps, _p(out),
                                               out.stride(0), rows, H, _stream()), "rmsnorm_train_fwd")
        else:
            xf = x2.float()
            y = xf * torch.rsqrt(xf.pow(2).mean(-1, keepdim=True) + eps)
            if w is not None:
                y = y * w.float()
            if res is not None:
                y = y + _rows(res).float()
            out = wide(rows, H, out_extra, x2)
            out.copy_(y * alpha)
        return out if out_extra else out.view(x.shape)

    @staticmethod
    def backward(ctx, dy):
        x2, w = ctx.saved_tensors
        rows, H = x2.shape
        d2 = _rows(dy)
        alpha = ctx.alpha
        if x2.is_cuda:
            dx = _empty(rows, H, dtype=x2.dtype, device=x2.device)
            dres = None
            if ctx.has_res:
                dres = d2 if alpha == 1.0 else _empty(rows, H, dtype=x2.dtype, device=x2.device)
            wr = dres if (dres is not None and dres is not d2) else None
            check(lib().mary_rmsnorm_train_bwd(_p(d2), d2.stride(0), _p(x2), x2.stride(0), _p(w), alpha, ctx.eps, _p(dx), dx.stride(0), _p(wr),
                                               wr.stride(0) if wr is not None else 0, rows, H, _stream()), "rmsnorm_train_bwd")
        else:
            xf, g = x2.float(), d2.float() * alpha
            dres = g.to(x2.dtype) if ctx.has_res else None
            if w is not None:
                g = g * w.float()
            rstd = torch.rsqrt(xf.pow(2).mean(-1, keepdim=True) + ctx.eps)
            xh = xf * rstd
            dx = (rstd * (g - xh * (g * xh).mean(-1, keepdim=True))).to(x2.dtype)
        return dx.view(ctx.shape), None, (dres.reshape(ctx.shape) if dres is not None else None), None, None, None


def rmsnorm(x, w=None, eps: float = 1e-6, res=None, alpha: float = 1.0, out_extra: int = 0):
    """``(res + x * rstd(x) * w) * alpha`` over the last dimension.  With ``out_extra`` the result is 2-D and sits in a wide
    buffer (see the module text)."""
    return _RmsNorm.apply(x, w.detach() if w is not None else None, res, float(alpha), float(eps), int(out_extra))


# --------------------------------------------------------------------------------------------------------------- GeGLU
def _gelu_tanh_grad(g):
    k0, k1 = 0.7978845608028654, 0.044715
    t = torch.tanh(k0 * (g + k1 * g ** 3))
    return 0.5 * g * (1 + t), 0.5 * (1 + t) + 0.5 * g * (1 - t * t) * k0 * (1 + 3 * k1 * g * g)


class _GeGlu(torch.autograd.Function):
    @staticmethod
    def forward(ctx, gu, out_extra, grad_extra):
        g2 = _rows(gu)
        ctx.save_for_backward(g2)
        ctx.shape, ctx.grad_extra = gu.shape, grad_extra
        rows, F2 = g2.shape
        F = F2 // 2
        out = wide(rows, F, out_extra, g2)
        if g2.is_cuda:
            check(lib().mary_geglu_train_fwd(_p(g2), g2.stride(0), _p(out), out.stride(0), rows, F, _stream()), "geglu_train_fwd")
        else:
            out.copy_(torch.nn.functional.gelu(g2[:, :F].float(), approximate="tanh") * g2[:, F:].float())
        return out if out_extra else out.view(*gu.shape[:-1], F)

    @staticmethod
    def backward(ctx, dout):
        (g2,) = ctx.saved_tensors
        rows, F2 = g2.shape
        F = F2 // 2
        d2 = _rows(dout)
        dgu = wide(rows, F2, ctx.grad_extra, g2)
        if g2.is_cuda:
            check(lib().mary_geglu_train_bwd(_p(d2), d2.stride(0), _p(g2), g2.stride(0), _p(dgu), dgu.stride(0), rows, F, _stream()),
                  "geglu_train_bwd")
        else:
            val, grad = _gelu_tanh_grad(g2[:, :F].float())
            df = d2.float()
            dgu[:, :F].copy_(df * g2[:, F:].float() * grad)
            dgu[:, F:].copy_(df * val)
        return (dgu if ctx.grad_extra else dgu.view(ctx.shape)), None, None


def geglu(gu, out_extra: int = 0, grad_extra: int = 0):
    """``gelu_tanh(gate) * up`` over ``gu = [gate | up]``.  ``grad_extra``: the gradient with respect to ``gu`` is produced in a
    wide buffer with that many spare columns (for the linear layer that made ``gu``); ``gu`` must then be 2-D."""
    return _GeGlu.apply(gu, int(out_extra), int(grad_extra))


# --------------------------------------------------------------------------------------------------------------- q | k | v
def _rope_cpu(x, pos, inv_freq, transpose=False):
    ang = pos.float()[:, None] * inv_freq[None, :]
    cos, sin = ang.cos()[:, None, :], ang.sin()[:, None, :]
    if transpose:
        sin = -sin
    d = x.shape[-1] // 2
    x1, x2 = x[..., :d], x[..., d:]
    return torch.cat([x1 * cos - x2 * sin, x1 * sin + x2 * cos], -1)


class _QkvNormRope(torch.autograd.Function):
    @staticmethod
    def forward(ctx, qkv, pos, inv_freq, qw, kw, eps, n_q, n_kv, D, grad_extra):
        x2 = _rows(qkv)
        rows = x2.shape[0]
        heads = n_q + 2 * n_kv
        assert x2.shape[1] == heads * D
        p32 = pos.to(torch.int32)
        ctx.save_for_backward(x2, p32, inv_freq, qw, kw)
        ctx.cfg = (eps, n_q, n_kv, D, grad_extra, qkv.shape)
        out = _empty(rows, heads * D, dtype=x2.dtype, device=x2.device)
        if x2.is_cuda:
            check(lib().mary_qkv_norm_rope_train(_p(x2), x2.stride(0), None, 0, _p(p32), _p(inv_freq), _p(qw), _p(kw), eps, _p(out), out.stride(0),
                                                 n_q, n_kv, D, rows, 0, _stream()), "qkv_norm_rope_fwd")
        else:
            xf = x2.float().view(rows, heads, D)
            y = xf * torch.rsqrt(xf.pow(2).mean(-1, keepdim=True) + eps)
            y[:, :n_q] *= qw.float()
            y[:, n_q:n_q + n_kv] *= kw.float()
            y = y.to(x2.dtype).float()
            y[:, :n_q + n_kv] = _rope_cpu(y[:, :n_q + n_kv], p32, inv_freq)
            out.copy_(y.view(rows, -1))
        return out

    @staticmethod
    def backward(ctx, dout):
        x2, p32, inv_freq, qw, kw = ctx.saved_tensors
        eps, n_q, n_kv, D, grad_extra, shape = ctx.cfg
        rows = x2.shape[0]
        heads = n_q + 2 * n_kv
        d2 = _rows(dout)
        dx = wide(rows, heads * D, grad_extra, x2)
        if x2.is_cuda:
            check(lib().mary_qkv_norm_rope_train(_p(d2), d2.stride(0), _p(x2), x2.stride(0), _p(p32), _p(inv_freq), _p(qw), _p(kw), eps, _p(dx),
                                                 dx.stride(0), n_q, n_kv, D, rows, 1, _stream()), "qkv_norm_rope_bwd")
        else:
            g = d2.float().view(rows, heads, D).clone()
            g[:, :n_q + n_kv] = _rope_cpu(g[:, :n_q + n_kv], p32, inv_freq, transpose=True)
            g[:, :n_q] *= qw.float()
            g[:, n_q:n_q + n_kv] *= kw.float()
            xf = x2.float().view(rows, heads, D)
            rstd = torch.rsqrt(xf.pow(2).mean(-1, keepdim=True) + eps)
            xh = xf * rstd
            dx.copy_((rstd * (g - xh * (g * xh).mean(-1, keepdim=True))).view(rows, -1))
        return (dx if grad_extra else dx.view(shape)), None, None, None, None, None, None, None, None, None


def qkv_norm_rope(qkv, pos, inv_freq, q_gain, k_gain, eps: float, n_q: int, n_kv: int, D: int, grad_extra: int = 0):
    """Rows ``[q heads | k heads | v heads] x D`` of a fused projection: RMS norm per head (q and k with their gains, v without),
    then the split-half rotation of the q and k heads at ``pos``.  Returns ``[rows, (n_q + 2 n_kv) * D]``."""
    return _QkvNormRope.apply(qkv, pos, inv_freq, q_gain.detach(), k_gain.detach(), float(eps), n_q, n_kv, D, int(grad_extra))


# --------------------------------------------------------------------------------------------------------------- adapters
def _mm(x, w, out=None, alpha: float = 1.0):
    """``alpha * x @ w^T``; ``x`` and ``out`` may be column slices of wider buffers."""
    if x.is_cuda:
        from . import cuda as K
        return K.gemm(x, w, out=out, alpha=alpha)
    r = (x.float() @ w.float().t()) * alpha
    if out is None:
        return r.to(x.dtype)
    out.copy_(r)
    return out


def lora_wgrad(small, big):
    """``small[M, R]^T @ big[M, C]`` in f32: the adapter weight gradients, streaming ``big`` once per 48 columns of ``small``."""
    M, R = small.shape
    C = big.shape[1]
    if not small.is_cuda:
        return small.float().t() @ big.float()
    out = _empty(R, C, dtype=torch.float32, device=small.device)
    for g in range(0, R, 48):
        n = min(48, R - g)
        splits = lib().mary_lora_wgrad_splits(M, C, n)
        ws = _empty(splits, n, C, dtype=torch.float32, device=small.device)
        sg = small[:, g:g + n]
        check(lib().mary_lora_wgrad(_p(sg), sg.stride(0), _p(big), big.stride(0), M, n, C, _p(ws), _p(out[g:g + n]), _stream()), "lora_wgrad")
    return out


class LoraLinear:
    """Frozen ``w [N, K]`` with adapters ``(A [r, K], B [n_j, r])`` on the row ranges ``(row0_j, n_j)`` of the output.

    Holds the widened operands: ``wf [N, K + R]`` = ``[W | B blocks]`` for the forward GEMM, ``wb [K, N + R]`` = ``[W^T | A^T]``
    for the input-gradient GEMM, ``a16 [R, K]`` and ``bt [R, N]`` for the two thin GEMMs (``R`` = r x number of adapters, rounded up to a multiple of 8).  The
    adapter columns are refreshed from the f32 master parameters by ``refresh()`` (once per step, after the optimiser).  A wide
    buffer (module text) serves ONE ``LoraLinear``: its spare columns are this layer's ``s u``."""

    def __init__(self, w: torch.Tensor, adapters, scale: float):
        self.N, self.K = w.shape
        self.adapters = [(ad, int(r0), int(n)) for ad, r0, n in adapters if ad is not None]
        self.scale = float(scale)
        self.r = self.adapters[0][0].A.shape[0] if self.adapters else 0
        self.R = (self.r * len(self.adapters) + 7) // 8 * 8          # spare columns: 16-byte row pitches; the padding stays zero
        N, K, R = self.N, self.K, self.R
        wd = w.detach()
        self.wf = torch.zeros(N, K + R, dtype=wd.dtype, device=wd.device)
        self.wf[:, :K].copy_(wd)
        self.wb = torch.zeros(K, N + R, dtype=wd.dtype, device=wd.device)
        self.wb[:, :N].copy_(wd.t())
        self.a16 = torch.zeros(max(R, 1), K, dtype=wd.dtype, device=wd.device)
        self.bt = torch.zeros(max(R, 1), N, dtype=wd.dtype, device=wd.device)
        self.refresh()

    def base_view(self) -> torch.Tensor:
        """The base weight as a view of the widened forward operand (lets the owner drop its own copy)."""
        return self.wf[:, :self.K]

    @torch.no_grad()
    def refresh(self):
        r, N, K = self.r, self.N, self.K
        for j, (ad, r0, n) in enumerate(self.adapters):
            self.a16[j * r:(j + 1) * r].copy_(ad.A)
            self.wb[:, N + j * r:N + (j + 1) * r].copy_(ad.A.t())
            self.wf[r0:r0 + n, K + j * r:K + (j + 1) * r].copy_(ad.B)
            self.bt[j * r:(j + 1) * r, r0:r0 + n].copy_(ad.B.t())

    def __call__(self, x, grad_extra: int = 0):
        """``x [..., K]`` (or the view of a wide buffer with ``R`` spare columns) -> ``[..., N]``.  ``grad_extra``: the gradient
        with respect to ``x`` is produced in a wide buffer with that many spare columns."""
        params = [p for ad, _, _ in self.adapters for p in (ad.A, ad.B)]
        return _LoraLinearFn.apply(x, self, grad_extra, *params)


class _LoraLinearFn(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x, mod, grad_extra, *params):
        K, N, R = mod.K, mod.N, mod.R
        x2 = _rows(x)
        M = x2.shape[0]
        xe = _wide_base(x2, R) if R else None
        if R and xe is None:
            xe = _empty(M, K + R, dtype=x2.dtype, device=x2.device)
            xe[:, :K].copy_(x2)
        if R:
            _mm(xe[:, :K], mod.a16, out=xe[:, K:], alpha=mod.scale)            # s u = s x A^T into the spare columns
            y = _mm(xe, mod.wf)                                                # x W^T + (s u) B^T
            ctx.save_for_backward(xe)
        else:
            y = _mm(x2, mod.wf)
        ctx.mod, ctx.shape, ctx.grad_extra = mod, x.shape, grad_extra
        return y if x.dim() == 2 else y.view(*x.shape[:-1], N)

    @staticmethod
    def backward(ctx, dy):
        mod = ctx.mod
        K, N, R, r = mod.K, mod.N, mod.R, mod.r
        d2 = _rows(dy)
        M = d2.shape[0]
        dx = wide(M, K, ctx.grad_extra, d2)
        if not R:
            _mm(d2, mod.wb, out=dx)
            return ((dx if ctx.grad_extra else dx.view(ctx.shape)), None, None)
        (xe,) = ctx.saved_tensors
        de = _wide_base(d2, R)
        if de is None:
            de = _empty(M, N + R, dtype=d2.dtype, device=d2.device)
            de[:, :N].copy_(d2)
        _mm(de[:, :N], mod.bt, out=de[:, N:], alpha=mod.scale)                 # dL/du = s dy B into the spare columns
        _mm(de, mod.wb, out=dx)                                                # dy W + (dL/du) A
        dA = lora_wgrad(de[:, N:], xe[:, :K])                                  # [R, K]
        dBt = lora_wgrad(xe[:, K:], de[:, :N])                                 # [R, N] = (s u)^T dy
        grads = []
        for j, (ad, r0, n) in enumerate(mod.adapters):
            grads.append(dA[j * r:(j + 1) * r])
            grads.append(dBt[j * r:(j + 1) * r, r0:r0 + n].t())
        return ((dx if ctx.grad_extra else dx.view(ctx.shape)), None, None, *grads)


# --------------------------------------------------------------------------------------------------------------- head + loss
class _HeadLoss(torch.autograd.Function):
    """Mean soft-capped cross-entropy of ``x W^T`` against ``labels``, chunked over the rows so that the ``[rows, vocab]`` logits
    exist one chunk at a time and only in bf16: per chunk the head GEMM, ONE kernel that turns the logits into loss values and
    (in place) their gradient, and the GEMM that carries that gradient back to ``x``.  Nothing of vocabulary width is kept for
    the backward pass: the gradient with respect to ``x`` is complete when the forward returns."""

    @staticmethod
    def forward(ctx, x, w, wt, labels, cap, chunk):
        n, V = x.shape[0], w.shape[0]
        dx = torch.empty_like(x)
        total = torch.zeros((), dtype=torch.float32, device=x.device)
        lab = labels.to(torch.int64).contiguous()
        for i in range(0, n, chunk):
            xc = x[i:i + chunk]
            if x.is_cuda:
                from . import cuda as K
                lg = K.gemm(xc.contiguous(), w)
                rows = lg.shape[0]
                loss = _empty(rows, dtype=torch.float32, device=x.device)
                check(lib().mary_softcap_ce(_p(lg), lg.stride(0), _p(lab[i:i + chunk]), rows, V, float(cap or 0.0), 1.0 / n, _p(loss), _stream()),
                      "softcap_ce")
                total += loss.sum()
                K.gemm(lg, wt, out=dx[i:i + chunk])
            else:
                lg = (xc.float() @ w.float().t()).requires_grad_()
                with torch.enable_grad():
                    z = cap * torch.tanh(lg / cap) if cap and cap > 0 else lg
                    ls = torch.nn.functional.cross_entropy(z, lab[i:i + chunk], reduction="sum")
                (g,) = torch.autograd.grad(ls, lg)
                total += ls.detach()
                dx[i:i + chunk] = ((g / n) @ w.float()).to(x.dtype)
        ctx.save_for_backward(dx)
        return total / n

    @staticmethod
    def backward(ctx, g):
        (dx,) = ctx.saved_tensors
        return dx * g.to(dx.dtype), None, None, None, None, None


def head_loss(x, w, wt, labels, cap: float | None, chunk: int = 1024):
    """Mean cross-entropy of the (soft-capped) logits ``x @ w^T`` against ``labels``; ``wt = w^T`` contiguous."""
    return _HeadLoss.apply(x, w.detach(), wt, labels, float(cap or 0.0), int(chunk))
