"""Forward and backward of the training-path ops (``ops/train_ops.py``: one forward and one backward kernel each) against torch
autograd over the plain f32 formulas; on CPU the same tests exercise the PyTorch branch of every op."""
import pytest
import torch

from mary_b200.ops import reference as ref
from mary_b200.ops import train_ops as T

DEVICES = ["cpu", pytest.param("cuda", marks=pytest.mark.gpu)]


def _setup(device):
    dt = torch.bfloat16 if device == "cuda" else torch.float32
    tol = 2e-2 if device == "cuda" else 1e-5
    return dt, tol


def _close(a, b, tol):
    a, b = a.float(), b.float()
    err = (a - b).abs().max().item() / (b.abs().max().item() + 1e-12)
    assert err < tol, err


@pytest.mark.parametrize("device", DEVICES)
@pytest.mark.parametrize("H,use_w,use_res,alpha", [(3840, True, False, 1.0), (512, True, True, 0.7), (264, False, True, 1.0)])
def test_rmsnorm_forward_and_backward(device, H, use_w, use_res, alpha):
    dt, tol = _setup(device)
    torch.manual_seed(H)
    x = torch.randn(37, H, device=device).to(dt).requires_grad_()
    res = torch.randn(37, H, device=device).to(dt).requires_grad_() if use_res else None
    w = (1 + 0.1 * torch.randn(H, device=device)).to(dt) if use_w else None
    y = T.rmsnorm(x, w, 1e-6, res=res, alpha=alpha, out_extra=16)
    assert y._base is not None and y._base.shape == (37, H + 16)
    dy = torch.randn(37, H, device=device).to(dt)
    y.backward(dy)
    xf = x.detach().float().requires_grad_()
    rf = res.detach().float().requires_grad_() if use_res else None
    yf = xf * torch.rsqrt(xf.pow(2).mean(-1, keepdim=True) + 1e-6)
    if use_w:
        yf = yf * w.float()
    if use_res:
        yf = yf + rf
    yf = yf * alpha
    yf.backward(dy.float())
    _close(y, yf, tol)
    _close(x.grad, xf.grad, tol)
    if use_res:
        _close(res.grad, rf.grad, tol)


@pytest.mark.parametrize("device", DEVICES)
def test_geglu_forward_and_backward(device):
    dt, tol = _setup(device)
    torch.manual_seed(1)
    gu = (2 * torch.randn(19, 2 * 1032, device=device)).to(dt).requires_grad_()
    out = T.geglu(gu, out_extra=16, grad_extra=32)
    dy = torch.randn(19, 1032, device=device).to(dt)
    out.backward(dy)
    gf = gu.detach().float().requires_grad_()
    of = torch.nn.functional.gelu(gf[:, :1032], approximate="tanh") * gf[:, 1032:]
    of.backward(dy.float())
    _close(out, of, tol)
    _close(gu.grad, gf.grad, tol)


@pytest.mark.parametrize("device", DEVICES)
@pytest.mark.parametrize("D,n_q,n_kv", [(256, 4, 2), (128, 8, 8), (512, 2, 1), (64, 4, 2)])
def test_qkv_head_norm_and_rotation_forward_and_backward(device, D, n_q, n_kv):
    dt, tol = _setup(device)
    torch.manual_seed(D)
    rows, heads = 23, n_q + 2 * n_kv
    qkv = torch.randn(rows, heads * D, device=device).to(dt).requires_grad_()
    pos = torch.randint(0, 4096, (rows,), device=device)
    inv = ref.rope_inv_freq(D, 10000.0, 0.5 if D == 512 else 1.0, device=device)
    qw = (1 + 0.1 * torch.randn(D, device=device)).to(dt)
    kw = (1 + 0.1 * torch.randn(D, device=device)).to(dt)
    out = T.qkv_norm_rope(qkv, pos, inv, qw, kw, 1e-6, n_q, n_kv, D, grad_extra=48)
    dy = torch.randn(rows, heads * D, device=device).to(dt)
    out.backward(dy)
    xf = qkv.detach().float().requires_grad_()
    x3 = xf.view(rows, heads, D)
    q = ref.rope(ref.rmsnorm(x3[:, :n_q], qw.float()), pos, inv)
    k = ref.rope(ref.rmsnorm(x3[:, n_q:n_q + n_kv], kw.float()), pos, inv)
    v = ref.rmsnorm(x3[:, n_q + n_kv:], None)
    of = torch.cat([q, k, v], 1).reshape(rows, -1)
    of.backward(dy.float())
    _close(out, of, tol)
    _close(qkv.grad, xf.grad, tol)


class _Ad:
    def __init__(self, r, fin, fout, device):
        self.A = (torch.randn(r, fin, device=device) / fin ** 0.5).requires_grad_()
        self.B = (0.05 * torch.randn(fout, r, device=device)).requires_grad_()


@pytest.mark.parametrize("device", DEVICES)
@pytest.mark.parametrize("n_ad,r", [(0, 16), (1, 16), (2, 16), (3, 16), (3, 8), (1, 4), (2, 32)])
def test_lora_linear_equals_base_plus_adapters_with_all_gradients(device, n_ad, r):
    """The widened GEMMs give ``x W^T + s (x A^T) B^T`` per row range, the input gradient and the f32 gradients of every factor;
    a wide input (made by ``rmsnorm(out_extra=R)``) and a wide output gradient (``geglu(grad_extra=R)``) are used in place."""
    dt, tol = _setup(device)
    torch.manual_seed(n_ad)
    M, K, s = 203, 520, 2.0
    ranges = [(0, 256), (256, 128), (384, 128)][:n_ad]
    N = 512
    w = (torch.randn(N, K, device=device) / K ** 0.5).to(dt)
    ads = [_Ad(r, K, n, device) for _, n in ranges]
    lin = T.LoraLinear(w, [(a, r0, n) for a, (r0, n) in zip(ads, ranges)], s)
    h = torch.randn(M, K, device=device).to(dt).requires_grad_()
    x = T.rmsnorm(h, None, 1e-6, out_extra=lin.R)
    y = lin(x, grad_extra=0)
    out = T.geglu(y, grad_extra=lin.R)
    dy = torch.randn(M, N // 2, device=device).to(dt)
    out.backward(dy)
    # plain autograd in f32 over the same (rounded) operands
    hf = h.detach().float().requires_grad_()
    xf = hf * torch.rsqrt(hf.pow(2).mean(-1, keepdim=True) + 1e-6)
    yf = xf @ w.float().t()
    Af = [a.A.detach().clone().requires_grad_() for a in ads]
    Bf = [a.B.detach().clone().requires_grad_() for a in ads]
    parts = []
    for (r0, n), A, B in zip(ranges, Af, Bf):
        parts.append((r0, n, s * (xf @ A.t()) @ B.t()))
    if parts:
        delta = torch.zeros_like(yf)
        for r0, n, d in parts:
            delta = delta + torch.nn.functional.pad(d, (r0, N - r0 - n))
        yf = yf + delta
    of = torch.nn.functional.gelu(yf[:, :N // 2], approximate="tanh") * yf[:, N // 2:]
    of.backward(dy.float())
    _close(out, of, tol)
    _close(h.grad, hf.grad, tol)
    for a, A, B in zip(ads, Af, Bf):
        assert a.A.grad.dtype == torch.float32 and a.B.grad.dtype == torch.float32
        _close(a.A.grad, A.grad, tol)
        _close(a.B.grad, B.grad, tol)
    # after an optimiser step the widened operands follow the master parameters
    if ads:
        with torch.no_grad():
            ads[0].B.add_(0.5)
        lin.refresh()
        y2 = lin(x.detach())
        want = x.detach().float() @ w.float().t()
        for (r0, n), a in zip(ranges, ads):
            want[:, r0:r0 + n] += s * (x.detach().float() @ a.A.detach().t()) @ a.B.detach().t()
        _close(y2, want, tol)


@pytest.mark.gpu
@pytest.mark.parametrize("R,C,M", [(16, 3840, 4096), (32, 1032, 517), (48, 8192, 1000), (24, 512, 100), (96, 256, 300), (8, 264, 31),
                                   (20, 512, 333), (3, 1024, 64)])
def test_adapter_weight_gradient_kernel(R, C, M):
    """Ranks that are a multiple of 8 take the tensor-core kernel (operands as column slices of one wide buffer, as the adapter
    layers pass them), the others the SIMT kernel."""
    torch.manual_seed(R)
    if R % 8 == 0:
        buf = torch.randn(M, C + R, device="cuda").bfloat16()
        small, big = buf[:, C:], buf[:, :C]
    else:
        small, big = torch.randn(M, R, device="cuda").bfloat16(), torch.randn(M, C, device="cuda").bfloat16()
    got = T.lora_wgrad(small, big)
    want = small.double().t() @ big.double()
    assert (got.double() - want).abs().max().item() < 2e-3 * want.abs().max().item()


@pytest.mark.parametrize("device", DEVICES)
@pytest.mark.parametrize("cap,V", [(30.0, 4104), (0.0, 520), (30.0, 262144)])
def test_head_loss_equals_chunked_cross_entropy_with_its_gradient(device, cap, V):
    if device == "cpu" and V > 10000:
        pytest.skip("vocabulary-sized case runs on the GPU only")
    dt, tol = _setup(device)
    torch.manual_seed(V)
    n, H = 77, 256
    x = torch.randn(n, H, device=device).to(dt).requires_grad_()
    w = (torch.randn(V, H, device=device) * 0.2).to(dt)
    y = torch.randint(0, V, (n,), device=device)
    loss = T.head_loss(x, w, w.t().contiguous(), y, cap, chunk=32)
    loss.backward()
    xf = x.detach().float().requires_grad_()
    lg = (xf @ w.float().t()).to(dt).float() if device == "cuda" else xf @ w.float().t()
    lg = cap * torch.tanh(lg / cap) if cap else lg
    want = torch.nn.functional.cross_entropy(lg, y)
    assert abs(float(loss.detach()) - float(want.detach())) < (2e-3 if device == "cuda" else 1e-5) * abs(float(want.detach()))
    if device == "cpu":
        want.backward()
        _close(x.grad, xf.grad, tol)
    else:
        # the GPU reference without the bf16 rounding of the logits (which autograd cannot see through)
        lg2 = xf @ w.float().t()
        torch.nn.functional.cross_entropy(cap * torch.tanh(lg2 / cap) if cap else lg2, y).backward()
        _close(x.grad, xf.grad, 5e-2)
