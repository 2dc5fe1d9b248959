"""Guard bands around kernel outputs (``utils/canary.py``): the check finds a write outside a buffer, and the package's kernels
leave every band intact on representative launches."""
import pytest
import torch

from mary_b200.utils import canary


@pytest.fixture
def canaries():
    canary.set_enabled(True)
    canary._live.clear()
    yield
    canary._live.clear()
    canary.set_enabled(False)


def test_guard_bands_catch_writes_before_and_after_a_buffer(canaries):
    t = canary.empty(7, 33, dtype=torch.bfloat16, what="probe")
    assert t.shape == (7, 33) and t.dtype == torch.bfloat16
    t.fill_(1.0)                                   # writing the whole extent touches no band
    assert canary.check_all() == 1
    for where in ("after", "before"):
        t = canary.empty(100, dtype=torch.float32, what=where)
        g = canary._live[-1]
        g.raw[canary.GUARD + g.n if where == "after" else canary.GUARD - 1] = 0      # the byte next to the buffer
        with pytest.raises(RuntimeError, match=where):
            canary.check_all()
        canary._live.clear()


def test_off_by_default_allocates_plainly():
    canary.set_enabled(False)
    t = canary.empty(4, 4, dtype=torch.float32)
    assert t._base is None and not canary._live


@pytest.mark.gpu
def test_kernels_write_only_inside_their_outputs(canaries):
    from mary_b200.ops import cuda, cuda_moe
    from mary_b200.ops import train_ops as T
    from mary_b200.ops.moe import NVFP4Experts
    torch.manual_seed(0)
    dev = "cuda"
    # GEMMs with ragged extents (tiles clipped in both directions), decode- and prefill-shaped
    for M, N, K in ((37, 1000, 520), (300, 264, 1032), (1, 8, 64)):
        cuda.gemm(torch.randn(M, K, device=dev).bfloat16(), torch.randn(N, K, device=dev).bfloat16())
        cuda.gemm_splitk(torch.randn(M, K, device=dev).bfloat16(), torch.randn(N, K, device=dev).bfloat16(), 0)
    # expert pipeline at both tile widths
    ex = NVFP4Experts.random(8, 512, 256, dev, std=0.05, seed=1)
    for Tn, nt in ((70, 32), (700, 128)):
        x = torch.randn(Tn, 512, device=dev).bfloat16()
        idx, w = cuda.router_topk(torch.randn(Tn, 8, device=dev), 2, "softmax")
        cuda_moe.experts_forward(x, idx, w, ex, None, nt)
    # training ops, forward and backward, with row-pitched outputs
    h = torch.randn(203, 520, device=dev).bfloat16().requires_grad_()
    ads = [type("A", (), {"A": torch.randn(16, 520, device=dev).requires_grad_(), "B": torch.randn(256, 16, device=dev).requires_grad_()})()]
    lin = T.LoraLinear(torch.randn(512, 520, device=dev).bfloat16(), [(ads[0], 0, 256)], 2.0)
    out = T.geglu(lin(T.rmsnorm(h, None, 1e-6, out_extra=lin.R)), grad_extra=lin.R)
    out.backward(torch.randn_like(out))
    qkv = torch.randn(23, 8 * 256, device=dev).bfloat16().requires_grad_()
    inv = torch.rand(128, device=dev)
    g = torch.ones(256, device=dev).bfloat16()
    T.qkv_norm_rope(qkv, torch.arange(23, device=dev), inv, g, g, 1e-6, 4, 2, 256).sum().backward()
    T.head_loss(torch.randn(50, 256, device=dev).bfloat16().requires_grad_(), torch.randn(1032, 256, device=dev).bfloat16(),
                torch.randn(256, 1032, device=dev).bfloat16(), torch.randint(0, 1032, (50,), device=dev), 30.0, chunk=32).backward()
    assert canary.check_all() > 20
    assert cuda.last_status() == 0
