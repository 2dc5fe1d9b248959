"""LoRA training on the GPU: the frozen-GEMM autograd path, the fused AdamW kernel and the q4/q8 matvec kernels."""
import numpy as np
import pytest
import torch

pytestmark = pytest.mark.gpu


def test_fused_adamw_matches_reference_formula():
    from mary_b200.train.trainer import FlatAdamW
    torch.manual_seed(0)
    p = torch.nn.Parameter(torch.randn(1000, device="cuda"))
    q = torch.nn.Parameter(p.detach().cpu().clone())
    a, b = FlatAdamW([p], lr=1e-2), FlatAdamW([q], lr=1e-2)
    for _ in range(5):
        g = torch.randn(1000)
        p.grad.copy_(g.cuda())
        q.grad.copy_(g)
        a.step(0.5)
        b.step(0.5)
    assert torch.allclose(p.detach().cpu(), q.detach(), atol=1e-6)


def test_lora_training_step_on_gpu_reduces_loss_and_matches_cpu_gradients():
    from mary_b200.models.gemma4 import Gemma4Model, Gemma4TextConfig
    from mary_b200.models.gemma4.weights import init_random_
    from mary_b200.train.lora import Gemma4LoraForward, LoraWeights
    from mary_b200.train.trainer import LoraTrainer
    cfg = Gemma4TextConfig(hidden_size=256, num_hidden_layers=2, num_attention_heads=4, num_key_value_heads=2, head_dim=64,
                           intermediate_size=512, vocab_size=512, sliding_window=16)
    gpu = Gemma4Model(cfg, dtype=torch.bfloat16, device="cuda")
    init_random_(gpu, 0, std=0.05)
    cpu = Gemma4Model(cfg, dtype=torch.float32)
    cpu.load_state_dict({k: v.float().cpu() for k, v in gpu.state_dict().items()}, strict=False)
    ids = torch.randint(0, 512, (2, 48))
    grads = []
    master = LoraWeights.init_gemma4(cpu, rank=8, seed=3)
    for a in master.adapters.values():
        a.B.data.normal_(0, 0.02, generator=torch.Generator().manual_seed(1))
    for m, dev in ((cpu, "cpu"), (gpu, "cuda")):
        lw = LoraWeights.init_gemma4(m, rank=8, seed=3)
        lw.load_state_dict({k: v.to(dev) for k, v in master.state_dict().items()})   # same adapters on both devices
        loss = Gemma4LoraForward(m, lw).loss(ids.to(dev))
        loss.backward()
        grads.append((float(loss.detach()), lw.get(1, "q_proj").B.grad.float().cpu(), lw.get(0, "down_proj").A.grad.float().cpu()))
    assert abs(grads[0][0] - grads[1][0]) < 0.05 * abs(grads[0][0])
    for i in (1, 2):                              # bf16 activations: directions agree
        cos = torch.nn.functional.cosine_similarity(grads[0][i].flatten(), grads[1][i].flatten(), dim=0)
        assert cos > 0.9, cos
    tr = LoraTrainer(gpu, rank=8, alpha=16.0, lr=5e-3)
    losses = [tr.step(ids.cuda()) for _ in range(40)]
    assert losses[-1] < 0.7 * losses[0], (losses[0], losses[-1])
    from mary_b200.ops import cuda
    assert cuda.last_status() == 0


def test_q4_q8_bf16_matvec_kernels():
    from mary_b200.nn.q4 import QLinear
    rng = np.random.default_rng(0)
    w = rng.standard_normal((2 * 264, 1024)).astype(np.float32) * 0.05
    x = torch.randn(1024).bfloat16()
    for fmt in ("q4", "q8", "bf16"):
        for sw in (False, True):
            lin_c, lin_g = QLinear(w, fmt, "cpu", swiglu=sw), QLinear(w, fmt, "cuda", swiglu=sw)
            want, got = lin_c(x).float(), lin_g(x.cuda()).float().cpu()
            assert (got - want).abs().max() < 2e-2 * want.abs().max() + 1e-3, (fmt, sw)
