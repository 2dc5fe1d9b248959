"""Multi-GPU tests (one process per GPU, 2 / 4 / 8 ranks where the box has them): our all-reduce kernels against NCCL, the sharded
model and the expert-parallel pipelines against the single-GPU result, and a bounded peer wait that runs out without hanging
the GPU."""
import os
import subprocess
import sys
from pathlib import Path

import pytest
import torch

pytestmark = [pytest.mark.gpu, pytest.mark.multigpu]
ROOT = Path(__file__).resolve().parents[1]


def _ranks(*ns):
    """Parametrisation over rank counts; counts the box cannot serve are skipped."""
    have = torch.cuda.device_count() if torch.cuda.is_available() else 0
    return pytest.mark.parametrize("nproc", [pytest.param(n, marks=pytest.mark.skipif(n > have, reason=f"needs {n} GPUs")) for n in ns])


def _torchrun(script_args, nproc=2, env=None, timeout=600):
    cmd = [sys.executable, "-m", "torch.distributed.run", "--nnodes=1", f"--nproc-per-node={nproc}", "--master-addr", "127.0.0.1",
           "--master-port", "29517", str(ROOT / "tests" / "dist_worker.py")] + script_args
    e = dict(os.environ)
    e.update(env or {})
    r = subprocess.run(cmd, capture_output=True, text=True, timeout=timeout, env=e, cwd=str(ROOT))
    assert r.returncode == 0, r.stdout[-3000:] + r.stderr[-3000:]
    return r.stdout


@_ranks(2, 4, 8)
def test_allreduce_kernels_match_nccl(nproc):
    out = _torchrun(["allreduce"], nproc)
    assert "ALLREDUCE_OK" in out, out[-2000:]


@_ranks(2, 4)
def test_sharded_model_matches_single_gpu(nproc):
    out = _torchrun(["model"], nproc)
    assert "MODEL_OK" in out, out[-2000:]


@_ranks(2, 4, 8)
def test_expert_parallel_all_to_all_matches_single_gpu(nproc):
    out = _torchrun(["a2a"], nproc)
    assert "A2A_OK" in out, out[-2000:]


@_ranks(2, 4, 8)
def test_fused_expert_pipeline_over_real_peers_equals_single_gpu_bitwise(nproc):
    out = _torchrun(["a2a_fused"], nproc)
    assert "A2A_FUSED_OK" in out, out[-2000:]


def test_gemm_reduce_scatter_and_fused_norm_all_gather_match_nccl():
    out = _torchrun(["sp"], timeout=240)
    assert "SP_OK" in out, out[-2000:]


def test_gemma_tensor_parallel_all_reduce_and_sequence_parallel_arms_match_single_gpu():
    out = _torchrun(["gemma_sp"], timeout=240)
    assert "GEMMA_SP_OK" in out, out[-2000:]


@_ranks(2, 4, 8)
def test_vocab_parallel_head_merge_kernel_matches_full_head(nproc):
    out = _torchrun(["vocab"], nproc, timeout=240)
    assert "VOCAB_OK" in out, out[-2000:]


def test_layer_pipeline_over_nccl_matches_single_gpu():
    out = _torchrun(["pp"], timeout=240)
    assert "PP_OK" in out, out[-2000:]


def test_peer_wait_times_out_with_status_and_context_survives():
    # NVLS off: a rank that leaves must not hold a multicast binding (plain peer loads only)
    out = _torchrun(["timeout"], env={"NCCL_NVLS_ENABLE": "0", "MARY_MULTIMEM": "0"})
    assert "TIMEOUT_OK" in out, out[-2000:]
