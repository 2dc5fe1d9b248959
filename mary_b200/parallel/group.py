"""Parallel group used by the models: tensor-parallel attention / dense FFN and expert-parallel routed experts, both of
which leave a PARTIAL hidden state on every rank that one sum over the group completes.

``mode="nccl"`` is the library baseline (``torch.distributed.all_reduce``); ``mode="fused"`` uses this package's own
kernels over peer memory (``parallel.symm``): partial sums are written into a symmetric buffer and reduced by a
one-shot / two-shot kernel that reads the peers directly (or through the NVSwitch multicast address).
The reference has no collective at all: its only multi-device mode is a 2-stage layer pipeline over TCP
(src/bin/inkling_forward.rs:1192-1271); tensor parallelism is priced there but not built (:68-99)."""
from __future__ import annotations

import torch

from .. import ops


class ParallelGroup:
    def __init__(self, rank: int = 0, size: int = 1, mode: str = "nccl", group=None, symm=None, ep_mode: str = "replicated",
                 vocab_parallel: bool = False):
        """``ep_mode="replicated"``: tokens are replicated, attention is tensor parallel over the group and every rank adds
        the partial sums of its own experts (one reduction per block).  ``ep_mode="a2a"``: tokens stay on their home rank
        (data-parallel attention, full heads everywhere) and the routed experts are reached through the all-to-all of
        ``parallel.ep``; nothing is reduced."""
        self.rank, self.size, self.mode, self.group, self.symm = rank, size, mode, group, symm
        self.ep_mode = ep_mode
        self.vocab_parallel = vocab_parallel and ep_mode != "a2a"      # tokens must be replicated over the group
        self.tp_rank, self.tp_size = (0, 1) if ep_mode == "a2a" else (rank, size)
        self.ep_rank, self.ep_size = rank, size
        self.sp = None                  # parallel.sp.SequenceParallel: reduce-scatter / all-gather arm of the dense decoders
        self.ep_factory = None          # callable(experts, cfg) -> EPLayer, set by the launcher in a2a mode
        self.ep_decode_cap = None       # a2a mode: rows per rank the decode-sized slabs hold (larger batches take ep_prefill_cap slabs)
        self.ep_prefill_cap = None
        self.bytes_reduced = 0
        self.calls = 0

    def reduce(self, partial, residual=None):
        if self.tp_size == 1:
            return partial
        self.calls += 1
        self.bytes_reduced += partial.numel() * partial.element_size()
        if self.mode == "fused" and self.symm is not None and partial.is_cuda:
            return self.symm.all_reduce(partial)
        import torch.distributed as dist
        out = partial.contiguous()
        dist.all_reduce(out, group=self.group)
        return out

    all_reduce = reduce

    def row_linear(self, x, w, lora=None):
        """Row-parallel GEMM: the result is this rank's partial sum (the caller reduces it).  In fused mode the GEMM
        epilogue stores straight into the symmetric input region, so the reduction kernel needs no staging copy."""
        if self.tp_size > 1 and self.mode == "fused" and self.symm is not None and x.is_cuda:
            from ..ops import cuda as K
            M, N, Kd = x.shape[0], w.shape[0], x.shape[1]
            out = self.symm.input_view((M, N))
            sk = K._auto_split_k(M, N, Kd)
            if sk > 1:
                K.gemm_splitk(x.contiguous(), w, 0, out=out)
            else:
                K.gemm(x.contiguous(), w, out=out)
            if lora is not None:
                out += lora(x)
            return out
        y = ops.linear(x, w)
        return y if lora is None else y + lora(x)


def init_distributed(device_index: int | None = None):
    """``torch.distributed`` over NCCL from the torchrun environment.  Returns ``(rank, world, local_rank)``."""
    import os
    import torch.distributed as dist
    world = int(os.environ.get("WORLD_SIZE", "1"))
    rank = int(os.environ.get("RANK", "0"))
    local = int(os.environ.get("LOCAL_RANK", str(rank)))
    if torch.cuda.is_available():
        torch.cuda.set_device(local if device_index is None else device_index)
    if world > 1 and not dist.is_initialized():
        dist.init_process_group("nccl" if torch.cuda.is_available() else "gloo",
                                device_id=torch.device("cuda", local) if torch.cuda.is_available() else None)
    return rank, world, local
