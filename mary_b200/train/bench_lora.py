"""LoRA finetuning step time on the Gemma-4-12B-style decoder (rank 16, alpha 32, AdamW lr 1e-4, sequences of 4096 tokens),
data parallel over the ranks of a ``torchrun`` launch with the adapter gradients reduced per layer bucket, overlapped with
the backward pass of the earlier layers.

    python -m mary_b200.train.bench_lora [--seq 4096] [--batch 1] [--steps 5] [--layers 48] [--comm fused|nccl] [--tp T] [--checkpoint]

Prints one JSON line: tokens/s over all ranks (device time, max over ranks).  Data are synthetic token ids, weights random."""
from __future__ import annotations

import argparse
import json
import os

# a 4096-token step without activation checkpointing fills a 180 GB GPU to within a few GB: segments that can grow keep the
# caching allocator from failing on fragmentation (must be set before the first CUDA allocation)
os.environ.setdefault("PYTORCH_CUDA_ALLOC_CONF", "expandable_segments:True")

import torch  # noqa: E402


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--seq", type=int, default=4096)
    ap.add_argument("--batch", type=int, default=1, help="sequences per rank")
    ap.add_argument("--steps", type=int, default=5)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--layers", type=int, default=48)
    ap.add_argument("--comm", default="fused", choices=["fused", "nccl"])
    ap.add_argument("--no-overlap", action="store_true")
    ap.add_argument("--checkpoint", action="store_true", help="recompute each layer in the backward pass (activation checkpointing)")
    ap.add_argument("--tp", type=int, default=1, help="tensor-parallel group size; the world is (world / tp) data-parallel replicas of tp ranks each")
    ap.add_argument("--sp", action="store_true", help="sequence parallelism over all ranks: ONE sequence per step, every rank runs the layers "
                    "on its chunk of the rows, attention through all-to-alls (excludes --tp)")
    ap.add_argument("--kernel-table", action="store_true", help="after the timed steps run one more step under torch.profiler and print "
                    "the 30 kernels with the largest device time (shares only: times under a profiler are not benchmark values)")
    a = ap.parse_args()
    from ..models.gemma4 import Gemma4Model, gemma_12b_config
    from ..models.gemma4.weights import init_random_
    from ..ops import cuda as K
    from ..parallel.group import init_distributed
    from .trainer import LoraTrainer
    rank, world, local = init_distributed()
    dev = torch.device("cuda", local)
    cfg = gemma_12b_config()
    cfg.num_hidden_layers = a.layers
    cfg.layer_types = cfg.layer_types[:a.layers]
    tp = a.tp
    assert world % tp == 0, "--tp must divide the number of ranks"
    assert not (a.sp and tp > 1), "--sp and --tp are separate layouts"
    dp = 1 if a.sp else world // tp
    tp_rank, dp_rank = rank % tp, rank // tp
    reduce_fn = tp_reduce_fn = par = None
    if world > 1:
        import torch.distributed as dist
        from ..parallel.group import ParallelGroup
        tp_groups = [dist.new_group(list(range(d * tp, (d + 1) * tp))) for d in range(dp)] if 1 < tp < world else None
        dp_groups = [dist.new_group(list(range(t, world, tp))) for t in range(tp)] if 1 < tp < world else None
        heap = None
        if a.comm == "fused" and (tp == 1 or tp == world):
            # one group spans the world: this package's all-reduce kernels over peer memory carry the activations of the
            # tensor-parallel regions (bf16, one sequence batch) and the adapter gradients (f32)
            from ..parallel.symm import SymmetricHeap
            heap = SymmetricHeap(rank, world, dev, max_bytes=max(8 << 20, a.batch * a.seq * cfg.hidden_size * 4 if tp > 1 else 0))
        if tp > 1:
            if heap is not None:
                par = ParallelGroup(tp_rank, tp, "fused", symm=heap)
                # the gradient buckets are reduced on a side stream while the backward pass reduces activations: a heap of their own
                tp_reduce_fn = SymmetricHeap(rank, world, dev, max_bytes=8 << 20).all_reduce_f32_
            else:
                grp = tp_groups[dp_rank] if tp_groups else None
                par = ParallelGroup(tp_rank, tp, "nccl", group=grp)
                tp_reduce_fn = lambda g_, grp=grp: dist.all_reduce(g_, group=grp)  # noqa: E731
        if a.sp:
            reduce_fn = heap.all_reduce_f32_ if heap is not None else (lambda g_: dist.all_reduce(g_))
        elif dp > 1:
            if heap is not None and tp == 1:
                reduce_fn = heap.all_reduce_f32_
            else:
                grp = dp_groups[tp_rank] if dp_groups else None
                reduce_fn = lambda g_, grp=grp: dist.all_reduce(g_, group=grp)  # noqa: E731
    model = Gemma4Model(cfg, tp=par, dtype=torch.bfloat16, device=dev)
    init_random_(model, 0)
    tr = LoraTrainer(model, rank=16, alpha=32.0, lr=1e-4, dp_size=dp, reduce_fn=reduce_fn, tp_reduce_fn=tp_reduce_fn, overlap=not a.no_overlap,
                     checkpoint=a.checkpoint, seq_parallel=(rank, world, None) if a.sp and world > 1 else None)
    if a.sp:
        dp_rank = 0                                                         # every rank of the group works on the same sequence
    g = torch.Generator(device=dev).manual_seed(dp_rank)                    # the ranks of one tensor-parallel group see the same sequences
    ids = torch.randint(0, cfg.vocab_size, (a.batch, a.seq), device=dev, generator=g)
    for _ in range(a.warmup):
        loss = tr.step(ids)
    torch.cuda.synchronize()
    if world > 1:
        dist.barrier()
    K.LAUNCHES = 0
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    for _ in range(a.steps):
        loss = tr.step(ids)
    e1.record()
    torch.cuda.synchronize()
    ms = torch.tensor([e0.elapsed_time(e1)], dtype=torch.float64, device=dev)
    if world > 1:
        dist.all_reduce(ms, op=dist.ReduceOp.MAX)
    ms = float(ms) / a.steps
    if rank == 0:
        print(json.dumps({"metric": "LoRA finetune tokens/s (Gemma-4-12B-style, rank 16, seq %d)" % a.seq,
                          "value": round(dp * a.batch * a.seq / (ms / 1e3), 1), "unit": "tokens/s", "n_gpus": world, "parallelism": f"sp{world}" if a.sp else f"dp{dp} x tp{tp}",
                          "ms_per_step": round(ms, 2), "loss": round(loss, 4), "layers": a.layers, "comm": a.comm if world > 1 else "none",
                          "overlap": not a.no_overlap, "checkpointing": a.checkpoint, "gpu_launches_per_step": K.LAUNCHES // a.steps,
                          "peak_mem_gb": round(torch.cuda.max_memory_allocated(dev) / 2 ** 30, 1), "kernel_status": K.last_status()}))
    if a.kernel_table and rank == 0:
        from torch.profiler import ProfilerActivity, profile
        with profile(activities=[ProfilerActivity.CUDA]) as prof:
            tr.step(ids)
            torch.cuda.synchronize()
        print(prof.key_averages().table(sort_by="cuda_time_total", row_limit=30, max_name_column_width=90))
    if world > 1:
        dist.destroy_process_group()


if __name__ == "__main__":
    main()
