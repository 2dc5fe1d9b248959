"""Collective micro-benchmarks over NVLink / NVSwitch, one process per GPU under ``torch.distributed.run``:

    python -m torch.distributed.run --nproc-per-node N -m mary_b200.parallel.bench_comm

Times this package's own kernels over peer memory (two-shot all-reduce with ``multimem`` or peer loads / stores; the
GEMM -> reduce-scatter epilogue followed by the fused sum + norm + all-gather kernel) against the library arm (NCCL through
``torch.distributed``) with CUDA events on the launching stream, after warm-up, maximum over ranks.  Bus bandwidth of an
all-reduce = ``2 (N - 1) / N * bytes / time``; the measured references of the machine are 725 GB/s bus bandwidth for an 8-rank
1 GiB NCCL all-reduce and 770 GB/s per direction for a peer copy."""
from __future__ import annotations

import json

import torch
import torch.distributed as dist


def _time(fn, iters=20, warmup=5):
    for _ in range(warmup):
        fn()
    torch.cuda.synchronize()
    dist.barrier()
    a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    a.record()
    for _ in range(iters):
        fn()
    b.record()
    torch.cuda.synchronize()
    t = torch.tensor([a.elapsed_time(b) / iters], device="cuda", dtype=torch.float64)
    dist.all_reduce(t, op=dist.ReduceOp.MAX)
    return float(t)


def main():
    from ..ops import cuda as K
    from .group import init_distributed
    from .sp import SequenceParallel
    from .symm import SymmetricHeap
    rank, world, local = init_distributed()
    dev = torch.device("cuda", local)
    rows = []
    heaps = {mc: SymmetricHeap(rank, world, dev, max_bytes=64 << 20, use_multicast=mc) for mc in (True, False)}
    for n in (48 * 7168, 384 * 7168, 32 * 3840, 4 << 20, 32 << 20):
        x = torch.randn(n, device=dev).bfloat16()
        nbytes = n * 2
        res = {"op": "all_reduce bf16", "bytes": nbytes}
        y = x.clone()
        res["nccl_us"] = round(_time(lambda: dist.all_reduce(y)) * 1e3, 2)
        for mc, heap in heaps.items():
            if mc and not heap.multicast:
                continue
            v = heap.input_view((n,))
            v.copy_(x)
            res["multimem_us" if mc else "p2p_us"] = round(_time(lambda: heap.all_reduce(v)) * 1e3, 2)
        best = min(res.get("multimem_us", 1e30), res["p2p_us"])
        res["busbw_gbs_ours"] = round(2 * (world - 1) / world * nbytes / (best * 1e-6) / 1e9, 1)
        res["busbw_gbs_nccl"] = round(2 * (world - 1) / world * nbytes / (res["nccl_us"] * 1e-6) / 1e9, 1)
        rows.append(res)
    # GEMM -> reduce-scatter epilogue + fused sum / norm / all-gather against GEMM + NCCL all-reduce + norm kernel
    for T, H, Kl in ((32, 3840, 15360 // world), (2048, 3840, 15360 // world)):
        T = (T + world - 1) // world * world
        sp = SequenceParallel.distributed(rank, world, T, H, dev)
        x = torch.randn(T, Kl, device=dev).bfloat16()
        w = (torch.randn(H, Kl, device=dev) * 0.02).bfloat16()
        gain = torch.ones(H, device=dev).bfloat16()
        hs = torch.zeros(T // world, H, device=dev).bfloat16()
        hfull = torch.zeros(T, H, device=dev).bfloat16()

        def ours():
            sp.row_linear_rs(x, w)
            sp.reduce_add_rmsnorm(hs, gain, 1e-6)

        def lib():
            y = K.linear(x, w)
            dist.all_reduce(y)
            K.add_rmsnorm(y, hfull, gain, 1e-6)
        t_ours, t_lib = _time(ours), _time(lib)
        link_bytes = (world - 1) / world * T * H * 2 * 2                # reduce-scatter + all-gather, per GPU and direction
        rows.append({"op": "gemm->reduce-scatter + sum/norm/all-gather", "tokens": T, "hidden": H, "k_local": Kl,
                     "ours_us": round(t_ours * 1e3, 2), "gemm+nccl_allreduce+norm_us": round(t_lib * 1e3, 2),
                     "nvlink_roofline_us": round(link_bytes / 770e9 * 1e6, 2),
                     "gemm_flops_roofline_us": round(2.0 * T * H * Kl / 1.4e15 * 1e6, 2)})
    if rank == 0:
        for r in rows:
            print(json.dumps(r))
        print(json.dumps({"world": world, "multimem": heaps[True].multicast, "kernel_status": K.last_status()}))
    dist.barrier()
    dist.destroy_process_group()


if __name__ == "__main__":
    main()
