"""Sequence-parallel tensor parallelism with the collectives fused into the compute kernels.

The residual stream is sharded by token rows (rank ``r`` keeps rows ``[r * rpr, (r + 1) * rpr)``); between two blocks:

* **GEMM -> reduce-scatter**: the row-parallel GEMM (``o_proj`` / ``down_proj``) never stores its partial result locally; its
  epilogue writes every output row straight into the staging buffer of the rank that owns that token
  (``mary_gemm_bf16_rs``: peer stores from inside the tcgen05 kernel, tile by tile);
* **reduce + residual + RMSNorm -> all-gather**: the owner sums the ``world`` staged partial rows in rank order, adds them to
  its residual rows, norms, and writes the normed rows into EVERY rank's activation buffer (one ``multimem.st`` per 16 bytes
  through NVSwitch, or peer stores) — so the next column-parallel GEMM reads its input from local memory;
* two rank barriers (kernels of their own) separate the phases.
The reference prices tensor parallelism at 84 all-reduces per token over a 26.84 us NCCL all-reduce and does not build it
(src/bin/inkling_forward.rs:80-85,656-662)."""
from __future__ import annotations

import ctypes

import torch

from ..ops.cuda import _p, _stream, check, declare, lib

declare("mary_gemm_bf16_rs", "ppiiilllpiiiis")
declare("mary_rs_add_rmsnorm", "ppppliiliifs")
declare("mary_rank_barrier", "piipils")


class SequenceParallel:
    def __init__(self, rank: int, world: int, rows: int, hidden: int, device, staging=None, xbuf=None, peers_staging=None, peers_x=None,
                 x_mc: int = 0, sig_ptrs=None, wait_ns: int = int(2e9)):
        assert rows % world == 0, "token rows must divide evenly over the ranks"
        self.rank, self.world, self.rows, self.H = rank, world, rows, hidden
        self.rpr = rows // world
        dev = torch.device(device)
        self.staging = staging if staging is not None else torch.zeros(world * self.rpr * hidden, dtype=torch.bfloat16, device=dev)
        self.xbuf = xbuf if xbuf is not None else torch.zeros(rows * hidden, dtype=torch.bfloat16, device=dev)
        self.p_staging = (ctypes.c_uint64 * 8)(*(peers_staging or [self.staging.data_ptr()]))
        self.p_x = (ctypes.c_uint64 * 8)(*(peers_x or [self.xbuf.data_ptr()]))
        self.x_mc, self.sig_ptrs, self.wait_ns = x_mc, sig_ptrs, wait_ns
        self.epoch_slot = torch.zeros(1, dtype=torch.int32, device=dev)

    @staticmethod
    def distributed(rank, world, rows, hidden, device, use_multicast: bool = True):
        import torch.distributed as dist
        import torch.distributed._symmetric_memory as symm_mem
        rpr = rows // world
        st = symm_mem.empty(world * rpr * hidden, dtype=torch.bfloat16, device=device)
        xb = symm_mem.empty(rows * hidden, dtype=torch.bfloat16, device=device)
        fl = symm_mem.empty(1024, dtype=torch.int32, device=device)
        for t in (st, xb, fl):
            t.zero_()
        hs, hx, hf = (symm_mem.rendezvous(t, dist.group.WORLD) for t in (st, xb, fl))
        mc = 0
        if use_multicast:
            try:
                mc = int(hx.multicast_ptr or 0)
            except Exception:
                mc = 0
        sp = SequenceParallel(rank, world, rows, hidden, device, st, xb, list(hs.buffer_ptrs)[:world], list(hx.buffer_ptrs)[:world], mc,
                              (ctypes.c_uint64 * 8)(*list(hf.buffer_ptrs)[:world]))
        sp._keep = (fl,)
        torch.cuda.synchronize()
        dist.barrier()
        return sp

    def barrier(self):
        if self.sig_ptrs is None:
            return
        check(lib().mary_rank_barrier(self.sig_ptrs, self.rank, self.world, self.epoch_slot.data_ptr(), 61, self.wait_ns, _stream()),
              "rank_barrier")

    def row_linear_rs(self, x, w):
        """``x[T, K_local] @ w[N, K_local]^T`` with the partial rows delivered to their owners' staging buffers."""
        M, Kd = x.shape
        assert M == self.rows and w.shape[0] == self.H
        check(lib().mary_gemm_bf16_rs(_p(x.contiguous()), _p(w), M, self.H, Kd, x.stride(0), w.stride(0), self.H, self.p_staging,
                                      self.world, self.rank, self.rpr, -1, _stream()), "gemm_bf16_rs")

    def push_partial(self, partial):
        """A partial result that did not come from a GEMM epilogue (e.g. the expert un-permute): copy rows to their owners."""
        v = partial.view(self.world, self.rpr, self.H)
        for o in range(self.world):
            dst = self._peer_staging_view(o)
            dst[self.rank].copy_(v[o])

    def _peer_staging_view(self, owner):
        raise NotImplementedError("peer views need symmetric-memory tensors; use row_linear_rs for GEMM outputs")

    def reduce_add_rmsnorm(self, h_slice, w, eps: float = 1e-6):
        """Finish the reduce-scatter on this rank's rows, add to ``h_slice`` (in place), norm, all-gather.  Returns the
        normed activations of ALL rows ``[T, H]`` (valid until the next call)."""
        self.barrier()
        check(lib().mary_rs_add_rmsnorm(_p(self.staging), _p(h_slice), _p(w), self.p_x, self.x_mc, self.rank, self.world, 0, self.rpr,
                                        self.H, eps, _stream()), "rs_add_rmsnorm")
        self.barrier()
        return self.xbuf.view(self.rows, self.H)
