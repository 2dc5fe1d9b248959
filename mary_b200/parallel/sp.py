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
declare("mary_rs_add_rmsnorm", "ppppfpliiliifs")
declare("mary_rank_barrier", "piipils")


class SequenceParallel:
    """``rows`` is the capacity in token rows; a call with ``T <= rows`` rows uses ``ceil(T / world)`` rows per rank (the last
    rank's tail rows are padding that nothing reads)."""

    def __init__(self, rank: int, world: int, rows: int, hidden: int, device, staging=None, xbuf=None, peers_staging=None, peers_x=None,
                 x_mc: int = 0, sig_ptrs=None, wait_ns: int = int(2e9)):
        self.rank, self.world, self.H = rank, world, hidden
        self.rows = (rows + world - 1) // world * world
        self.rpr = self.rows // world
        dev = torch.device(device)
        self.dev = dev
        self.staging = staging if staging is not None else torch.zeros(self.rows * hidden, dtype=torch.bfloat16, device=dev)
        self.xbuf = xbuf if xbuf is not None else torch.zeros(self.rows * hidden, dtype=torch.bfloat16, device=dev)
        self.p_staging = (ctypes.c_uint64 * 8)(*(peers_staging or [self.staging.data_ptr()]))
        self.p_x = (ctypes.c_uint64 * 8)(*(peers_x or [self.xbuf.data_ptr()]))
        self.x_mc, self.sig_ptrs, self.wait_ns = x_mc, sig_ptrs, wait_ns
        self.epoch_slot = torch.zeros(1, dtype=torch.int32, device=dev)
        self.T = self.rows

    @staticmethod
    def distributed(rank, world, rows, hidden, device, use_multicast: bool = True):
        import torch.distributed as dist
        import torch.distributed._symmetric_memory as symm_mem
        rows = (rows + world - 1) // world * world
        st = symm_mem.empty(rows * hidden, dtype=torch.bfloat16, device=device)
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

    def rows_per_rank(self, T: int) -> int:
        if T > self.rows:
            raise ValueError(f"{T} rows exceed the sequence-parallel capacity of {self.rows}")
        return (T + self.world - 1) // self.world

    def residual_slice(self, h):
        """This rank's rows of a replicated residual stream ``h [T, H]`` (zero-padded to the per-rank row count)."""
        T = h.shape[0]
        rpr = self.rows_per_rank(T)
        out = torch.zeros(rpr, self.H, dtype=h.dtype, device=h.device)
        lo, hi = self.rank * rpr, min((self.rank + 1) * rpr, T)
        if hi > lo:
            out[:hi - lo].copy_(h[lo:hi])
        return out

    def barrier(self):
        if self.sig_ptrs is None:
            return
        check(lib().mary_rank_barrier(self.sig_ptrs, self.rank, self.world, self.epoch_slot.data_ptr(), 61, self.wait_ns, _stream()),
              "rank_barrier")

    def row_linear_rs(self, x, w):
        """``x[T, K_local] @ w[N, K_local]^T`` with the partial rows delivered to their owners' staging buffers."""
        M, Kd = x.shape
        assert w.shape[0] == self.H
        self.T = M
        rpr = self.rows_per_rank(M)
        check(lib().mary_gemm_bf16_rs(_p(x.contiguous()), _p(w), M, self.H, Kd, x.stride(0), w.stride(0), self.H, self.p_staging,
                                      self.world, self.rank, rpr, -1, _stream()), "gemm_bf16_rs")

    def reduce_add_rmsnorm(self, h_slice, w, eps: float = 1e-6, w_post=None, scalar: float = 1.0):
        """Finish the reduce-scatter on this rank's rows, join the sum to ``h_slice`` (in place) — directly, or normed by
        ``w_post`` first and the new residual scaled by ``scalar`` (sandwich norms) —, norm by ``w``, all-gather.  Returns
        the normed activations of the ``T`` rows of the preceding ``row_linear_rs`` ``[T, H]`` (valid until the next call)."""
        rpr = self.rows_per_rank(self.T)
        assert h_slice is None or h_slice.shape[0] == rpr
        self.barrier()
        check(lib().mary_rs_add_rmsnorm(_p(self.staging), _p(h_slice), _p(w_post), _p(w), scalar, self.p_x, self.x_mc, self.rank,
                                        self.world, 0, rpr, self.H, eps, _stream()), "rs_add_rmsnorm")
        self.barrier()
        return self.xbuf[:self.T * self.H].view(self.T, self.H)
