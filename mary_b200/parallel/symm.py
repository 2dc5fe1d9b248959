"""Symmetric heap: one buffer per rank whose peer addresses (and NVSwitch multicast address) every rank knows, plus the
collectives this package runs on it with its own kernels (``csrc/kernels/comm.cu``).

``torch.distributed._symmetric_memory`` does the plumbing only (allocation, handle exchange, multicast binding); the
data movement is ours: the all-reduce reads the peers through ``multimem.ld_reduce`` (in-switch sum) or plain peer
loads and writes the result to every rank with ``multimem.st`` / peer stores."""
from __future__ import annotations

import ctypes
import os

import torch

from ..ops.cuda import _stream, check, declare, lib
from ..utils import flags

declare("mary_allreduce_bf16", "pplii" + "lllpiils")
declare("mary_allreduce_f32", "pplii" + "lllpiils")
declare("mary_allreduce_bf16_oneshot", "pppplii" + "lllpiils")
declare("mary_wait_flag", "piiiils")
declare("mary_argmax_merge", "ppiiipplii" + "pilpps")

FLAG_WORDS = 64 * 2 * 8        # grid <= 64 blocks, two barriers, eight ranks
PAIR_TOKENS = 4096             # rows one arg-max merge can carry
PAIR_BYTES = 2 * 8 * PAIR_TOKENS * 8
MERGE_SLOT = 62                # flag block of the arg-max merge (all-reduce grids stay below it)
ONESHOT_MAX_BYTES = 1 << 20    # vectors up to this size take the one-barrier form (every rank sums the whole vector itself)


class SymmetricHeap:
    def __init__(self, rank: int, world: int, device, max_bytes: int, use_multicast: bool | None = None, grid: int = 48,
                 wait_ms: float = 2000.0):
        import torch.distributed as dist
        import torch.distributed._symmetric_memory as symm_mem
        self.rank, self.world, self.dev = rank, world, torch.device(device)
        self.region = (max_bytes + 255) // 256 * 256
        self.grid = grid
        self.wait_ns = int(wait_ms * 1e6)
        self.buf = symm_mem.empty(2 * self.region + PAIR_BYTES, dtype=torch.uint8, device=self.dev)
        self.buf[2 * self.region:].zero_()
        self.hdl = symm_mem.rendezvous(self.buf, dist.group.WORLD)
        self.flags = symm_mem.empty(FLAG_WORDS, dtype=torch.int32, device=self.dev)
        self.flags.zero_()
        self.fhdl = symm_mem.rendezvous(self.flags, dist.group.WORLD)
        self.buf_ptrs = (ctypes.c_uint64 * 8)(*list(self.hdl.buffer_ptrs)[:world])
        self.sig_ptrs = (ctypes.c_uint64 * 8)(*list(self.fhdl.buffer_ptrs)[:world])
        mc = 0
        want_mc = use_multicast if use_multicast is not None else flags.get("MARY_MULTIMEM")
        if want_mc:
            try:
                mc = int(self.hdl.multicast_ptr or 0)
            except Exception:
                mc = 0
        self.mc = mc
        self.epochs = torch.zeros(64 + 8, dtype=torch.int32, device=self.dev)     # per-block flag epochs (+ barrier slots)
        self.local_out = torch.empty(min(self.region // 2, ONESHOT_MAX_BYTES), dtype=torch.uint8, device=self.dev)
        self.oneshot = flags.get("MARY_ONESHOT")
        torch.cuda.synchronize()
        dist.barrier()

    @property
    def multicast(self) -> bool:
        return self.mc != 0

    def input_view(self, shape, dtype=torch.bfloat16):
        """A tensor over the start of the input region: producers (the row-parallel GEMM) write their partial sums
        here directly, which saves the staging copy."""
        n = 1
        for s in shape:
            n *= s
        nbytes = n * torch.empty((), dtype=dtype).element_size()
        if nbytes > self.region:
            raise ValueError(f"{nbytes} bytes exceed the symmetric region of {self.region}")
        return self.buf[:nbytes].view(dtype).view(*shape)

    def all_reduce(self, partial):
        """Sum ``partial`` (bf16) over all ranks; returns a tensor over the output region (valid until the next call)."""
        assert partial.dtype == torch.bfloat16
        n = partial.numel()
        pad = (-n) % 8
        nbytes = (n + pad) * 2
        if nbytes > self.region:
            raise ValueError(f"{nbytes} bytes exceed the symmetric region of {self.region}")
        if self.oneshot and nbytes <= self.local_out.numel() and pad == 0 and partial.is_contiguous() and partial.data_ptr() % 16 == 0:
            # small vector: stage, one barrier, every rank sums the whole vector into a local buffer
            out = self.local_out[:nbytes].view(torch.bfloat16)
            grid = (n // 8 + 2047) // 2048            # block b owns vectors [2048 b, 2048 (b + 1)) whatever the length
            half = self.region // 2 // 16 * 16
            check(lib().mary_allreduce_bf16_oneshot(partial.data_ptr(), out.data_ptr(), self.buf_ptrs, self.sig_ptrs, self.mc, self.rank,
                                                    self.world, self.region, half, n, self.epochs.data_ptr(), grid, 1 if self.mc else 0,
                                                    self.wait_ns, _stream()), "allreduce_oneshot")
            return out.view(partial.shape)
        if partial.data_ptr() != self.buf.data_ptr():
            self.buf[:n * 2].view(torch.bfloat16).copy_(partial.reshape(-1))
        if pad:
            self.buf[n * 2:nbytes].zero_()
        check(lib().mary_allreduce_bf16(self.buf_ptrs, self.sig_ptrs, self.mc, self.rank, self.world, 0, self.region, n + pad,
                                        self.epochs.data_ptr(), self.grid, 1 if self.mc else 0, self.wait_ns, _stream()),
              "allreduce_bf16")
        return self.buf[self.region:self.region + n * 2].view(torch.bfloat16).view(partial.shape)

    def all_reduce_f32_(self, t):
        """In-place sum of an f32 tensor over all ranks (gradient buckets): staged through the symmetric region, reduced by the
        same two-shot kernel in f32 (``multimem.ld_reduce.add.f32`` in the switch, or peer loads in rank order)."""
        assert t.dtype == torch.float32
        n = t.numel()
        pad = (-n) % 4
        nbytes = (n + pad) * 4
        if nbytes > self.region:
            raise ValueError(f"{nbytes} bytes exceed the symmetric region of {self.region}")
        self.buf[:n * 4].view(torch.float32).copy_(t.reshape(-1))
        if pad:
            self.buf[n * 4:nbytes].zero_()
        check(lib().mary_allreduce_f32(self.buf_ptrs, self.sig_ptrs, self.mc, self.rank, self.world, 0, self.region, n + pad,
                                       self.epochs.data_ptr(), self.grid, 1 if self.mc else 0, self.wait_ns, _stream()),
              "allreduce_f32")
        t.reshape(-1).copy_(self.buf[self.region:self.region + n * 4].view(torch.float32))
        return t

    def wait_flag(self, slot: int, want: int):
        """Launch a bounded wait on one of this rank's flags (failure-detection tests)."""
        check(lib().mary_wait_flag(self.sig_ptrs, self.rank, self.world, slot, want, self.wait_ns, _stream()), "wait_flag")

    def argmax_merge(self, val, idx_local, vocab_offset: int):
        """Merge per-rank ``(max logit, local index)`` candidates of a vocabulary-parallel head: returns the global
        ``(ids, value)`` of the overall arg-max (ties -> lower index), the same on every rank."""
        T = val.numel()
        if T > PAIR_TOKENS:
            raise ValueError(f"{T} rows exceed the merge table of {PAIR_TOKENS}")
        val = val.float().contiguous()
        idx_local = idx_local.to(torch.int64).contiguous()
        out_i = torch.empty(T, dtype=torch.int64, device=self.dev)
        out_v = torch.empty(T, dtype=torch.float32, device=self.dev)
        check(lib().mary_argmax_merge(val.data_ptr(), idx_local.data_ptr(), T, PAIR_TOKENS, vocab_offset, self.buf_ptrs, self.sig_ptrs,
                                      2 * self.region, self.rank, self.world, self.epochs[MERGE_SLOT:].data_ptr(), MERGE_SLOT,
                                      self.wait_ns, out_i.data_ptr(), out_v.data_ptr(), _stream()), "argmax_merge")
        return out_i, out_v
