"""The four-launch expert pipeline (``csrc/kernels/ep_fused.cu`` + counter mode of ``gemm_nvfp4.cu``).

One MoE layer on decode-sized batches is::

    route + dispatch  ->  w13 grouped GEMM (waits for the sources, GLU, result quantised)  ->
    w2 grouped GEMM (rows stored to their home rank, flags)  ->  combine (+ residual add + next RMSNorm)

with no planning pass, no barrier kernels and no separate quantiser: rows are placed by atomics on the owner's per-expert
arrival counters, and kernels hand over through epoch flags in peer memory (every wait bounded, status word on timeout).
``local_only`` contexts run the same launches on one rank by itself (single GPU, or replicated tokens where every rank serves
its own experts and the partial sums are reduced afterwards).

The reference does this with a blocking router readback and a host planner per layer
(src/bin/inkling_forward.rs:4442-4478, src/models/inkling/moegroup.rs:978-1083) and has no expert parallelism."""
from __future__ import annotations

import ctypes

import torch

from ..ops.cuda import _p, _stream, check, declare, lib
from ..ops.moe import NVFP4Experts

MAX_RANKS = 8
NT = 32
MAX_TILES = 512

declare("mary_ep_route_dispatch", "plppliiiiiifiiippppps")
declare("mary_ep_combine", "pppppppiiifps")
declare("mary_gemm_nvfp4_grouped_ep", "pppppppp" + "iiiliips")
declare("mary_ep_ctx_bytes", "")


class EpCtx(ctypes.Structure):
    """Mirror of ``struct EpCtx`` (ep_ctx.cuh)."""
    _fields_ = [("cnt", ctypes.c_uint64 * MAX_RANKS), ("xq", ctypes.c_uint64 * MAX_RANKS), ("sf", ctypes.c_uint64 * MAX_RANKS),
                ("meta", ctypes.c_uint64 * MAX_RANKS), ("comb", ctypes.c_uint64 * MAX_RANKS), ("flags", ctypes.c_uint64 * MAX_RANKS),
                ("epoch", ctypes.c_void_p), ("done", ctypes.c_void_p),
                ("rank", ctypes.c_int), ("world", ctypes.c_int), ("e_local", ctypes.c_int), ("n_slots", ctypes.c_int),
                ("cap_e", ctypes.c_int), ("NT", ctypes.c_int), ("entry_stride", ctypes.c_int), ("local_only", ctypes.c_int),
                ("wait_ns", ctypes.c_uint64)]


SYMMETRIC = ("cnt", "xq", "sf", "meta", "comb", "flags")


def slab_shapes(world: int, e_local: int, H: int, t_cap: int, k_all: int, shared: bool, local_only: bool):
    """Sizes of one rank's slabs: ``(n_slots, cap_e, slab_rows, {name: (numel, dtype)})``.  ``t_cap``: token rows per rank
    (all rows of the step when tokens are replicated)."""
    n_slots = e_local + (1 if shared else 0)
    cap_e = ((t_cap if local_only else world * t_cap) + NT - 1) // NT * NT      # worst case: every row picks the same expert
    rows = n_slots * cap_e
    return n_slots, cap_e, rows, {
        "cnt": (max(n_slots, 4), torch.int32),
        "xq": (rows * (H // 2), torch.uint8),
        "sf": ((rows // NT) * (H // 64) * 512, torch.uint8),
        "meta": (rows, torch.int32),
        "comb": (t_cap * k_all * H, torch.bfloat16),
        "flags": (2 * MAX_RANKS, torch.int32),
    }


class FusedMoE:
    """Buffers and context of one rank.  All MoE layers of a model share one instance (they run one after the other)."""

    def __init__(self, rank: int, world: int, E_total: int, H: int, F: int, t_cap: int, k: int, shared: bool, device,
                 local_only: bool, bufs: dict | None = None, peer_ptrs: dict | None = None, wait_ns: int = int(2e9)):
        """``bufs``: this rank's symmetric tensors by name (default: plain local allocations); ``peer_ptrs``: for every name the
        list of all ranks' base addresses (default: only this rank's own, which is all a ``local_only`` context touches)."""
        assert E_total % world == 0 and H % 64 == 0 and F % 128 == 0
        self.rank, self.world, self.E, self.H, self.F = rank, world, E_total, H, F
        self.e_local = E_total // world
        self.k, self.shared, self.K1 = k, shared, k + (1 if shared else 0)
        self.t_cap, self.local_only = t_cap, local_only
        self.n_slots, self.cap_e, self.rows, shapes = slab_shapes(world, self.e_local, H, t_cap, self.K1, shared, local_only)
        if self.rows // NT > (1 << 24):
            raise ValueError("slabs too large")
        dev = torch.device(device)
        self.bufs = bufs or {n: torch.zeros(sz, dtype=dt, device=dev) for n, (sz, dt) in shapes.items()}
        for n, (sz, dt) in shapes.items():
            assert self.bufs[n].numel() >= sz and self.bufs[n].dtype == dt, n
        # local scratch: the quantised intermediate, routing outputs, epoch and CTA counters
        self.hq = torch.empty(self.rows * (F // 2), dtype=torch.uint8, device=dev)
        self.sfh = torch.empty((self.rows // NT) * (F // 64) * 512, dtype=torch.uint8, device=dev)
        self.idx_out = torch.zeros(t_cap, self.K1, dtype=torch.int32, device=dev)
        self.w_out = torch.zeros(t_cap, self.K1, dtype=torch.float32, device=dev)
        self.row_out = torch.zeros(t_cap, self.K1, dtype=torch.int32, device=dev)
        self.epoch = torch.zeros(1, dtype=torch.int32, device=dev)
        self.done = torch.zeros(4, dtype=torch.int32, device=dev)
        self.flag = torch.zeros(1, dtype=torch.int32, device=dev)          # non-finite router logit seen
        c = EpCtx()
        for n in SYMMETRIC:
            arr = getattr(c, n)
            ptrs = peer_ptrs[n] if peer_ptrs is not None else None
            for r in range(MAX_RANKS):
                arr[r] = 0
            if ptrs is None:
                arr[rank] = self.bufs[n].data_ptr()
            else:
                for r in range(world):
                    arr[r] = int(ptrs[r])
        c.epoch, c.done = self.epoch.data_ptr(), self.done.data_ptr()
        c.rank, c.world, c.e_local, c.n_slots, c.cap_e, c.NT = rank, world, self.e_local, self.n_slots, self.cap_e, NT
        c.entry_stride, c.local_only, c.wait_ns = t_cap * self.K1, int(local_only), wait_ns
        assert ctypes.sizeof(EpCtx) == lib().mary_ep_ctx_bytes(), "EpCtx layout differs between Python and the kernels"
        self.ctx = c

    def nbytes(self) -> int:
        return sum(t.numel() * t.element_size() for t in list(self.bufs.values()) + [self.hq, self.sfh])

    # ---- the four launches
    def route_dispatch(self, x, logits, router: dict):
        T = x.shape[0]
        if T > self.t_cap:
            raise ValueError(f"{T} rows exceed the expert pipeline's capacity of {self.t_cap} rows")
        if x.shape[1] != self.H or logits.shape != (T, self.E) or logits.dtype != torch.float32:
            raise ValueError("router logits must be f32 [rows, experts] and the rows hidden-size wide")
        bias = router.get("bias")
        check(lib().mary_ep_route_dispatch(_p(logits), logits.stride(0), _p(bias), _p(x), x.stride(0), T, self.E, self.k,
                                           0 if router["mode"] == "softmax" else 1, router.get("n_group", 1), router.get("topk_group", 1),
                                           float(router.get("scale", 1.0)), int(router.get("renorm", True)), int(self.shared), self.H,
                                           _p(self.idx_out), _p(self.w_out), _p(self.row_out), _p(self.flag), ctypes.byref(self.ctx),
                                           _stream()), "ep_route_dispatch")

    def gemm_w13(self, ex: NVFP4Experts):
        assert ex.E == self.n_slots and ex.H == self.H and ex.F == self.F
        g = {"geglu": 1, "swiglu": 2, "situ": 3}[ex.act]
        b = self.bufs
        check(lib().mary_gemm_nvfp4_grouped_ep(_p(ex.w13_q), _p(ex.w13_sf), _p(ex.w13_s2), _p(b["xq"]), _p(b["sf"]), _p(self.hq), _p(self.sfh),
                                               None, ex.E, ex.F, ex.H, self.rows, g, 1, ctypes.byref(self.ctx), _stream()),
              "gemm_nvfp4_grouped")

    def gemm_w2(self, ex: NVFP4Experts):
        b = self.bufs
        check(lib().mary_gemm_nvfp4_grouped_ep(_p(ex.w2_q), _p(ex.w2_sf), _p(ex.w2_s2), _p(self.hq), _p(self.sfh), None, None,
                                               _p(b["meta"]), ex.E, ex.H, ex.F, self.rows, 0, 2, ctypes.byref(self.ctx), _stream()),
              "gemm_nvfp4_grouped")

    def combine(self, T: int, add=None, res=None, w_norm=None, eps: float = 1e-6):
        """``res is None``: returns the weighted sum ``[T, H]``.  Otherwise ``res += sum`` in place and, with ``w_norm``, returns
        ``(rms(res) * w_norm, res)``; without it ``(None, res)``."""
        dev = self.hq.device
        out = torch.empty(T, self.H, dtype=torch.bfloat16, device=dev) if res is None else None
        y = torch.empty(T, self.H, dtype=torch.bfloat16, device=dev) if (res is not None and w_norm is not None) else None
        check(lib().mary_ep_combine(_p(self.w_out), _p(self.row_out), _p(add), _p(out), _p(res), _p(w_norm), _p(y), T, self.K1, self.H,
                                    eps, ctypes.byref(self.ctx), _stream()), "ep_combine")
        return out if res is None else (y, res)

    def forward(self, x, logits, router: dict, ex: NVFP4Experts, add=None, res=None, w_norm=None, eps: float = 1e-6):
        self.route_dispatch(x, logits, router)
        self.gemm_w13(ex)
        self.gemm_w2(ex)
        return self.combine(x.shape[0], add, res, w_norm, eps)


def emulate(ranks: list[FusedMoE], experts: list[NVFP4Experts], xs, logits, router: dict):
    """``world`` ranks that share one device, driven phase by phase: every kernel that waits runs after all kernels it waits
    for, so stream order satisfies the flags.  Returns every rank's combined output."""
    for r, x, lg in zip(ranks, xs, logits):
        r.route_dispatch(x, lg, router)
    for r, ex in zip(ranks, experts):
        r.gemm_w13(ex)
    for r, ex in zip(ranks, experts):
        r.gemm_w2(ex)
    return [r.combine(x.shape[0]) for r, x in zip(ranks, xs)]


def emulated_ranks(world: int, E_total: int, H: int, F: int, t_cap: int, k: int, shared: bool, device) -> list[FusedMoE]:
    """``world`` contexts on one device whose peer tables point at one another's buffers."""
    e_local = E_total // world
    _, _, _, shapes = slab_shapes(world, e_local, H, t_cap, k + (1 if shared else 0), shared, False)
    all_bufs = [{n: torch.zeros(sz, dtype=dt, device=device) for n, (sz, dt) in shapes.items()} for _ in range(world)]
    ptrs = {n: [b[n].data_ptr() for b in all_bufs] for n in SYMMETRIC}
    return [FusedMoE(r, world, E_total, H, F, t_cap, k, shared, device, False, all_bufs[r], ptrs) for r in range(world)]


def distributed(rank: int, world: int, E_total: int, H: int, F: int, t_cap: int, k: int, shared: bool, device,
                wait_ns: int = int(2e9)) -> FusedMoE:
    """Real multi-GPU context: the slabs come from the symmetric-memory allocator, which also tells every rank its peers'
    base addresses.  Collective: every rank must call it with the same arguments at the same point."""
    import torch.distributed as dist
    import torch.distributed._symmetric_memory as symm_mem
    e_local = E_total // world
    _, _, _, shapes = slab_shapes(world, e_local, H, t_cap, k + (1 if shared else 0), shared, False)
    bufs, ptrs = {}, {}
    for n in SYMMETRIC:
        sz, dt = shapes[n]
        t = symm_mem.empty(sz, dtype=dt, device=device)
        t.zero_()
        hdl = symm_mem.rendezvous(t, dist.group.WORLD)
        bufs[n], ptrs[n] = t, [int(p) for p in list(hdl.buffer_ptrs)[:world]]
    torch.cuda.synchronize()
    dist.barrier()
    return FusedMoE(rank, world, E_total, H, F, t_cap, k, shared, device, False, bufs, ptrs, wait_ns)
