"""Expert parallelism with tokens on their home rank: dispatch / combine as peer stores from our own kernels
(``csrc/kernels/ep_a2a.cu``), no library all-to-all.

Every rank owns ``E / world`` experts and four symmetric slabs: received activation codes, their scale tiles, the return
address of every received row, and the combine buffer its own tokens' expert outputs come back into.  One MoE layer is

    counts -> barrier -> plan -> dispatch (quantise + peer stores) -> barrier -> w13 GEMM -> quantise -> w2 GEMM whose
    epilogue stores each row into the home rank's combine buffer -> barrier -> weighted sum over the k slots.

``EPLayer`` runs that sequence for one rank; ``emulate`` drives several ranks that live on ONE device phase by phase (the
barriers are kernels of their own, never waits inside the data kernels, so stream order can stand in for them), which is
how the path is tested where only one GPU is available."""
from __future__ import annotations

import ctypes

import torch

from ..ops import cuda_moe
from ..ops.cuda import _p, _stream, check, declare, lib
from ..ops.moe import NVFP4Experts

declare("mary_ep_counts", "piiiips")
declare("mary_ep_plan", "piiiiippppis")
declare("mary_ep_dispatch", "plp" + "iiiiiiiiii" + "pp" + "ppp" + "s")
declare("mary_ep_return_ptrs", "pppiiiiipps")
declare("mary_rank_barrier", "piipils")
declare("mary_gemm_nvfp4_grouped_ex", "pppppppp" + "liiilii" + "ps")


def _ptrs(tensors):
    return (ctypes.c_uint64 * 8)(*[int(t.data_ptr()) if hasattr(t, "data_ptr") else int(t) for t in tensors])


class EPBuffers:
    """The symmetric slabs of one rank (plain tensors; ``peer_*`` hold every rank's base address)."""

    def __init__(self, world: int, E: int, H: int, F: int, t_cap: int, k: int, nt: int, device, alloc=None, shared: bool = False):
        """``shared``: every rank also serves one shared expert over its own ``t_cap`` rows inside the same GEMM launches; a
        token then has ``k + 1`` entries (``self.k`` counts them all)."""
        alloc = alloc or (lambda n, dt: torch.zeros(n, dtype=dt, device=device))
        self.shared = shared
        self.world, self.E, self.H, self.F, self.t_cap, self.nt = world, E, H, F, t_cap, nt
        self.k_routed, self.k = k, k + (1 if shared else 0)
        e_local = E // world
        entries = world * t_cap * k
        self.cap_rows = (entries + min(entries, e_local) * (nt - 1) + nt - 1) // nt * nt + ((t_cap + nt - 1) // nt * nt if shared else 0)
        self.entry_stride = t_cap * self.k
        self.count_mat = alloc(world * E, torch.int32)
        self.xq = alloc(self.cap_rows * (H // 2), torch.uint8)
        self.sf = alloc((self.cap_rows // nt) * (H // 64) * 512, torch.uint8)
        self.meta = alloc(self.cap_rows, torch.int32)
        self.comb = alloc(self.entry_stride * H, torch.bfloat16)


class EPLayer:
    def __init__(self, rank: int, world: int, experts: NVFP4Experts, bufs: EPBuffers, peers: list[EPBuffers], sig_ptrs=None,
                 wait_ns: int = int(2e9)):
        self.rank, self.world, self.ex, self.b = rank, world, experts, bufs
        self.e_local = bufs.E // world
        dev = bufs.xq.device
        self.p_count = _ptrs([p.count_mat for p in peers])
        self.p_xq = _ptrs([p.xq for p in peers])
        self.p_sf = _ptrs([p.sf for p in peers])
        self.p_meta = _ptrs([p.meta for p in peers])
        self.p_comb = _ptrs([p.comb for p in peers])
        self.tiles = torch.empty(bufs.cap_rows // bufs.nt, 4, dtype=torch.int32, device=dev)
        self.plan_meta = torch.zeros(2, dtype=torch.int32, device=dev)
        self.send_base = torch.empty(bufs.E + 1, dtype=torch.int32, device=dev)
        self.send_cnt = torch.empty(bufs.E + 1, dtype=torch.int32, device=dev)
        self.row_ptrs = torch.zeros(bufs.cap_rows, dtype=torch.int64, device=dev)
        self.ident = torch.arange(bufs.entry_stride, dtype=torch.int32, device=dev)
        self.sig_ptrs, self.wait_ns = sig_ptrs, wait_ns
        self.epoch_slot = torch.zeros(1, dtype=torch.int32, device=dev)   # device-resident, so graph replays advance it

    # ---- phases (each is a few kernel launches on the current stream)
    def barrier(self):
        if self.sig_ptrs is None:
            return                      # single-device emulation: stream order separates the phases
        check(lib().mary_rank_barrier(self.sig_ptrs, self.rank, self.world, self.epoch_slot.data_ptr(), 60, self.wait_ns, _stream()),
              "rank_barrier")

    def counts(self, idx):
        T, k = idx.shape
        check(lib().mary_ep_counts(_p(idx), T * k, self.b.E, self.rank, self.world, self.p_count, _stream()), "ep_counts")

    def plan_and_dispatch(self, x, idx):
        b = self.b
        T, k = idx.shape
        check(lib().mary_ep_plan(_p(b.count_mat), self.world, self.rank, b.E, self.e_local, b.nt, _p(self.tiles), _p(self.plan_meta),
                                 _p(self.send_base), _p(self.send_cnt), T if b.shared else 0, _stream()), "ep_plan")
        check(lib().mary_ep_dispatch(_p(x), x.stride(0), _p(idx), T * k, k, b.E, self.e_local, b.H, b.nt, self.rank, self.world,
                                     b.entry_stride, b.cap_rows, _p(self.send_base), _p(self.send_cnt), self.p_xq, self.p_sf, self.p_meta,
                                     _stream()), "ep_dispatch")

    def experts(self):
        b, ex = self.b, self.ex
        plan = cuda_moe.Plan()
        plan.tiles, plan.meta, plan.max_rows, plan.nt = self.tiles, self.plan_meta, b.cap_rows, b.nt
        xq = b.xq.view(b.cap_rows, b.H // 2)
        sfx = b.sf.view(b.cap_rows // b.nt, b.H // 64, 512)
        h = cuda_moe.grouped_gemm(ex.w13_q, ex.w13_sf, ex.w13_s2, xq, sfx, plan, ex.F, ex.H, ex.E, ex.act)
        hq, sfh, _ = cuda_moe.quantize_rows(h, b.nt, None, identity=True, rows=b.cap_rows, n_rows=self.plan_meta[1:2], zero_sf=False)
        check(lib().mary_ep_return_ptrs(_p(b.meta), _p(self.plan_meta), _p(self.tiles), b.cap_rows // b.nt, b.nt, b.entry_stride, b.H,
                                        self.world, self.p_comb, _p(self.row_ptrs), _stream()), "ep_return_ptrs")
        check(lib().mary_gemm_nvfp4_grouped_ex(_p(ex.w2_q), _p(ex.w2_sf), _p(ex.w2_s2), _p(hq), _p(sfh), _p(self.tiles), _p(self.plan_meta),
                                               None, 0, ex.E, ex.H, ex.F, b.cap_rows, b.nt, 0, _p(self.row_ptrs), _stream()),
              "gemm_nvfp4_grouped")

    def finish(self, w, T, shared=None):
        b = self.b
        k = w.shape[1]
        comb = b.comb.view(b.entry_stride, b.H)
        plan = cuda_moe.Plan()
        plan.row_of = self.ident
        return cuda_moe.unpermute(comb, plan, w, T, k, shared)

    def check_shape(self, x, idx):
        """Entry ids ``t * k + j`` address rows of the home rank's combine buffer and are packed into return addresses with
        ``entry_stride = t_cap * k``: a batch beyond ``t_cap`` rows, or another ``k``, would store outside the peers' slabs."""
        b = self.b
        if x.shape[0] > b.t_cap:
            raise ValueError(f"{x.shape[0]} rows exceed the expert-parallel slabs' capacity of {b.t_cap} rows per rank")
        if idx.shape[0] != x.shape[0] or idx.shape[1] not in (b.k_routed, b.k):
            raise ValueError(f"routing table {tuple(idx.shape)} does not match {x.shape[0]} rows x {b.k_routed} experts per token")
        if x.shape[1] != b.H:
            raise ValueError(f"hidden size {x.shape[1]} != {b.H}")

    def with_shared(self, idx, w):
        """Append the shared expert's entry (id ``E``, weight 1) to every token's routed entries."""
        T = idx.shape[0]
        tail = getattr(self, "_tail", None)
        if tail is None or tail[0].shape[0] != T:
            tail = (torch.full((T, 1), self.b.E, dtype=torch.int32, device=idx.device), torch.ones(T, 1, dtype=torch.float32, device=idx.device))
            self._tail = tail
        return torch.cat([idx.to(torch.int32), tail[0]], 1), torch.cat([w.float(), tail[1]], 1)

    def forward(self, x, idx, w, shared=None):
        """One MoE layer for this rank's tokens (``idx`` holds GLOBAL expert ids).  With a shared expert in the buffers'
        layout the caller passes the routed entries only; the shared entry is appended here."""
        self.check_shape(x, idx)
        if self.b.shared and idx.shape[1] == self.b.k_routed:
            idx, w = self.with_shared(idx, w)
        idx = idx.to(torch.int32).contiguous()
        self.counts(idx)
        self.barrier()
        self.plan_and_dispatch(x, idx)
        self.barrier()
        self.experts()
        self.barrier()
        return self.finish(w, x.shape[0], shared)


def emulate(layers: list[EPLayer], xs, idxs, ws):
    """Drive ``world`` ranks that share one device, phase by phase; returns each rank's output."""
    for l, x, i in zip(layers, xs, idxs):
        l.check_shape(x, i)
    if layers[0].b.shared and idxs[0].shape[1] == layers[0].b.k_routed:
        pairs = [l.with_shared(i, w) for l, i, w in zip(layers, idxs, ws)]
        idxs, ws = [p[0] for p in pairs], [p[1] for p in pairs]
    idxs = [i.to(torch.int32).contiguous() for i in idxs]
    for l, i in zip(layers, idxs):
        l.counts(i)
    for l, x, i in zip(layers, xs, idxs):
        l.plan_and_dispatch(x, i)
    for l in layers:
        l.experts()
    return [l.finish(w, x.shape[0]) for l, x, w in zip(layers, xs, ws)]


def distributed_factory(rank: int, world: int, device, t_cap: int, nt: int = 32, sig_ptrs=None, wait_ns: int = int(2e9)):
    """Returns ``factory(experts, cfg) -> EPLayer`` for real multi-GPU runs: the slabs come from the symmetric-memory
    allocator (every rank learns every peer's base address) and the phases are separated by the rank-barrier kernel.
    All layers of a model share ONE set of slabs (layers run one after the other on the stream)."""
    import types

    import torch.distributed as dist
    import torch.distributed._symmetric_memory as symm_mem
    state = {}

    def factory(experts, cfg, t_cap_override: int | None = None, nt_override: int | None = None):
        """``t_cap_override`` / ``nt_override`` build a second set of slabs for another batch shape (prefill chunks next to decode
        steps): every rank must ask for the same shapes in the same order."""
        tc, tile = t_cap_override or t_cap, nt_override or nt
        key = (tc, tile)
        st = state.setdefault(key, {})
        if "bufs" not in st:
            def alloc(n, dt):
                t = symm_mem.empty(n, dtype=dt, device=device)
                t.zero_()
                return t
            b = EPBuffers(world, cfg.n_routed_experts, cfg.hidden_size, cfg.moe_intermediate_size, tc, cfg.num_experts_per_tok, tile,
                          device, alloc, shared=bool(cfg.shared_expert_nvfp4 and cfg.n_shared_experts == 1))
            peers = [types.SimpleNamespace() for _ in range(world)]
            for name in ("count_mat", "xq", "sf", "meta", "comb"):
                hdl = symm_mem.rendezvous(getattr(b, name), dist.group.WORLD)
                for r in range(world):
                    setattr(peers[r], name, int(hdl.buffer_ptrs[r]))
            sp = sig_ptrs
            if sp is None:
                if "sig" not in state:
                    flags = symm_mem.empty(1024, dtype=torch.int32, device=device)
                    flags.zero_()
                    fh = symm_mem.rendezvous(flags, dist.group.WORLD)
                    state["sig"] = (ctypes.c_uint64 * 8)(*list(fh.buffer_ptrs)[:world])
                    state["flags"] = flags
                sp = state["sig"]
            torch.cuda.synchronize()
            dist.barrier()
            st.update(bufs=b, peers=peers, sig=sp)
        layer = EPLayer(rank, world, experts, st["bufs"], st["peers"], st["sig"], wait_ns)
        # one epoch word for all layers and shapes: they share the flag slots
        if "epoch_slot" not in state:
            state["epoch_slot"] = layer.epoch_slot
        layer.epoch_slot = state["epoch_slot"]
        return layer

    return factory
