"""LoRA trainer: AdamW over flat adapter buffers, data/tensor-parallel gradient reduction overlapped with backward,
checkpoint and resume through the pile.

Reference loop: src/bin/gemma_train_lora.rs:167-335 (single device, Burn autodiff, hand-rolled AdamW with
b1 .9 / b2 .999 / eps 1e-8 / wd .01, no resume).  Added here: DP x TP groups, per-layer gradient buckets reduced as soon
as their layer's backward finishes (on a side stream, so the reduction of layer i overlaps the backward of layer i-1),
a fused AdamW kernel, and optimizer-state checkpoints (train N, save, reload, train N == train 2N)."""
from __future__ import annotations

import io

import numpy as np
import torch

from ..format import schema as S
from ..pile.trible import TribleBuilder, r_u256, v_handle, v_u256
from .lora import Gemma4LoraForward, LoraWeights


class FlatAdamW:
    """All adapter parameters live in ONE f32 buffer (per-layer slices), gradients in a second one; the step is a
    single fused kernel on the GPU."""

    def __init__(self, params, lr=1e-4, betas=(0.9, 0.999), eps=1e-8, weight_decay=0.01):
        self.params = list(params)
        self.lr, self.b1, self.b2, self.eps, self.wd = lr, betas[0], betas[1], eps, weight_decay
        n = sum(p.numel() for p in self.params)
        dev = self.params[0].device
        self.flat = torch.zeros(n, dtype=torch.float32, device=dev)
        self.grad = torch.zeros(n, dtype=torch.float32, device=dev)
        self.m = torch.zeros(n, dtype=torch.float32, device=dev)
        self.v = torch.zeros(n, dtype=torch.float32, device=dev)
        self.offsets = []
        o = 0
        for p in self.params:                    # re-home every parameter (and its gradient) inside the flat buffers
            k = p.numel()
            self.flat[o:o + k].copy_(p.data.reshape(-1))
            p.data = self.flat[o:o + k].view_as(p)
            p.grad = self.grad[o:o + k].view_as(p)
            self.offsets.append((o, k))
            o += k
        self.step_count = 0

    def zero_grad(self):
        self.grad.zero_()

    def step(self, grad_scale: float = 1.0):
        self.step_count += 1
        if self.flat.is_cuda:
            from ..ops.cuda import _p, _stream, check, declare, lib
            declare("mary_adamw", "pppplfffffifs")
            check(lib().mary_adamw(_p(self.flat), _p(self.grad), _p(self.m), _p(self.v), self.flat.numel(), self.lr, self.b1, self.b2,
                                   self.eps, self.wd, self.step_count, grad_scale, _stream()), "adamw")
            return
        g = self.grad * grad_scale
        self.m.mul_(self.b1).add_(g, alpha=1 - self.b1)
        self.v.mul_(self.b2).addcmul_(g, g, value=1 - self.b2)
        mhat = self.m / (1 - self.b1 ** self.step_count)
        vhat = self.v / (1 - self.b2 ** self.step_count)
        self.flat.sub_(self.lr * (mhat / (vhat.sqrt() + self.eps) + self.wd * self.flat))

    def state_bytes(self) -> bytes:
        buf = io.BytesIO()
        np.savez(buf, flat=self.flat.cpu().numpy(), m=self.m.cpu().numpy(), v=self.v.cpu().numpy(),
                 step=np.int64(self.step_count))
        return buf.getvalue()

    def load_state_bytes(self, b: bytes):
        z = np.load(io.BytesIO(b), allow_pickle=False)
        self.flat.copy_(torch.from_numpy(z["flat"]))
        self.m.copy_(torch.from_numpy(z["m"]))
        self.v.copy_(torch.from_numpy(z["v"]))
        self.step_count = int(z["step"])


class LoraTrainer:
    def __init__(self, model, rank: int = 16, alpha: float = 32.0, lr: float = 1e-4, seed: int = 0, dp_group=None, dp_size: int = 1,
                 reduce_fn=None, overlap: bool = True, checkpoint: bool = False, tp_reduce_fn=None, lora=None, seq_parallel=None):
        """``reduce_fn(g)``: in-place sum of a gradient slice over the DATA-parallel group (all replicas of this rank's shard).
        ``tp_reduce_fn(g)``: in-place sum over the TENSOR-parallel group, applied to the factors every rank of the group holds
        identically (their gradients are partial sums, see ``LoraWeights.tp_replicated``).  ``lora``: adapters to train instead of
        freshly initialised ones (already cut for this rank).  ``seq_parallel = (rank, world, group)``: the ranks of the group
        share ONE sequence, each running the layers on its chunk of the rows (attention through all-to-alls); every rank's loss
        and adapter gradients are its share of the whole sequence's, so ``reduce_fn`` must SUM over that group and ``dp_size``
        stays the number of data-parallel replicas (1 when the group is the world)."""
        self.model = model
        self.lora = lora if lora is not None else LoraWeights.init_gemma4(model, rank, alpha, seed)
        self.fwd = Gemma4LoraForward(model, self.lora)
        self.fwd.checkpoint = checkpoint          # recompute every layer in the backward pass instead of keeping its activations
        self.fwd.sp = seq_parallel
        if seq_parallel is not None and reduce_fn is None:
            raise ValueError("sequence-parallel training needs reduce_fn: every rank holds a share of the adapter gradients")
        # parameters ordered by layer so that a layer's gradients are one contiguous bucket; inside a layer the factors that are
        # replicated over the tensor-parallel group come first, so that their partial gradients are one contiguous slice too
        tp = getattr(model, "tp", None)
        tp_size = tp.size if tp is not None else 1
        self.layer_params, self.rep_counts = [], []
        for i, L in enumerate(model.layers):
            kv_rep = tp_size > 1 and model.cfg.layer_kv_heads(i) < tp_size
            rep, shard = [], []
            for k, ad in self.lora.adapters.items():
                li, proj = k.split("_", 1)
                if li != str(i):
                    continue
                for which, p in (("A", ad.A), ("B", ad.B)):
                    (rep if LoraWeights.tp_replicated(proj, which, kv_rep) else shard).append(p)
            self.layer_params.append(rep + shard)
            self.rep_counts.append(sum(p.numel() for p in rep))
        self.opt = FlatAdamW([p for ps in self.layer_params for p in ps], lr=lr)
        self.buckets = []
        o = 0
        for ps in self.layer_params:
            k = sum(p.numel() for p in ps)
            self.buckets.append((o, k))
            o += k
        self.dp_group, self.dp_size = dp_group, dp_size
        self.reduce_fn = reduce_fn               # callable(tensor) -> in-place sum over the data-parallel group
        self.tp_reduce_fn = tp_reduce_fn if tp_size > 1 else None
        if tp_size > 1 and tp_reduce_fn is None:
            raise ValueError("a tensor-parallel model needs tp_reduce_fn: the replicated adapter factors hold partial gradients")
        any_reduce = self.reduce_fn is not None or self.tp_reduce_fn is not None
        self.overlap = overlap and any_reduce
        self.side = torch.cuda.Stream() if (self.overlap and model.embed.is_cuda) else None
        self._pending = [0] * len(self.layer_params)
        self.reduced_bytes = 0
        if any_reduce:
            for li, ps in enumerate(self.layer_params):
                for p in ps:
                    p.register_post_accumulate_grad_hook(self._make_hook(li))

    def _make_hook(self, li):
        def hook(_p):
            self._pending[li] += 1
            if self._pending[li] == len(self.layer_params[li]):
                self._pending[li] = 0
                self._reduce_bucket(li)
        return hook

    def _reduce_bucket(self, li):
        o, k = self.buckets[li]
        g = self.opt.grad[o:o + k]
        g_rep = self.opt.grad[o:o + self.rep_counts[li]]

        def run():
            if self.tp_reduce_fn is not None and g_rep.numel():
                self.tp_reduce_fn(g_rep)             # partial gradients of the replicated factors: sum over the tensor-parallel group
                self.reduced_bytes += g_rep.numel() * 4
            if self.reduce_fn is not None:
                self.reduce_fn(g)                    # every factor: sum over the replicas of this shard
                self.reduced_bytes += k * 4
        if self.side is not None:
            self.side.wait_stream(torch.cuda.current_stream())
            with torch.cuda.stream(self.side):
                run()
        else:
            run()

    def step(self, ids) -> float:
        self.opt.zero_grad()
        loss = self.fwd.loss(ids)
        loss.backward()
        if self.side is not None:
            torch.cuda.current_stream().wait_stream(self.side)
        self.opt.step(grad_scale=1.0 / self.dp_size)
        loss = loss.detach()
        if self.fwd.sp is not None:
            import torch.distributed as dist
            loss = loss.clone()
            dist.all_reduce(loss, group=self.fwd.sp[2])           # the shares add up to the sequence's mean loss
        return float(loss)

    # ------------------------------------------------------------------ checkpoint / resume through the pile
    def save_checkpoint(self, store, tb: TribleBuilder, model_root: bytes | None = None) -> bytes:
        aid = self.lora.save_to_pile(store, tb, model_root)
        h = store.put(self.opt.state_bytes())
        rng = store.put(torch.get_rng_state().numpy().tobytes())
        return tb.entity([(S.TRAIN_RUN, v_handle(rng)), (S.TRAIN_STATE, v_handle(h)), (S.TRAIN_STEP, v_u256(self.opt.step_count)),
                          (S.TRAIN_ADAPTER, bytes(16) + aid)])

    def load_checkpoint(self, store, facts, ckpt: bytes) -> None:
        self.opt.load_state_bytes(bytes(store.get(facts.one(ckpt, S.TRAIN_STATE))))
        assert self.opt.step_count == r_u256(facts.one(ckpt, S.TRAIN_STEP))
        torch.set_rng_state(torch.from_numpy(np.frombuffer(bytes(store.get(facts.one(ckpt, S.TRAIN_RUN))), dtype=np.uint8).copy()))
