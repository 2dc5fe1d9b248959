"""The Inkling decoder as the reference defines it, on the package's paged runtime (GPU kernels or CPU oracles behind ``ops``).

Reference: layer with four additive paths and three stateful ones (src/models/inkling/layer.rs:8-174), attention with K / V
short convolutions, per-head norms, rank-``d_rel`` relative bias and log scaling (attn.rs:130-492), sigmoid router whose
weights are a softmax over the log-sigmoids of the chosen experts AND the shared-expert sinks (block.rs:140-250), dense MLP
with a global scale (mlp.rs:69-87), stack ends (stack.rs:1-121), MTP heads (mtp.rs:1-244), the device lane with its
speculative rollback (burn.rs:381-481 ``AttnCache::commit``) and slot caches (burn.rs:1415-1473).

Differences of design, not of arithmetic:

* K / V live in the paged cache; rows past a sequence's committed length are simply overwritten, so rejected speculative rows
  leave no trace without a ``Pending`` region.
* the four short convolutions keep their histories in small POSITION-INDEXED rings per slot (``ring[slot, pos % RING]`` holds the
  pre-convolution row of position ``pos``): a step reads the ``taps - 1`` rows before its first position from the ring and the
  rest from its own batch rows, then writes its rows.  Rolling back is therefore also free: the next step rewrites the
  rejected positions, and the rows it reads as history are positions it has committed.  ``RING`` must cover ``taps - 1`` history
  rows plus the widest decode step.
* parameters are kept under their CHECKPOINT names (``models.inkling.layout``), so loading is filling a dictionary and the
  layout gate is the loader's completeness check.

Expert weights: a quantised layer holds packed NVFP4 experts (``ops.moe.NVFP4Experts``: activations are re-quantised before
each GEMM as in src/bin/inkling_forward.rs:2355-2434), a bf16 layer holds ``[E, 2F, H]`` / ``[E, H, F]`` tensors and runs the
grouped bf16 lane (moegroup.rs:556-719); the shared experts are bf16 and weighted by their router gammas."""
from __future__ import annotations

import torch
import torch.nn.functional as F

from ... import ops
from ...ops import reference as ref
from ...ops.moe import NVFP4Experts, experts_forward
from . import layout as L
from .config import GLOBAL, LOCAL, InklingConfig
from .ops import log_scale_tau

RING = 16


def conv_ring(x, w, ring, slots, meta):
    """``y = x + depthwise_causal_conv(x)`` over the rows of a flattened batch with the history taken from (and the rows written
    to) the position ring.  ``x [T, C]``; ``w [C, taps]`` (tap ``taps - 1`` multiplies the current row, block.rs:48-127);
    ``ring [slots + 1, RING, C]`` (the last row is a spare that takes the writes of rows too old to keep); ``slots [S]`` int64 ring
    row of every sequence of the batch."""
    T, C = x.shape
    taps = w.shape[1]
    pos = meta.positions.long()
    seq = meta.seq_index.long()
    first = (meta.kv_len.long() - (meta.q_start[1:] - meta.q_start[:-1]).long())[seq]      # position of the sequence's first row of this batch
    off = pos - first                                                                      # row offset within its sequence's rows
    slot = slots.long()[seq]
    wf = w.float()
    xf = x.float()
    acc = xf * (1.0 + wf[:, taps - 1])
    rows = torch.arange(T, device=x.device)
    for j in range(taps - 1):
        d = taps - 1 - j                                         # this tap reads the row d positions back
        in_batch = off >= d
        src = (rows - d).clamp_min(0)
        p = pos - d
        hist = ring[slot, p.clamp_min(0) % ring.shape[1]].float()
        hist = torch.where((p >= 0)[:, None], hist, torch.zeros_like(hist))              # zero padding before the sequence start
        tap = torch.where(in_batch[:, None], xf[src], hist)
        acc = acc + tap * wf[:, j]
    # only the last RING rows of a long chunk may be written (earlier ones would collide in the ring)
    n_rows = (meta.q_start[1:] - meta.q_start[:-1]).long()[seq]
    # rows that may not be written go to the spare ring row behind the last slot instead: no data-dependent shapes, so the step
    # can be captured in a CUDA graph
    keep = off >= n_rows - ring.shape[1]
    ring.index_put_((torch.where(keep, slot, ring.shape[0] - 1), pos % ring.shape[1]), x.to(ring.dtype))
    return acc.to(x.dtype)


class InklingDecoder(torch.nn.Module):
    def __init__(self, cfg: InklingConfig, quantized: set | None = None, dtype=torch.bfloat16, device="cpu", max_slots: int = 8,
                 w13_interleaved: bool = False):
        super().__init__()
        self.cfg, self.t = cfg, cfg.text_config
        t = self.t
        self.dtype, self.dev = dtype, torch.device(device)
        self.quantized = {i for i in range(t.num_hidden_layers) if not t.is_dense(i)} if quantized is None else set(quantized)
        self.w13_interleaved = w13_interleaved
        self.n_llm, self.n_mtp = t.num_hidden_layers, cfg.mtp_config.num_nextn_predict_layers
        self.P: dict[str, torch.Tensor] = {}                 # checkpoint name -> tensor (bf16 / f32), see layout.slots
        self.experts: dict[int, NVFP4Experts] = {}           # quantised MoE layers
        self.max_slots = max_slots
        self.rings: list[dict] = []                          # per block: {"k", "v", "attn", "mlp"} rings
        self._derived: dict = {}
        self.slots_default = torch.arange(max_slots, device=self.dev)
        kinds = [t.attn_kind(i) for i in range(self.n_llm)] + [cfg.mtp_config.attn_kind(i) for i in range(self.n_mtp)]
        self.kinds = kinds
        for kind in kinds:
            kv = t.kv_dim(kind)
            z = lambda c: torch.zeros(max_slots + 1, RING, c, dtype=dtype, device=self.dev)  # noqa: E731
            self.rings.append({"k": z(kv), "v": z(kv), "attn": z(t.hidden_size), "mlp": z(t.hidden_size)})

    # ------------------------------------------------------------------ parameters
    def expected(self):
        """``(slot, name, shape, dtype)`` of every TEXT tensor this decoder reads (the vision / audio towers are separate modules)."""
        return [s for s in L.slots(self.cfg, self.quantized) if s[0][0] not in ("vision", "audio")]

    def init_random_(self, seed: int = 0, std: float = 0.05):
        g = torch.Generator().manual_seed(seed)
        t = self.t
        for slot, name, shape, dt in self.expected():
            if slot[0] in ("llm", "mtp") and "expert" in slot and slot[-1] != "weight":
                continue                                      # sidecars are produced by quantising the bf16 expert weights below
            if name.endswith("norm.weight"):
                v = 1.0 + 0.1 * torch.randn(shape, generator=g)
            elif name.endswith("sconv.weight"):
                v = 0.2 * torch.randn(shape, generator=g)
            elif name.endswith("global_scale"):
                v = torch.full(shape, 1.25)
            elif name.endswith("gate.bias"):
                v = 0.05 * torch.randn(shape, generator=g)
            elif "expert" in slot and slot[-1] == "weight":
                E, H, N = t.n_routed_experts, t.hidden_size, (2 if slot[-2] == "w13" else 1) * t.intermediate_size
                v = std * torch.randn(E, H, N, generator=g)  # logical [experts, hidden, out] whatever the stored dtype
            else:
                v = std * torch.randn(shape, generator=g)
            self.set_tensor(name, v)
        return self

    def set_tensor(self, name: str, value):
        """Install one checkpoint tensor.  Expert matrices arrive in their logical bf16 form ``[E, hidden, out]`` (or as the
        packed parts through :meth:`set_experts_nvfp4`) and are stored in the layout the GEMMs read."""
        slot = L.parse(name)
        if slot is None:
            raise KeyError(f"not an Inkling tensor name: {name}")
        f32 = name.endswith(("gate.bias", "gate.global_scale")) or name.endswith(".scale2")
        v = torch.as_tensor(value)
        if "expert" in slot and slot[-1] == "weight" and slot[0] == "llm":
            layer, mat = slot[1], slot[-2]
            w = v.to(torch.float32).transpose(1, 2).contiguous()            # [E, out, hidden] = the GEMMs' [N, K]
            if mat == "w13" and self.w13_interleaved:                        # gate / up rows interleaved -> halved [gate; up]
                w = torch.cat([w[:, 0::2], w[:, 1::2]], 1).contiguous()
            self._derived.setdefault(("expert_dense", layer), {})[mat] = w.to(self.dtype).to(self.dev)
            self._derived.pop(("packed", layer), None)
            return
        self.P[name] = v.to(torch.float32 if f32 else self.dtype).to(self.dev)
        self._derived.pop(name, None)

    def _experts(self, layer: int):
        """Packed NVFP4 experts of a quantised layer (built from the bf16 tensors on first use), or the bf16 pair."""
        d = self._derived[("expert_dense", layer)]
        if layer not in self.quantized:
            return d["w13"], d["w2"]
        key = ("packed", layer)
        if key not in self._derived:
            self._derived[key] = NVFP4Experts.from_dense(d["w13"].float(), d["w2"].float(), act="swiglu")
        return self._derived[key]

    def set_experts_nvfp4(self, layer: int, ex: NVFP4Experts):
        self._derived[("packed", layer)] = ex
        self._derived.setdefault(("expert_dense", layer), {})

    def kv_spec(self) -> dict:
        t = self.t
        return dict(num_layers=self.n_llm + self.n_mtp, kv_heads=[t.heads(k)[1] for k in self.kinds], head_dim=[t.heads(k)[2] for k in self.kinds])

    # ------------------------------------------------------------------ blocks
    def _w(self, prefix: str, part: tuple):
        return self.P[prefix + L._block_name(part)]

    def _attention(self, prefix: str, bi: int, x, meta, cache, slots):
        t, kind = self.t, self.kinds[bi]
        Hq, Hkv, D = t.heads(kind)
        dr, T = t.d_rel, x.shape[0]
        key = prefix + "qkvr"
        if key not in self._derived:
            self._derived[key] = (torch.cat([self._w(prefix, ("attn", a)) for a in ("wq", "wk", "wv", "wr")], 0).contiguous(),
                                  self._w(prefix, ("attn", "rel_proj")).t().contiguous())
        w_qkvr, rel_w = self._derived[key]
        y = ops.linear(x, w_qkvr)
        q, k, v, r = y.split([Hq * D, Hkv * D, Hkv * D, Hq * dr], -1)
        rg = self.rings[bi]
        k = conv_ring(k.contiguous(), self._w(prefix, ("attn", "k_sconv"))[:, 0, :], rg["k"], slots, meta)
        v = conv_ring(v.contiguous(), self._w(prefix, ("attn", "v_sconv"))[:, 0, :], rg["v"], slots, meta)
        qkv = torch.cat([q, k, v], -1).contiguous()
        qn = ops.qk_norm_rope_append(qkv, Hq, Hkv, D, self._w(prefix, ("attn", "q_norm")), self._w(prefix, ("attn", "k_norm")), False, None,
                                     meta, cache.k[bi], cache.v[bi], t.rms_norm_eps)
        rel = ops.linear(r.reshape(T * Hq, dr).contiguous(), rel_w).float().view(T, Hq, -1)
        if kind == GLOBAL and t.log_scaling_alpha:
            tau = log_scale_tau(meta.positions, t.log_scaling_alpha, max(t.log_scaling_n_floor, 1)).to(x.device)
            qn = (qn.float() * tau[:, None, None]).to(qn.dtype)
            rel = rel * tau[:, None, None]
        o = ops.paged_attention(qn, cache.k[bi], cache.v[bi], meta, 1.0 / D, t.sliding_window_size if kind == LOCAL else 0,
                                rel_bias=rel.contiguous())
        return ops.linear(o.reshape(T, Hq * D), self._w(prefix, ("attn", "wo")))

    def _scalar(self, name: str) -> float:
        """A scalar parameter as a Python float, read from the device once (never inside a captured step)."""
        key = ("scalar", name)
        if key not in self._derived:
            self._derived[key] = float(self.P[name].float().reshape(-1)[0])
        return self._derived[key]

    def _dense_mlp(self, prefix: str, y):
        gs = self._scalar(prefix + "mlp.global_scale") if self.t.use_global_scale else 1.0
        h = ops.linear_glu(y, self._w(prefix, ("mlp", "dense", "w13")), "swiglu")
        out = ops.linear(h, self._w(prefix, ("mlp", "dense", "w2")))
        return out if gs == 1.0 else (out.float() * gs).to(out.dtype)

    def route(self, prefix: str, y):
        """``(idx [T, k], w [T, k], gammas [T, n_shared])`` by the reference's rule (block.rs:140-250)."""
        t = self.t
        logits = ops.linear_f32(y, self._w(prefix, ("mlp", "moe", "gate_weight")))
        n_r = t.n_routed_experts
        lr = logits[:, :n_r]
        bias = self._w(prefix, ("mlp", "moe", "gate_bias")) if t.use_gate_bias else torch.zeros(n_r, device=y.device)
        sel = torch.sigmoid(lr) + bias.float()
        _, idx = ref.topk_first(sel, t.num_experts_per_tok)
        chosen = lr.gather(-1, idx)
        sinks = logits[:, n_r:] if t.shared_expert_sink else logits.new_zeros(logits.shape[0], t.n_shared_experts)
        pool = torch.cat([F.logsigmoid(chosen), F.logsigmoid(sinks)], -1)
        gs = self._scalar(prefix + "mlp.gate.global_scale") if t.use_global_scale else 1.0
        w = torch.softmax(pool, -1) * (t.route_scale * gs)
        k = t.num_experts_per_tok
        return idx.int(), w[:, :k].contiguous(), w[:, k:].contiguous()

    def _moe(self, prefix: str, layer: int, y):
        t = self.t
        idx, w, gam = self.route(prefix, y)
        T = y.shape[0]
        key = prefix + "shared"
        if key not in self._derived:                          # shared experts [n, hidden, out] -> [n, out, hidden]
            self._derived[key] = (self._w(prefix, ("mlp", "moe", "shared_w13")).transpose(1, 2).contiguous(),
                                  self._w(prefix, ("mlp", "moe", "shared_w2")).transpose(1, 2).contiguous())
        s13, s2 = self._derived[key]
        sh_idx = torch.arange(t.n_shared_experts, dtype=torch.int32, device=y.device)[None].expand(T, -1).contiguous()
        shared = ops.bf16_experts(y, sh_idx, gam.to(torch.float32), s13, s2, 0, "swiglu")
        ex = self._experts(layer)
        if isinstance(ex, NVFP4Experts):
            return experts_forward(y, idx, w.float(), ex, shared)
        return (ops.bf16_experts(y, idx, w.float(), ex[0], ex[1], 0, "swiglu").float() + shared.float()).to(y.dtype)

    def block(self, prefix: str, bi: int, layer: int, dense: bool, h, meta, cache, slots):
        """``h += sconv_attn(attn(rms(h)))``; ``h += sconv_mlp(mlp(rms(h)))`` (layer.rs:8-174).  ``bi``: cache / ring index of the block."""
        eps, rg = self.t.rms_norm_eps, self.rings[bi]
        a = self._attention(prefix, bi, ops.rmsnorm(h, self._w(prefix, ("attn_norm",)), eps), meta, cache, slots)
        a = conv_ring(a, self._w(prefix, ("attn_sconv",))[:, 0, :], rg["attn"], slots, meta)
        h = (h.float() + a.float()).to(h.dtype)
        y = ops.rmsnorm(h, self._w(prefix, ("mlp_norm",)), eps)
        m = self._dense_mlp(prefix, y) if dense else self._moe(prefix, layer, y)
        m = conv_ring(m, self._w(prefix, ("mlp_sconv",))[:, 0, :], rg["mlp"], slots, meta)
        return (h.float() + m.float()).to(h.dtype)

    # ------------------------------------------------------------------ stack
    def embed_in(self, ids):
        e = ops.embed(ids, self.P["model.llm.embed.weight"])
        return ops.rmsnorm(e, self.P["model.llm.embed_norm.weight"], self.t.rms_norm_eps) if self.t.use_embed_norm else e

    def trunk(self, ids, meta, cache, slots=None):
        slots = self.slots_default[:meta.num_seqs] if slots is None else slots
        h = self.embed_in(ids)
        for i in range(self.n_llm):
            h = self.block(f"model.llm.layers.{i}.", i, i, self.t.is_dense(i), h, meta, cache, slots)
        return h

    def logits(self, h):
        """final norm, DIVIDE by the muP width multiplier, un-embed, truncate to the real vocabulary (stack.rs:60-121)."""
        x = ops.rmsnorm(h, self.P["model.llm.norm.weight"], self.t.rms_norm_eps)
        m = self.t.logits_mup_width_multiplier or 1.0
        if m != 1.0:
            x = (x.float() / m).to(x.dtype)
        return ops.linear(x, self.P["model.llm.unembed.weight"]).float()[:, :self.t.effective_vocab()]

    def forward(self, ids, meta, cache, rows=None, slots=None):
        h = self.trunk(ids, meta, cache, slots)
        return self.logits(h if rows is None else h[rows])

    def head_argmax(self, h):
        return ref.argmax_first(self.logits(h))

    # ------------------------------------------------------------------ speculative decoding (runtime.spec_decode protocol)
    def _head_rows(self, h, rows):
        """Arg-max token of the rows ``rows`` of ``h`` (None: every row; an empty index: no un-embedding at all)."""
        if rows is not None:
            if rows.numel() == 0:
                return torch.empty(0, dtype=torch.int64, device=h.device)
            h = h[rows]
        return self.head_argmax(h)

    def verify(self, ids, meta, cache, slots=None, rows=None):
        h = self.trunk(ids, meta, cache, slots)
        return self._head_rows(h, rows), h

    def draft(self, d: int, h_prev, next_ids, meta, cache, slots=None, rows=None):
        """MTP head ``d`` over rows ``(hidden of row j, token after row j)``: hidden first in the concatenation (mtp.rs:108-244),
        one DENSE block with its own cache rows and rings, the shared un-embedding."""
        slots = self.slots_default[:meta.num_seqs] if slots is None else slots
        d = min(d, self.n_mtp - 1)
        pre = f"model.mtp.layers.{d}."
        eps = self.t.rms_norm_eps
        e = self.embed_in(next_ids)
        x = torch.cat([ops.rmsnorm(h_prev, self.P[pre + "hidden_norm.weight"], eps), ops.rmsnorm(e, self.P[pre + "embed_norm.weight"], eps)], -1)
        h = ops.linear(x, self.P[pre + "input_proj.weight"])
        h = self.block(pre + "transformer_block.", self.n_llm + d, -1, True, h, meta, cache, slots)
        return self._head_rows(h, rows), h

    def greedy(self, ids, meta, cache, rows, slots=None):
        return self.head_argmax(self.trunk(ids, meta, cache, slots)[rows])


# ---------------------------------------------------------------------------------------------------------------------------------
# The same model through the reference operators of ``models.inkling.ops`` (one sequence at a time, concatenating caches): the oracle
# the paged decoder is compared with, layer by layer.
def reference_params(dec: InklingDecoder, prefix: str, dense: bool, layer: int) -> dict:
    t = dec.t
    g = lambda part: dec._w(prefix, part).float().cpu()  # noqa: E731
    p = {"attn_norm": g(("attn_norm",)), "mlp_norm": g(("mlp_norm",)), "attn_sconv": g(("attn_sconv",))[:, 0, :], "mlp_sconv": g(("mlp_sconv",))[:, 0, :],
         "wq": g(("attn", "wq")), "wk": g(("attn", "wk")), "wv": g(("attn", "wv")), "wo": g(("attn", "wo")), "wr": g(("attn", "wr")),
         "rel_proj": g(("attn", "rel_proj")), "q_norm": g(("attn", "q_norm")), "k_norm": g(("attn", "k_norm")),
         "k_conv": g(("attn", "k_sconv"))[:, 0, :], "v_conv": g(("attn", "v_sconv"))[:, 0, :]}
    if dense:
        w13 = g(("mlp", "dense", "w13"))
        Fd = w13.shape[0] // 2
        p.update(w_gate=w13[:Fd], w_up=w13[Fd:], w_down=g(("mlp", "dense", "w2")))
    return p


def reference_forward(dec: InklingDecoder, ids, caches: list | None = None):
    """Logits of ONE sequence through ``models.inkling.ops`` (f32, CPU).  ``caches``: one dict per LLM layer to continue from."""
    from . import ops as R
    t = dec.t
    P = {k: v.float().cpu() for k, v in dec.P.items()}
    h = P["model.llm.embed.weight"][torch.as_tensor(ids).long()]
    if t.use_embed_norm:
        h = ref.rmsnorm(h, P["model.llm.embed_norm.weight"], t.rms_norm_eps)
    hs = []
    for i in range(dec.n_llm):
        pre = f"model.llm.layers.{i}."
        kind = t.attn_kind(i)
        cfg = t.op_cfg(kind)
        p = reference_params(dec, pre, t.is_dense(i), i)
        cfg["global_scale"] = float(dec._w(pre, ("mlp", "dense", "global_scale")).float().reshape(-1)[0]) if (t.is_dense(i) and t.use_global_scale) else 1.0
        mlp = None
        if not t.is_dense(i):
            def mlp(y, pre=pre, i=i):
                idx, w, gam = dec.route(pre, y.to(dec.dtype).to(dec.dev))
                idx, w, gam = idx.cpu(), w.float().cpu(), gam.float().cpu()
                s13 = dec._w(pre, ("mlp", "moe", "shared_w13")).float().cpu().transpose(1, 2)
                s2 = dec._w(pre, ("mlp", "moe", "shared_w2")).float().cpu().transpose(1, 2)
                Fh = s13.shape[1] // 2
                out = torch.zeros_like(y, dtype=torch.float32)
                for s in range(t.n_shared_experts):
                    hh = F.silu(y.float() @ s13[s, :Fh].t()) * (y.float() @ s13[s, Fh:].t())
                    out += gam[:, s:s + 1] * (hh @ s2[s].t())
                ex = dec._experts(i)
                if isinstance(ex, NVFP4Experts):
                    from ...ops.moe import experts_reference
                    out += experts_reference(y.to(torch.bfloat16), idx, w, ex).float()
                else:
                    w13, w2 = ex[0].float().cpu(), ex[1].float().cpu()
                    Fe = w13.shape[1] // 2
                    for e in idx.unique().tolist():
                        tt, jj = (idx == e).nonzero(as_tuple=True)
                        hh = F.silu(y[tt].float() @ w13[e, :Fe].t()) * (y[tt].float() @ w13[e, Fe:].t())
                        out.index_put_((tt,), (hh @ w2[e].t()) * w[tt, jj][:, None], accumulate=True)
                return out
        h = R.decoder_layer(h, p, cfg, None if caches is None else caches[i], is_global=(kind == GLOBAL), mlp=mlp)
        hs.append(h)
    x = ref.rmsnorm(h, P["model.llm.norm.weight"], t.rms_norm_eps).float() / (t.logits_mup_width_multiplier or 1.0)
    return (x @ P["model.llm.unembed.weight"].t())[:, :t.effective_vocab()], hs
