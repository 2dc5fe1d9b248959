"""LoRA adapters for the Gemma-4 decoder and their training forward.

Reference: src/models/gemma/lora.rs — ``LoraAdapter{A[r,in] ~ U(+-sqrt(3/in)), B[out,r] = 0, scale = alpha/r}`` (:59-89),
targets q,k,v,o,gate,up,down (:106-158), ``y = base + (x A^T B^T) * scale`` (:413-428), PEFT safetensors names (:180-290),
pile schema ``lora_rank/alpha/adapter/projection/a/b`` (:34-57,297-407).

Tensor parallel layout: a column-parallel projection shards ``B`` by output rows and replicates ``A`` (its gradient is a
partial sum over the group); a row-parallel projection shards ``A`` by input columns and replicates ``B``, and the adapter's
contribution is added to the rank's partial sum BEFORE the group reduction, so the adapters need no collective of their own
in the forward pass."""
from __future__ import annotations

import math

import numpy as np
import torch
from torch import nn

from ..format import schema as S
from ..format.leaf import put_array, resolve
from ..ops import reference as ref
from ..ops.autograd import copy_to_tp, linear_frozen, reduce_from_tp
from ..pile.trible import TribleBuilder, r_f64, r_genid, r_shortstring, r_u256, v_f64, v_genid, v_shortstring, v_u256

PROJECTIONS = ("q_proj", "k_proj", "v_proj", "o_proj", "gate_proj", "up_proj", "down_proj")


class LoraAdapter(nn.Module):
    def __init__(self, in_features: int, out_features: int, rank: int, alpha: float, device="cpu", generator=None):
        super().__init__()
        bound = math.sqrt(3.0 / in_features)
        a = torch.empty(rank, in_features, dtype=torch.float32, device=device).uniform_(-bound, bound, generator=generator)
        self.A = nn.Parameter(a)
        self.B = nn.Parameter(torch.zeros(out_features, rank, dtype=torch.float32, device=device))
        self.scale = alpha / rank

    def forward(self, x):
        return ((x.float() @ self.A.t()) @ self.B.t() * self.scale).to(x.dtype)


class LoraWeights(nn.Module):
    """Adapters of every target projection of every layer: ``adapters[f"{layer}.{proj}"]``."""

    def __init__(self, rank: int, alpha: float):
        super().__init__()
        self.rank, self.alpha = rank, alpha
        self.adapters = nn.ModuleDict()

    @staticmethod
    def init_gemma4(model, rank: int = 16, alpha: float = 32.0, seed: int = 0, targets=PROJECTIONS) -> "LoraWeights":
        cfg, tp = model.cfg, model.tp
        dev = model.embed.device
        g = torch.Generator(device=dev).manual_seed(seed)
        lw = LoraWeights(rank, alpha)
        H = cfg.hidden_size
        for i, L in enumerate(model.layers):
            D = cfg.layer_head_dim(i)
            shapes = {"q_proj": (H, L.n_q * D), "k_proj": (H, L.n_kv * D), "v_proj": (H, L.n_kv * D), "o_proj": (L.n_q * D, H),
                      "gate_proj": (H, L.F), "up_proj": (H, L.F), "down_proj": (L.F, H)}
            for p in targets:
                fin, fout = shapes[p]
                lw.adapters[f"{i}_{p}"] = LoraAdapter(fin, fout, rank, alpha, dev, g)
        return lw

    def get(self, layer: int, proj: str):
        k = f"{layer}_{proj}"
        return self.adapters[k] if k in self.adapters else None

    @staticmethod
    def tp_replicated(proj: str, which: str, kv_replicated: bool = False) -> bool:
        """Whether factor ``which`` ("A" / "B") of a ``proj`` adapter is held identically by every tensor-parallel rank (its
        gradient is then a partial sum over the group) or is a shard (its gradient is complete on its rank).  ``kv_replicated``:
        the model has fewer kv heads than ranks, so the k / v projections themselves are replicated."""
        if proj in ("o_proj", "down_proj"):
            return which == "B"
        if proj in ("k_proj", "v_proj") and kv_replicated:
            return True
        return which == "A"

    @staticmethod
    def shard_from_full(full: "LoraWeights", model, full_model) -> "LoraWeights":
        """The adapters of tensor-parallel rank ``model.tp.rank`` cut out of unsharded ones, by the rule that cuts the base weights
        (``models.gemma4.weights.shard_from_full``): column-parallel ``B`` by output rows (whole heads), row-parallel ``A`` by
        input columns, the other factor copied."""
        have = {k.split("_", 1)[1] for k in full.adapters}
        lw = LoraWeights.init_gemma4(model, full.rank, full.alpha, targets=tuple(p for p in PROJECTIONS if p in have))   # one order on every rank
        r, n = model.tp.rank, model.tp.size
        with torch.no_grad():
            for i, (L, Fl) in enumerate(zip(model.layers, full_model.layers)):
                D = L.D
                kv0 = (r * Fl.n_kv) // n if Fl.n_kv >= n else 0
                rows = {"q_proj": (r * L.n_q * D, L.n_q * D), "k_proj": (kv0 * D, L.n_kv * D), "v_proj": (kv0 * D, L.n_kv * D),
                        "gate_proj": (r * L.F, L.F), "up_proj": (r * L.F, L.F)}
                cols = {"o_proj": (r * L.n_q * D, L.n_q * D), "down_proj": (r * L.F, L.F)}
                for p in PROJECTIONS:
                    src, dst = full.get(i, p), lw.get(i, p)
                    if src is None:
                        continue
                    if p in rows:
                        o, k = rows[p]
                        dst.A.copy_(src.A)
                        dst.B.copy_(src.B[o:o + k])
                    else:
                        o, k = cols[p]
                        dst.A.copy_(src.A[:, o:o + k])
                        dst.B.copy_(src.B)
        return lw

    # ------------------------------------------------------------------ persistence
    def peft_state_dict(self) -> dict:
        out = {}
        for k, ad in self.adapters.items():
            i, p = k.split("_", 1)
            blk = "self_attn" if p in ("q_proj", "k_proj", "v_proj", "o_proj") else "mlp"
            base = f"base_model.model.model.layers.{i}.{blk}.{p}"
            out[base + ".lora_A.weight"] = ad.A.detach().cpu().numpy()
            out[base + ".lora_B.weight"] = ad.B.detach().cpu().numpy()
        return out

    def save_safetensors(self, path: str) -> None:
        from ..format.safetensors import save_file
        save_file(self.peft_state_dict(), path, metadata={"lora_rank": self.rank, "lora_alpha": self.alpha})

    def load_safetensors(self, path: str) -> None:
        from ..format.safetensors import SafeTensors
        st = SafeTensors(path)
        for name, arr in self.peft_state_dict().items():
            src = torch.from_numpy(np.array(st.array(name)))
            i = name.split(".layers.")[1].split(".")[0]
            p = name.split(".")[-3]
            ad = self.adapters[f"{i}_{p}"]
            (ad.A if "lora_A" in name else ad.B).data.copy_(src)

    def save_to_pile(self, store, tb: TribleBuilder, model_root: bytes | None = None) -> bytes:
        aid = tb.entity([(S.LORA_RANK, v_u256(self.rank)), (S.LORA_ALPHA, v_f64(self.alpha))] +
                        ([(S.OWNER, v_genid(model_root))] if model_root else []))
        for k, ad in self.adapters.items():
            a = put_array(store, tb, ad.A.detach().cpu().numpy())
            b = put_array(store, tb, ad.B.detach().cpu().numpy())
            tb.entity([(S.LORA_ADAPTER, v_genid(aid)), (S.LORA_PROJECTION, v_shortstring(k)), (S.LORA_A, v_genid(a)),
                       (S.LORA_B, v_genid(b))])
        return aid

    def load_from_pile(self, store, facts, adapter_id: bytes) -> None:
        assert r_u256(facts.one(adapter_id, S.LORA_RANK)) == self.rank
        for e in facts.entities_where(S.LORA_ADAPTER, v_genid(adapter_id)):
            k = r_shortstring(facts.one(e, S.LORA_PROJECTION))
            ad = self.adapters[k]
            ad.A.data.copy_(torch.from_numpy(np.array(resolve(store, facts, r_genid(facts.one(e, S.LORA_A))).to_f32())))
            ad.B.data.copy_(torch.from_numpy(np.array(resolve(store, facts, r_genid(facts.one(e, S.LORA_B))).to_f32())))


class Gemma4LoraForward(nn.Module):
    """Training forward of the Gemma-4 decoder over whole sequences ``ids[B, S]`` with frozen base weights.

    The base projections run through the hand-written GEMM (``linear_frozen``: forward and input-gradient); norms, RoPE and
    the causal (sliding-window) attention are differentiable PyTorch code, the adapters plain autograd parameters."""

    def __init__(self, model, lora: LoraWeights):
        super().__init__()
        self.model, self.lora = model, lora
        self._wt: dict[int, torch.Tensor] = {}

    def _lin(self, x, w):
        wt = self._wt.get(id(w))
        if wt is None:
            wt = w.detach().t().contiguous()
            self._wt[id(w)] = wt
        return linear_frozen(x, w.detach(), wt)

    def _attn(self, q, k, v, window):
        """q [B,S,Hq,D], k/v [B,S,Hkv,D]; scale 1.0; causal, optional sliding window.  Global layers take the fused causal path
        (no mask tensor, no materialised scores).  Sliding layers attend chunk by chunk: queries of chunk ``c`` (``window``
        tokens) can only see keys of chunks ``c - 1`` and ``c``, so the scores are ``[W, 2W]`` blocks instead of ``[S, S]``."""
        B, Sq, Hq, D = q.shape
        g = Hq // k.shape[2]
        qt = q.transpose(1, 2)
        kt, vt = k.transpose(1, 2), v.transpose(1, 2)
        sdpa = torch.nn.functional.scaled_dot_product_attention
        if not window or window >= Sq:
            return sdpa(qt, kt, vt, is_causal=True, scale=1.0, enable_gqa=g > 1).transpose(1, 2)
        W = window
        outs = []
        for c0 in range(0, Sq, W):
            c1 = min(c0 + W, Sq)
            k0 = max(0, c0 - W)
            qpos = torch.arange(c0, c1, device=q.device)
            kpos = torch.arange(k0, c1, device=q.device)
            mask = (kpos[None, :] <= qpos[:, None]) & ((qpos[:, None] - kpos[None, :]) < W)
            outs.append(sdpa(qt[:, :, c0:c1], kt[:, :, k0:c1], vt[:, :, k0:c1], attn_mask=mask, scale=1.0, enable_gqa=g > 1))
        return torch.cat(outs, 2).transpose(1, 2)

    def _layer(self, i, h, pos, B, Sq):
        m, c = self.model, self.model.cfg
        L = m.layers[i]
        if L.kv_source is not None or L.moe or L.ple:
            raise NotImplementedError("LoRA training of decoders with KV-shared layers, a routed-expert block or per-layer embeddings is not built")
        ad = lambda p: self.lora.get(i, p)  # noqa: E731
        # tensor parallel: the normed activation enters the sharded region (its gradient is summed over the group), the partial
        # sums of the row-parallel projections leave it through the group reduction
        x = copy_to_tp(ref.rmsnorm(h, L.ln_in.detach(), c.rms_norm_eps), m.tp)
        qkv = self._lin(x, L.w_qkv)
        nq, nkv, D = L.n_q * L.D, L.n_kv * L.D, L.D
        deltas = [ad(p)(x) if ad(p) is not None else None for p in ("q_proj", "k_proj", "v_proj")]
        q, k, v = qkv.split([nq, nkv, nkv], -1)
        q = q + deltas[0] if deltas[0] is not None else q
        k = k + deltas[1] if deltas[1] is not None else k
        v = v + deltas[2] if deltas[2] is not None else v
        q = ref.rmsnorm(q.reshape(B * Sq, L.n_q, D), L.q_norm.detach(), c.rms_norm_eps)
        k = ref.rmsnorm(k.reshape(B * Sq, L.n_kv, D), L.k_norm.detach(), c.rms_norm_eps)
        v = ref.rmsnorm(v.reshape(B * Sq, L.n_kv, D), None, c.rms_norm_eps)
        q, k = ref.rope(q, pos, L.inv_freq), ref.rope(k, pos, L.inv_freq)
        o = self._attn(q.view(B, Sq, L.n_q, D), k.view(B, Sq, L.n_kv, D), v.view(B, Sq, L.n_kv, D), L.window)
        o = o.reshape(B, Sq, nq)
        a = self._lin(o, L.w_o)
        if ad("o_proj") is not None:
            a = a + ad("o_proj")(o)
        a = reduce_from_tp(a, m.tp)
        h = h + ref.rmsnorm(a, L.ln_post_attn.detach(), c.rms_norm_eps)
        x = copy_to_tp(ref.rmsnorm(h, L.ln_pre_ffn.detach(), c.rms_norm_eps), m.tp)
        gu = self._lin(x, L.w_gu)
        g_, u_ = gu[..., :L.F], gu[..., L.F:]
        if ad("gate_proj") is not None:
            g_ = g_ + ad("gate_proj")(x)
        if ad("up_proj") is not None:
            u_ = u_ + ad("up_proj")(x)
        mm = ref.geglu(g_, u_)
        d = self._lin(mm, L.w_down)
        if ad("down_proj") is not None:
            d = d + ad("down_proj")(mm)
        d = reduce_from_tp(d, m.tp)
        return (h + ref.rmsnorm(d, L.ln_post_ffn.detach(), c.rms_norm_eps)) * L.layer_scalar

    def forward(self, ids):
        """``checkpoint = True`` keeps only every layer's input for the backward pass and recomputes the layer there: the
        activations of a 4096-token sequence through 48 layers otherwise take on the order of 100 GB."""
        m, c = self.model, self.model.cfg
        B, Sq = ids.shape
        h = (m.embed.detach()[ids.long()].float() * m.embed_scale).to(m.dtype)
        pos = torch.arange(Sq, device=ids.device).repeat(B)
        for i in range(len(m.layers)):
            if getattr(self, "checkpoint", False) and torch.is_grad_enabled():
                from torch.utils.checkpoint import checkpoint
                h = checkpoint(self._layer, i, h, pos, B, Sq, use_reentrant=False)
            else:
                h = self._layer(i, h, pos, B, Sq)
        x = ref.rmsnorm(h, m.norm.detach(), c.rms_norm_eps)
        return x

    def loss(self, ids, chunk: int = 1024):
        """Mean next-token cross-entropy (labels = ids shifted by one); the vocabulary projection is chunked over tokens so
        the [tokens, vocab] logits never exist at once."""
        x = self.forward(ids)[:, :-1].reshape(-1, self.model.cfg.hidden_size)
        y = ids[:, 1:].reshape(-1).long()
        W = self.model.head_weight().detach()
        cap = self.model.cfg.final_logit_softcapping
        total = x.new_zeros((), dtype=torch.float32)
        for i in range(0, x.shape[0], chunk):
            lg = self._lin(x[i:i + chunk], W).float()
            lg = cap * torch.tanh(lg / cap)
            total = total + torch.nn.functional.cross_entropy(lg, y[i:i + chunk], reduction="sum")
        return total / x.shape[0]
