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
from ..ops.autograd import copy_to_tp, reduce_from_tp
from ..pile.trible import TribleBuilder, r_genid, r_shortstring, r_u256, v_f64, v_genid, v_shortstring, v_u256

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

    def num_params(self) -> int:
        """Trainable scalars over all adapters (src/models/gemma/lora.rs:166-178)."""
        return sum(ad.A.numel() + ad.B.numel() for ad in self.adapters.values())

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

    Every linear layer is a ``train_ops.LoraLinear`` (the adapters folded into the base GEMMs, forward and backward on the
    hand-written GEMM, weight gradients by a streaming kernel); norms, the q / k / v head norm with rotation and GeGLU are
    ``train_ops`` functions with a forward and a backward kernel each; the attention itself is PyTorch's fused causal attention.
    The widened operands REPLACE the model's own weight storage (the parameters become views of them)."""

    def __init__(self, model, lora: LoraWeights):
        super().__init__()
        from ..ops.train_ops import LoraLinear
        self.model, self.lora = model, lora
        self._wt: dict[int, torch.Tensor] = {}
        self._flash = None                     # None: not tried yet; True / False: the flash-attention library works / does not
        # (rank, world, group) of a sequence-parallel group, or None: every rank then runs the layers on its contiguous chunk of
        # the sequence's rows, attention goes through two all-to-alls (rows <-> heads, ``parallel.seq_attention``), the loss is
        # normalised by the tokens of the whole sequence, and the caller sums the adapter gradients over the group
        self.sp = None
        self.fused: list[dict] = []
        s = lora.alpha / lora.rank
        for i, L in enumerate(model.layers):
            if L.kv_source is not None or L.moe or L.ple:
                raise NotImplementedError("LoRA training of decoders with KV-shared layers, a routed-expert block or per-layer embeddings is not built")
            ad = lambda p: lora.get(i, p)  # noqa: E731
            nq, nkv, F = L.n_q * L.D, L.n_kv * L.D, L.F
            f = {"qkv": LoraLinear(L.w_qkv, [(ad("q_proj"), 0, nq), (ad("k_proj"), nq, nkv), (ad("v_proj"), nq + nkv, nkv)], s),
                 "o": LoraLinear(L.w_o, [(ad("o_proj"), 0, L.w_o.shape[0])], s),
                 "gu": LoraLinear(L.w_gu, [(ad("gate_proj"), 0, F), (ad("up_proj"), F, F)], s),
                 "down": LoraLinear(L.w_down, [(ad("down_proj"), 0, L.w_down.shape[0])], s)}
            for name, key in (("w_qkv", "qkv"), ("w_o", "o"), ("w_gu", "gu"), ("w_down", "down")):
                getattr(L, name).data = f[key].base_view()          # one copy of every base weight stays alive
            self.fused.append(f)

    def refresh(self):
        """Copy the adapters' master parameters into the widened GEMM operands (after every optimiser step)."""
        for f in self.fused:
            for m in f.values():
                m.refresh()

    def _attn(self, q, k, v, window):
        """q [B,S,Hq,D], k/v [B,S,Hkv,D]; scale 1.0; causal, optional sliding window.  Global layers take the fused causal path
        (no mask tensor, no materialised scores).  Sliding layers attend chunk by chunk: queries of chunk ``c`` (``window``
        tokens) can only see keys of chunks ``c - 1`` and ``c``, so the scores are ``[W, 2W]`` blocks instead of ``[S, S]``."""
        B, Sq, Hq, D = q.shape
        g = Hq // k.shape[2]
        if self.sp is not None and not getattr(self, "_inside_sp", False):
            # rows -> heads: this rank attends the WHOLE sequence for its share of the heads with the local attention below
            from ..parallel.seq_attention import ulysses_attention
            rank, world, group = self.sp

            def local(qh, kh, vh, scale, causal, w):
                self._inside_sp = True
                try:
                    return self._attn(qh[None], kh[None], vh[None], w)[0]
                finally:
                    self._inside_sp = False
            return torch.stack([ulysses_attention(q[b], k[b], v[b], rank, world, group, scale=1.0, causal=True, window=window, attn_fn=local)
                                for b in range(B)])
        if q.is_cuda and q.dtype in (torch.bfloat16, torch.float16) and D <= 256 and self._flash is not False:
            # the flash-attention library where the machine has it: grouped heads and the sliding window natively, forward and
            # backward on tensor cores (PyTorch's fused attention refuses masks together with grouped heads and falls back to
            # f32 matrix products for the sliding layers)
            try:
                from flash_attn import flash_attn_func
                o = flash_attn_func(q, k, v, softmax_scale=1.0, causal=True,
                                    window_size=(window - 1, 0) if window and window < Sq else (-1, -1))
                self._flash = True
                return o
            except Exception:
                if self._flash:
                    raise
                self._flash = False
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
        """``h [B * Sq, H]`` -> the residual stream after layer ``i``."""
        from ..ops import train_ops as T
        m, c = self.model, self.model.cfg
        L, f = m.layers[i], self.fused[i]
        eps = c.rms_norm_eps
        nq, nkv, D = L.n_q * L.D, L.n_kv * L.D, L.D
        # tensor parallel: the normed activation enters the sharded region (its gradient is summed over the group), the partial
        # sums of the row-parallel projections leave it through the group reduction
        x = copy_to_tp(T.rmsnorm(h, L.ln_in, eps, out_extra=f["qkv"].R), m.tp)
        qkv = f["qkv"](x)
        qkv = T.qkv_norm_rope(qkv, pos, L.inv_freq, L.q_norm, L.k_norm, eps, L.n_q, L.n_kv, D, grad_extra=f["qkv"].R)
        q, k, v = qkv.split([nq, nkv, nkv], -1)
        o = self._attn(q.view(B, Sq, L.n_q, D), k.view(B, Sq, L.n_kv, D), v.view(B, Sq, L.n_kv, D), L.window)
        a = reduce_from_tp(f["o"](o.reshape(B * Sq, nq)), m.tp)
        h = T.rmsnorm(a, L.ln_post_attn, eps, res=h)
        x = copy_to_tp(T.rmsnorm(h, L.ln_pre_ffn, eps, out_extra=f["gu"].R), m.tp)
        gu = f["gu"](x)
        mm = T.geglu(gu, out_extra=f["down"].R, grad_extra=f["gu"].R)
        d = reduce_from_tp(f["down"](mm), m.tp)
        return T.rmsnorm(d, L.ln_post_ffn, eps, res=h, alpha=float(L.layer_scalar))

    def forward(self, ids):
        """``checkpoint = True`` keeps only every layer's input for the backward pass and recomputes the layer there: the
        activations of a 4096-token sequence through 48 layers otherwise take on the order of 100 GB."""
        m, c = self.model, self.model.cfg
        p0 = 0
        if self.sp is not None:
            rank, world, _ = self.sp
            if ids.shape[1] % world:
                raise ValueError(f"a sequence of {ids.shape[1]} tokens cannot be cut into {world} equal chunks")
            n = ids.shape[1] // world
            p0 = rank * n
            ids = ids[:, p0:p0 + n]
        B, Sq = ids.shape
        self.refresh()
        h = (m.embed.detach()[ids.long()].float() * m.embed_scale).to(m.dtype).view(B * Sq, -1)
        pos = torch.arange(p0, p0 + Sq, device=ids.device, dtype=torch.int32).repeat(B)
        for i in range(len(m.layers)):
            if getattr(self, "checkpoint", False) and torch.is_grad_enabled():
                from torch.utils.checkpoint import checkpoint
                h = checkpoint(self._layer, i, h, pos, B, Sq, use_reentrant=False)
            else:
                h = self._layer(i, h, pos, B, Sq)
        from ..ops import train_ops as T
        return T.rmsnorm(h, m.norm, c.rms_norm_eps).view(B, Sq, -1)

    def loss(self, ids, chunk: int = 1024):
        """Mean next-token cross-entropy (labels = ids shifted by one); the vocabulary projection is chunked over tokens so
        the [tokens, vocab] logits never exist at once."""
        if self.sp is not None:
            return self._loss_sp(ids, chunk)
        x = self.forward(ids)[:, :-1].reshape(-1, self.model.cfg.hidden_size)
        y = ids[:, 1:].reshape(-1).long()
        W = self.model.head_weight().detach()
        wt = self._wt.get(W.data_ptr())               # keyed by storage: ``detach()`` makes a new tensor object every call
        if wt is None:
            wt = W.t().contiguous()
            self._wt[W.data_ptr()] = wt
        from ..ops import train_ops as T
        return T.head_loss(x.contiguous(), W, wt, y, self.model.cfg.final_logit_softcapping, chunk)

    def _loss_sp(self, ids, chunk: int):
        """This rank's share of the mean next-token cross-entropy: the sum over its rows' tokens divided by the token count of the
        WHOLE sequence, so that the ranks' losses (and adapter gradients) add up to the single-rank values."""
        from ..ops import train_ops as T
        rank, world, _ = self.sp
        B, S = ids.shape
        n = S // world
        p0 = rank * n
        x = self.forward(ids)                                            # [B, n, H]: rows p0 .. p0 + n - 1
        keep = n if p0 + n < S else n - 1                                # the sequence's last row has no label
        x = x[:, :keep].reshape(-1, self.model.cfg.hidden_size)
        y = ids[:, p0 + 1:p0 + 1 + keep].reshape(-1).long()
        W = self.model.head_weight().detach()
        wt = self._wt.get(W.data_ptr())
        if wt is None:
            wt = W.t().contiguous()
            self._wt[W.data_ptr()] = wt
        total = B * (S - 1)
        return T.head_loss(x.contiguous(), W, wt, y, self.model.cfg.final_logit_softcapping, chunk) * (x.shape[0] / total)
