"""NumPy restatement of the Gemma-4 text decoder — the CPU oracle and timed CPU baseline.

Every step follows the reference's math (src/models/gemma/gemma4/{decoder,layers}.rs, src/models/gemma/rope.rs):

1. ``h0 = E[ids] * sqrt(hidden)`` (decoder.rs:79-80).
2. per layer: ``r=h; a=attn(rms(h,w_in)); h=r+rms(a,w_post_attn); r=h; m=mlp(rms(h,w_pre_ffn));
   h=r+rms(m,w_post_ffn); h*=layer_scalar`` (layers.rs:562-613); RMSNorm uses the gain as stored.
3. attention: learned q_norm/k_norm over head_dim, weightless v_norm, split-half RoPE at absolute positions,
   scale 1.0, causal mask, softmax over keys, GQA by repeating kv heads (layers.rs:90-207,254-262).
4. MLP ``down(gelu_tanh(gate(x)) * up(x))`` (layers.rs:450-469).
5. head: final norm, tied ``h E^T``, ``cap*tanh(logits/cap)`` (decoder.rs:299-319).
6. greedy decode, first maximum wins (lm.rs:22-32).
The sliding window (which the reference's text path leaves out) is applied when ``cfg.apply_sliding_window``."""
from __future__ import annotations

import math

import numpy as np


def rms(x, w, eps):
    y = x * (1.0 / np.sqrt(np.mean(x.astype(np.float32) ** 2, axis=-1, keepdims=True) + np.float32(eps)))
    return (y * w).astype(np.float32) if w is not None else y.astype(np.float32)


def inv_freq(d, theta, partial=1.0):
    j = np.arange(d // 2, dtype=np.float64)
    f = theta ** (-2.0 * j / d)
    f[int(d // 2 * partial):] = 0.0
    return f.astype(np.float32)


def rope(x, pos, invf):
    ang = pos.astype(np.float32)[:, None] * invf[None, :]
    c, s = np.cos(ang)[:, None, :], np.sin(ang)[:, None, :]
    d = x.shape[-1] // 2
    x1, x2 = x[..., :d], x[..., d:]
    return np.concatenate([x1 * c - x2 * s, x1 * s + x2 * c], axis=-1).astype(np.float32)


def gelu_tanh(x):
    return (0.5 * x * (1.0 + np.tanh(np.float32(math.sqrt(2.0 / math.pi)) * (x + np.float32(0.044715) * x ** 3)))).astype(np.float32)


class Gemma4Oracle:
    def __init__(self, cfg, weights: dict):
        self.cfg, self.w = cfg, {k: np.asarray(v, dtype=np.float32) for k, v in weights.items()}
        self.kc = [None] * cfg.num_hidden_layers
        self.vc = [None] * cfg.num_hidden_layers
        self.len = 0

    def forward(self, ids):
        c, w = self.cfg, self.w
        ids = np.asarray(ids, dtype=np.int64)
        S = len(ids)
        pos = np.arange(self.len, self.len + S)
        h = w["model.embed_tokens.weight"][ids] * np.float32(np.float32(math.sqrt(c.hidden_size)))
        for i in range(c.num_hidden_layers):
            p = f"model.layers.{i}."
            D, Hq, Hkv = c.layer_head_dim(i), c.num_attention_heads, c.layer_kv_heads(i)
            x = rms(h, w[p + "input_layernorm.weight"], c.rms_norm_eps)
            q = (x @ w[p + "self_attn.q_proj.weight"].T).reshape(S, Hq, D)
            q = rms(q, w[p + "self_attn.q_norm.weight"], c.rms_norm_eps)
            sliding = c.is_sliding(i)
            f = inv_freq(D, c.rope_theta_local) if sliding else inv_freq(D, c.rope_theta_global, c.partial_rotary_factor_global)
            q = rope(q, pos, f)
            src = c.kv_source(i)
            if src is None:
                k = (x @ w[p + "self_attn.k_proj.weight"].T).reshape(S, Hkv, D)
                vname = p + "self_attn.v_proj.weight"
                v = k.copy() if (c.k_eq_v(i) and vname not in w) else (x @ w[vname].T).reshape(S, Hkv, D)
                k = rope(rms(k, w[p + "self_attn.k_norm.weight"], c.rms_norm_eps), pos, f)
                v = rms(v, None, c.rms_norm_eps)
                self.kc[i] = k if self.kc[i] is None else np.concatenate([self.kc[i], k], 0)
                self.vc[i] = v if self.vc[i] is None else np.concatenate([self.vc[i], v], 0)
            else:                                   # KV-shared layer: the source layer's keys and values, this layer's queries
                self.kc[i], self.vc[i] = self.kc[src], self.vc[src]
            K, V = np.repeat(self.kc[i], Hq // Hkv, axis=1), np.repeat(self.vc[i], Hq // Hkv, axis=1)
            sc = np.einsum("nhd,lhd->hnl", q, K)                       # scale 1.0
            kpos = np.arange(K.shape[0])
            mask = kpos[None, :] <= pos[:, None]
            if sliding and c.apply_sliding_window:
                mask &= (pos[:, None] - kpos[None, :]) < c.sliding_window
            sc = np.where(mask[None], sc, -np.inf)
            sc = sc - sc.max(-1, keepdims=True)
            pr = np.exp(sc)
            pr /= pr.sum(-1, keepdims=True)
            o = np.einsum("hnl,lhd->nhd", pr, V).reshape(S, Hq * D).astype(np.float32)
            a = o @ w[p + "self_attn.o_proj.weight"].T
            h = h + rms(a, w[p + "post_attention_layernorm.weight"], c.rms_norm_eps)
            x = rms(h, w[p + "pre_feedforward_layernorm.weight"], c.rms_norm_eps)
            m = (gelu_tanh(x @ w[p + "mlp.gate_proj.weight"].T) * (x @ w[p + "mlp.up_proj.weight"].T)) @ w[p + "mlp.down_proj.weight"].T
            h = h + rms(m, w[p + "post_feedforward_layernorm.weight"], c.rms_norm_eps)
            ls = w.get(p + "layer_scalar")
            if ls is not None:
                h = h * ls.reshape(())
        self.len += S
        h = rms(h, w["model.norm.weight"], c.rms_norm_eps)
        head = w["model.embed_tokens.weight"] if c.tie_word_embeddings else w["lm_head.weight"]
        logits = h @ head.T
        cap = np.float32(c.final_logit_softcapping)
        return (cap * np.tanh(logits / cap)).astype(np.float32)

    def generate(self, prompt, n):
        logits = self.forward(prompt)
        out, all_logits = [], [logits[-1]]
        tok = int(np.argmax(logits[-1]))
        out.append(tok)
        for _ in range(n - 1):
            logits = self.forward([tok])
            all_logits.append(logits[-1])
            tok = int(np.argmax(logits[-1]))
            out.append(tok)
        return out, np.stack(all_logits)
