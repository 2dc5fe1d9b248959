"""Pre-norm GQA + SwiGLU decoders of the Mistral / Qwen3 family over the flattened ragged batch and the paged KV cache.

The reference keeps this "Mistral shell" beside its Gemma code: presets for Ministral 3B / 8B / 14B and
DeepSeek-R1-0528-Qwen3-8B (src/models/gemma/config.rs:40-123), a decoder with one forward per cache kind
(src/models/gemma/decoder.rs:56-207), ``SwiGluFfn`` / ``GqaAttention`` / ``TransformerLayer`` blocks
(src/models/gemma/layers.rs) and YaRN frequency scaling (src/models/gemma/rope.rs:102-162).  Here there is one forward:
the cache kind is the paged cache every model of this package uses, and continuous batching comes from the shared engine.

Layer: ``h += o(attn(rope(q), rope(k), v))`` on ``rms(h)``; ``h += down(silu(gate(x)) * up(x))`` on ``rms(h)``; scores scaled
by ``head_dim ** -0.5``; optional learned per-head q/k RMSNorm (the Qwen3 variant).  Weights are torch ``[out, in]`` with q/k/v
and gate/up fused; tensor parallelism shards them by whole heads / FFN columns exactly as the Gemma decoder does."""
from __future__ import annotations

import math
from dataclasses import dataclass

import torch
from torch import nn

from ... import ops
from ...ops import reference as ref


@dataclass
class MistralConfig:
    num_hidden_layers: int = 26
    hidden_size: int = 3072
    intermediate_size: int = 9216
    num_attention_heads: int = 32
    num_key_value_heads: int = 8
    head_dim: int = 128
    vocab_size: int = 131072
    rope_theta: float = 1e6
    rms_norm_eps: float = 1e-5
    max_seq_len: int = 16384
    yarn_max_seq_len: int | None = None
    yarn_beta_fast: float = 32.0
    yarn_beta_slow: float = 1.0
    yarn_mscale: float = 1.0
    yarn_mscale_all_dim: float = 0.0
    tie_word_embeddings: bool = True
    qk_norm: bool = False
    name: str = "ministral-3b"

    @staticmethod
    def ministral_3b():
        return MistralConfig(yarn_max_seq_len=262144)

    @staticmethod
    def ministral_8b():
        return MistralConfig(34, 4096, 12288, 32, 8, 128, 131072, 1e9, 1e-5, 16384, 262144, name="ministral-8b")

    @staticmethod
    def ministral_14b():
        return MistralConfig(40, 5120, 16384, 32, 8, 128, 131072, 1e9, 1e-5, 16384, 262144, tie_word_embeddings=False,
                             name="ministral-14b")

    @staticmethod
    def deepseek_r1_qwen3_8b():
        return MistralConfig(36, 4096, 12288, 32, 8, 128, 151936, 1e6, 1e-6, 32768, 131072, tie_word_embeddings=False, qk_norm=True,
                             name="deepseek-r1-qwen3-8b")

    @staticmethod
    def from_hf(d: dict):
        rp = d.get("rope_scaling") or d.get("rope_parameters") or {}
        h, nh = d["hidden_size"], d["num_attention_heads"]
        c = MistralConfig(d["num_hidden_layers"], h, d["intermediate_size"], nh, d.get("num_key_value_heads", nh),
                          d.get("head_dim") or h // nh, d["vocab_size"], float(d.get("rope_theta", rp.get("rope_theta", 1e6))),
                          float(d.get("rms_norm_eps", 1e-5)), int(d.get("max_position_embeddings", 16384)),
                          tie_word_embeddings=bool(d.get("tie_word_embeddings", False)),
                          qk_norm=d.get("model_type", "") in ("qwen3",) or bool(d.get("qk_norm", False)),
                          name=d.get("_name_or_path", d.get("model_type", "mistral")))
        if rp.get("rope_type", rp.get("type")) == "yarn":
            c.yarn_max_seq_len = int(rp.get("original_max_position_embeddings", c.max_seq_len) * rp.get("factor", 1.0))
            c.max_seq_len = int(rp.get("original_max_position_embeddings", c.max_seq_len))
            c.yarn_beta_fast, c.yarn_beta_slow = float(rp.get("beta_fast", 32.0)), float(rp.get("beta_slow", 1.0))
            c.yarn_mscale, c.yarn_mscale_all_dim = float(rp.get("mscale", 1.0)), float(rp.get("mscale_all_dim", 0.0))
        return c


def yarn_inv_freq(head_dim: int, theta: float, original_max_pos: int, factor: float, beta_fast: float = 32.0, beta_slow: float = 1.0,
                  mscale: float = 1.0, mscale_all_dim: float = 0.0):
    """YaRN by wavelength bands (src/models/gemma/rope.rs:102-162): wavelengths below ``original/beta_fast`` keep their
    frequency, above ``original/beta_slow`` are divided by ``factor``, in between interpolate linearly in wavelength.
    Returns ``(inv_freq f32 [D/2], magnitude scale)``; the magnitude multiplies cos and sin, i.e. both q and k."""
    j = torch.arange(head_dim // 2, dtype=torch.float64)
    inv = theta ** (-2.0 * j / head_dim)
    wavelen = 2.0 * math.pi / inv
    low, high = original_max_pos / beta_slow, original_max_pos / beta_fast
    ramp = ((wavelen - high) / (low - high)).clamp(0.0, 1.0)             # 0 = keep, 1 = fully scaled
    out = inv * (1.0 - ramp) + (inv / factor) * ramp
    m = 1.0
    if mscale_all_dim > 0.0:
        m = max(1.0, mscale * (1.0 + math.log(factor) / (mscale_all_dim * 10.0)))
    return out.to(torch.float32), m


class _NoTP:
    rank, size = 0, 1

    def row_linear(self, x, w, lora=None):
        return ops.linear(x, w)

    def reduce(self, x, residual=None):
        return x


_LAYER_STEP = None
# The matrix-vector stages of the fused step beat a one-token tensor-core GEMM launch while the matrix is small (4.0 against 6.1 us
# at 4 MB) and lose to it on wide ones (38 against 25 us at 117 MB: 7168 rows over 2368 warps leave a quarter of the machine idle
# in the last pass), so layers whose gate / up matrix is larger than this stay on the GEMM path.
_STEP_MAX_BYTES = 24 << 20


def _layer_step_enabled() -> bool:
    global _LAYER_STEP
    if _LAYER_STEP is None:
        from ...utils import flags
        _LAYER_STEP = bool(flags.get("MARY_LAYER_STEP"))
    return _LAYER_STEP


def set_layer_step(on: bool) -> None:
    """Switch the fused one-token layer step on or off (tests compare the two paths)."""
    global _LAYER_STEP
    _LAYER_STEP = bool(on)


class MistralLayer(nn.Module):
    def __init__(self, cfg: MistralConfig, i: int, tp, inv_freq, q_scale: float, dtype, device):
        super().__init__()
        self.cfg, self.i, self.tp = cfg, i, tp
        H, D = cfg.hidden_size, cfg.head_dim
        self.n_q = cfg.num_attention_heads // tp.size
        self.n_kv = max(cfg.num_key_value_heads // tp.size, 1)
        self.F = cfg.intermediate_size // tp.size
        kw = dict(dtype=dtype, device=device)
        P = lambda *s: nn.Parameter(torch.empty(*s, **kw), requires_grad=False)  # noqa: E731
        self.w_qkv, self.w_o = P((self.n_q + 2 * self.n_kv) * D, H), P(H, self.n_q * D)
        self.w_gu, self.w_down = P(2 * self.F, H), P(H, self.F)
        self.ln_attn, self.ln_ffn = P(H), P(H)
        self.q_norm, self.k_norm = (P(D), P(D)) if cfg.qk_norm else (None, None)
        self.inv_freq, self.scale = inv_freq, q_scale

    def forward(self, x, h, meta, cache, next_norm):
        c = self.cfg
        qkv = ops.linear(x, self.w_qkv)
        q = ops.qk_norm_rope_append(qkv, self.n_q, self.n_kv, c.head_dim, self.q_norm, self.k_norm, False, self.inv_freq, meta,
                                    cache.k[self.i], cache.v[self.i], c.rms_norm_eps)
        o = ops.paged_attention(q, cache.k[self.i], cache.v[self.i], meta, self.scale)
        a = self.tp.reduce(self.tp.row_linear(o.reshape(o.shape[0], -1), self.w_o))
        x, h = ops.add_rmsnorm(a, h, self.ln_ffn, c.rms_norm_eps)
        d = self.tp.reduce(self.tp.row_linear(ops.linear_glu(x, self.w_gu, "swiglu"), self.w_down))
        if next_norm is None:
            return None, (h.float() + d.float()).to(h.dtype)
        return ops.add_rmsnorm(d, h, next_norm, c.rms_norm_eps)

    def step_supported(self, h, meta, cache) -> bool:
        """Whether the fused one-token step (``csrc/kernels/layer_step.cu``) applies: one new token of one sequence on the GPU,
        bf16 weights and cache, head dim 128, no tensor parallelism, widths the kernels hold in shared memory."""
        c = self.cfg
        k = cache.k[self.i]
        return (h.is_cuda and h.dtype == torch.bfloat16 and h.shape[0] == 1 and meta.num_seqs == 1 and c.head_dim == 128
                and self.tp.size == 1 and isinstance(k, torch.Tensor) and k.dtype == torch.bfloat16 and c.hidden_size <= 8192
                and self.F <= 8192 and self.n_q * c.head_dim <= 8192 and 2 * self.F * c.hidden_size * 2 <= _STEP_MAX_BYTES
                and _layer_step_enabled())

    def step(self, h, meta, cache):
        """One new token of one sequence in five launches: ``h [1, H]`` (residual stream) -> the residual stream after this layer."""
        from ...ops import cuda as K
        c = self.cfg
        qkv = K.step_matvec(h, self.w_qkv, self.ln_attn, c.rms_norm_eps)
        o = K.step_attention(qkv, self.q_norm, self.k_norm, self.inv_freq, meta, cache.k[self.i], cache.v[self.i], self.n_q, self.n_kv,
                             c.head_dim, c.rms_norm_eps, self.scale)
        h = K.step_matvec(o, self.w_o, res=h, mode="residual")
        m = K.step_matvec(h, self.w_gu, self.ln_ffn, c.rms_norm_eps, mode="swiglu")
        return K.step_matvec(m, self.w_down, res=h, mode="residual")


class MistralModel(nn.Module):
    def __init__(self, cfg: MistralConfig, tp=None, dtype=torch.float32, device="cpu", long_context: bool = False):
        super().__init__()
        self.cfg, self.tp, self.dtype = cfg, tp or _NoTP(), dtype
        kw = dict(dtype=dtype, device=device)
        D = cfg.head_dim
        mscale = 1.0
        if long_context and cfg.yarn_max_seq_len:
            inv, mscale = yarn_inv_freq(D, cfg.rope_theta, cfg.max_seq_len, cfg.yarn_max_seq_len / cfg.max_seq_len, cfg.yarn_beta_fast,
                                        cfg.yarn_beta_slow, cfg.yarn_mscale, cfg.yarn_mscale_all_dim)
            inv = inv.to(device)
        else:
            inv = ref.rope_inv_freq(D, cfg.rope_theta, 1.0, device)
        self.register_buffer("inv_freq", inv, persistent=False)
        scale = D ** -0.5 * mscale * mscale                      # the YaRN magnitude multiplies q and k alike
        self.embed = nn.Parameter(torch.empty(cfg.vocab_size, cfg.hidden_size, **kw), requires_grad=False)
        self.layers = nn.ModuleList([MistralLayer(cfg, i, self.tp, self.inv_freq, scale, dtype, device) for i in range(cfg.num_hidden_layers)])
        self.norm = nn.Parameter(torch.empty(cfg.hidden_size, **kw), requires_grad=False)
        self.lm_head = None if cfg.tie_word_embeddings else nn.Parameter(torch.empty(cfg.vocab_size, cfg.hidden_size, **kw), requires_grad=False)

    def kv_spec(self):
        c = self.cfg
        return dict(num_layers=c.num_hidden_layers, kv_heads=max(c.num_key_value_heads // self.tp.size, 1), head_dim=c.head_dim)

    def head_weight(self):
        return self.embed if self.lm_head is None else self.lm_head

    def hidden(self, ids, meta, cache):
        return self.hidden_from_embeds(ops.embed(ids, self.embed), meta, cache)

    def hidden_from_embeds(self, h, meta, cache):
        """The stack over given input embeddings ``[T, H]`` (speech models assemble them from several tables)."""
        c = self.cfg
        if self.layers[0].step_supported(h, meta, cache):
            for layer in self.layers:
                h = layer.step(h, meta, cache)
            return ops.rmsnorm(h, self.norm, c.rms_norm_eps)
        x = ops.rmsnorm(h, self.layers[0].ln_attn, c.rms_norm_eps)
        n = len(self.layers)
        for i, layer in enumerate(self.layers):
            x, h = layer(x, h, meta, cache, self.layers[i + 1].ln_attn if i + 1 < n else self.norm)
        return x

    def layer_states(self, ids, meta, cache, wanted):
        """Residual stream after the decoder layers in ``wanted`` (1-based: entry ``i`` is the state after ``i`` layers, 0 the input
        embeddings) — what image / speech models read when they use this decoder as a text encoder."""
        c = self.cfg
        h = ops.embed(ids, self.embed)
        out = {0: h.clone()} if 0 in wanted else {}
        x = ops.rmsnorm(h, self.layers[0].ln_attn, c.rms_norm_eps)
        n = len(self.layers)
        for i, layer in enumerate(self.layers):
            if i >= max(wanted):
                break
            x, h = layer(x, h, meta, cache, self.layers[i + 1].ln_attn if i + 1 < n else self.norm)
            if i + 1 in wanted:
                out[i + 1] = h.clone()
        return out

    def forward(self, ids, meta, cache, rows=None):
        x = self.hidden(ids, meta, cache)
        if rows is not None:
            x = x[rows]
        return ops.linear(x, self.head_weight()).float()

    def greedy(self, ids, meta, cache, rows):
        tok, _ = ops.lm_head_argmax(self.hidden(ids, meta, cache)[rows], self.head_weight())
        return tok


def init_random_(model: MistralModel, seed: int = 0, std: float = 0.02) -> None:
    g = torch.Generator(device=model.embed.device).manual_seed(seed)
    for _, p in model.named_parameters():
        if p.dim() == 1:
            p.data.fill_(1.0)
        else:
            p.data.normal_(0.0, std, generator=g)


PREFIXES = ("model.", "", "language_model.model.", "model.language_model.")


def load_into(model: MistralModel, loader) -> None:
    """Fill the model from a ``WeightLoader`` holding HF names (``model.layers.N.self_attn.q_proj.weight`` ...); tensor-parallel
    ranks take whole heads / FFN column blocks."""
    cfg, tp, dt = model.cfg, model.tp, model.dtype
    pre = next((p for p in PREFIXES if loader.has_weight(p + "embed_tokens.weight")), None)
    if pre is None:
        raise LookupError(f"no tensor named *embed_tokens.weight under any known prefix {PREFIXES}")

    def get(n):
        return loader.load_tensor(pre + n, dt)

    def put(p, t):
        p.data.copy_(t.to(p.device, dt))
    put(model.embed, get("embed_tokens.weight"))
    put(model.norm, get("norm.weight"))
    if model.lm_head is not None:
        name = "lm_head.weight" if loader.has_weight("lm_head.weight") else pre + "lm_head.weight"
        put(model.lm_head, loader.load_tensor(name, dt))
    D, r, n = cfg.head_dim, tp.rank, tp.size
    for i, L in enumerate(model.layers):
        p = f"layers.{i}."
        q = get(p + "self_attn.q_proj.weight").view(cfg.num_attention_heads, D, -1)
        k = get(p + "self_attn.k_proj.weight").view(cfg.num_key_value_heads, D, -1)
        v = get(p + "self_attn.v_proj.weight").view(cfg.num_key_value_heads, D, -1)
        kv0 = (r * cfg.num_key_value_heads) // n if cfg.num_key_value_heads >= n else 0
        put(L.w_qkv, torch.cat([q[r * L.n_q:(r + 1) * L.n_q].reshape(-1, q.shape[-1]), k[kv0:kv0 + L.n_kv].reshape(-1, k.shape[-1]),
                                v[kv0:kv0 + L.n_kv].reshape(-1, v.shape[-1])], 0))
        put(L.w_o, get(p + "self_attn.o_proj.weight")[:, r * L.n_q * D:(r + 1) * L.n_q * D])
        g, u = get(p + "mlp.gate_proj.weight"), get(p + "mlp.up_proj.weight")
        put(L.w_gu, torch.cat([g[r * L.F:(r + 1) * L.F], u[r * L.F:(r + 1) * L.F]], 0))
        put(L.w_down, get(p + "mlp.down_proj.weight")[:, r * L.F:(r + 1) * L.F])
        put(L.ln_attn, get(p + "input_layernorm.weight"))
        put(L.ln_ffn, get(p + "post_attention_layernorm.weight"))
        if cfg.qk_norm:
            put(L.q_norm, get(p + "self_attn.q_norm.weight"))
            put(L.k_norm, get(p + "self_attn.k_norm.weight"))
