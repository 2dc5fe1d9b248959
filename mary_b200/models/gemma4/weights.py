"""Weight naming, random initialisation into a pile, and loading a pile into a ``Gemma4Model``.

Name-prefix resolution (``""``, ``model.``, ``model.language_model.`` ...) follows
src/models/gemma/gemma4/weights.rs:100-145; ``layer_scalar`` is read per layer, 1.0 if absent (:653-656)."""
from __future__ import annotations

import numpy as np
import torch

from ...format import jsonfacts
from ...format.ingest import ingest_tensors
from ...format.model import build_model_root
from ...pile.trible import TribleBuilder
from .config import Gemma4TextConfig

PREFIXES = ("", "model.", "model.language_model.", "language_model.model.", "language_model.")


def tensor_names(cfg: Gemma4TextConfig) -> dict[str, tuple]:
    """Every tensor of the text decoder with its shape (torch ``[out, in]``)."""
    H, V = cfg.hidden_size, cfg.vocab_size
    P, n = cfg.hidden_size_per_layer_input, cfg.num_hidden_layers
    out = {"model.embed_tokens.weight": (V, H), "model.norm.weight": (H,)}
    if P:
        out.update({"model.embed_tokens_per_layer.weight": (cfg.ple_vocab, n * P),
                    "model.per_layer_model_projection.weight": (n * P, H), "model.per_layer_projection_norm.weight": (P,)})
    for i in range(cfg.num_hidden_layers):
        D, Hq, Hkv, F = cfg.layer_head_dim(i), cfg.num_attention_heads, cfg.layer_kv_heads(i), cfg.layer_intermediate(i)
        p = f"model.layers.{i}."
        if P:
            out.update({p + "per_layer_input_gate.weight": (P, H), p + "per_layer_projection.weight": (H, P),
                        p + "post_per_layer_input_norm.weight": (H,)})
        if cfg.enable_moe_block:
            E, Fm = cfg.num_experts, cfg.moe_intermediate_size
            out.update({p + "router.proj.weight": (E, H), p + "router.scale": (H,), p + "router.per_expert_scale": (E,),
                        p + "experts.gate_up_proj": (E, 2 * Fm, H), p + "experts.down_proj": (E, H, Fm),
                        p + "post_feedforward_layernorm_1.weight": (H,), p + "post_feedforward_layernorm_2.weight": (H,),
                        p + "pre_feedforward_layernorm_2.weight": (H,)})
        out.update({
            p + "input_layernorm.weight": (H,), p + "post_attention_layernorm.weight": (H,),
            p + "pre_feedforward_layernorm.weight": (H,), p + "post_feedforward_layernorm.weight": (H,),
            p + "self_attn.q_proj.weight": (Hq * D, H), p + "self_attn.o_proj.weight": (H, Hq * D),
            p + "self_attn.q_norm.weight": (D,),
            p + "mlp.gate_proj.weight": (F, H), p + "mlp.up_proj.weight": (F, H), p + "mlp.down_proj.weight": (H, F)})
        if cfg.kv_source(i) is None:                     # KV-shared layers carry no K/V tensors; K=V layers carry no v_proj
            out.update({p + "self_attn.k_proj.weight": (Hkv * D, H), p + "self_attn.k_norm.weight": (D,)})
            if not cfg.k_eq_v(i):
                out[p + "self_attn.v_proj.weight"] = (Hkv * D, H)
    if not cfg.tie_word_embeddings:
        out["lm_head.weight"] = (V, H)
    return out


def random_weights(cfg: Gemma4TextConfig, seed: int = 0, std: float = 0.02):
    """``normal(0, std)`` for matrices, ones for norm gains — generated tensor by tensor in name order."""
    rng = np.random.default_rng(seed)
    for name, shape in sorted(tensor_names(cfg).items()):
        if name.endswith("norm.weight") or "layernorm" in name or name.endswith(("router.scale", "per_expert_scale")):
            yield name, np.ones(shape, dtype=np.float32)
        else:
            yield name, (rng.standard_normal(shape, dtype=np.float32) * np.float32(std))


def write_random_pile(pile, key, cfg: Gemma4TextConfig, name: str = "gemma4-tiny", seed: int = 0, dtype: str = "f32") -> bytes:
    """Random-init model + its ``config.json`` as facts, published to the model-graph collection."""
    from ...format.persist import publish_fragment
    tb = TribleBuilder()
    members = ingest_tensors(pile, tb, random_weights(cfg, seed), dtype)
    root = build_model_root(pile, tb, members, name=name, source=f"random-init seed={seed}",
                            quantization=None if dtype == "f32" else dtype)
    jsonfacts.save_document(pile, tb, "config.json", cfg.to_json(), owner=root)
    publish_fragment(pile, key, tb.build(), f"random {name}"[:32])
    return root


def resolve_prefix(loader, probe: str = "embed_tokens.weight") -> str:
    for p in PREFIXES:
        if loader.has_weight(p + probe):
            return p
    raise LookupError(f"no tensor named *{probe} under any known prefix {PREFIXES}")


def load_into(model, loader, device=None) -> None:
    """Fill a ``Gemma4Model`` from a ``WeightLoader``; TP ranks take their shard of every projection."""
    cfg, tp = model.cfg, model.tp
    pre = resolve_prefix(loader)
    dt = model.dtype

    def get(n):
        return loader.load_tensor(pre + n, dt)

    def put(param, t):
        param.data.copy_(t.to(param.device, dt))

    put(model.embed, get("embed_tokens.weight"))
    put(model.norm, get("norm.weight"))
    if cfg.hidden_size_per_layer_input:
        put(model.ple_embed, get("embed_tokens_per_layer.weight"))
        put(model.ple_model_proj, get("per_layer_model_projection.weight"))
        put(model.ple_proj_norm, get("per_layer_projection_norm.weight"))
    for i, L in enumerate(model.layers):
        p = f"layers.{i}."
        D = cfg.layer_head_dim(i)
        r, n = tp.rank, tp.size
        q = get(p + "self_attn.q_proj.weight").view(cfg.num_attention_heads, D, -1)
        qs = q[r * L.n_q:(r + 1) * L.n_q]
        if L.kv_source is None:
            k = get(p + "self_attn.k_proj.weight").view(cfg.layer_kv_heads(i), D, -1)
            # K = V layers ship no v_proj: v is the same projection as k (before the norms)
            v = k if cfg.k_eq_v(i) and not loader.has_weight(pre + p + "self_attn.v_proj.weight") \
                else get(p + "self_attn.v_proj.weight").view(cfg.layer_kv_heads(i), D, -1)
            kv0 = (r * cfg.layer_kv_heads(i)) // n if cfg.layer_kv_heads(i) >= n else 0
            ks, vs = k[kv0:kv0 + L.n_kv], v[kv0:kv0 + L.n_kv]
            put(L.w_qkv, torch.cat([qs.reshape(-1, q.shape[-1]), ks.reshape(-1, k.shape[-1]), vs.reshape(-1, v.shape[-1])], 0))
        else:
            put(L.w_qkv, qs.reshape(-1, q.shape[-1]))
        o = get(p + "self_attn.o_proj.weight")
        put(L.w_o, o[:, r * L.n_q * D:(r + 1) * L.n_q * D])
        g, u = get(p + "mlp.gate_proj.weight"), get(p + "mlp.up_proj.weight")
        put(L.w_gu, torch.cat([g[r * L.F:(r + 1) * L.F], u[r * L.F:(r + 1) * L.F]], 0))
        put(L.w_down, get(p + "mlp.down_proj.weight")[:, r * L.F:(r + 1) * L.F])
        put(L.q_norm, get(p + "self_attn.q_norm.weight"))
        if L.kv_source is None:
            put(L.k_norm, get(p + "self_attn.k_norm.weight"))
        else:
            L.k_norm.data.fill_(1.0)
        put(L.ln_in, get(p + "input_layernorm.weight"))
        put(L.ln_post_attn, get(p + "post_attention_layernorm.weight"))
        put(L.ln_pre_ffn, get(p + "pre_feedforward_layernorm.weight"))
        put(L.ln_post_ffn, get(p + "post_feedforward_layernorm.weight"))
        if L.ple:
            put(L.ple_gate, get(p + "per_layer_input_gate.weight"))
            put(L.ple_proj, get(p + "per_layer_projection.weight"))
            put(L.ln_post_ple, get(p + "post_per_layer_input_norm.weight"))
        if L.moe:                                   # (weights.rs:807-883) experts of this rank: a contiguous index range
            e0 = r * L.e_local
            put(L.router_proj, get(p + "router.proj.weight"))
            put(L.router_scale, get(p + "router.scale"))
            put(L.per_expert_scale, get(p + "router.per_expert_scale"))
            put(L.ex_gate_up, get(p + "experts.gate_up_proj")[e0:e0 + L.e_local])
            put(L.ex_down, get(p + "experts.down_proj")[e0:e0 + L.e_local])
            put(L.ln_post_ffn_1, get(p + "post_feedforward_layernorm_1.weight"))
            put(L.ln_post_ffn_2, get(p + "post_feedforward_layernorm_2.weight"))
            put(L.ln_pre_ffn_2, get(p + "pre_feedforward_layernorm_2.weight"))
        if loader.has_weight(pre + p + "layer_scalar"):
            L.layer_scalar = float(loader.load_host_f32(pre + p + "layer_scalar").reshape(-1)[0])
    if not cfg.tie_word_embeddings and loader.has_weight("lm_head.weight"):
        model.lm_head = torch.nn.Parameter(loader.load_tensor("lm_head.weight", dt).to(model.embed.device), requires_grad=False)


def init_random_(model, seed: int = 0, std: float = 0.02) -> None:
    """Random-init directly on the model's device (benchmarks of the large configs: no host round trip)."""
    g = torch.Generator(device=model.embed.device).manual_seed(seed)
    for n, p in model.named_parameters():
        if p.dim() == 1:
            p.data.fill_(1.0)
        else:
            p.data.normal_(0.0, std, generator=g)


def shard_from_full(full, tp, device=None):
    """A tensor-parallel ``Gemma4Model`` (rank ``tp.rank`` of ``tp.size``) cut out of an unsharded one: q/k/v and gate/up by
    output rows (whole heads), o/down by input columns, everything else replicated."""
    from .model import Gemma4Model
    cfg = full.cfg
    dev = device or full.embed.device
    m = Gemma4Model(cfg, tp=tp, dtype=full.dtype, device=dev)
    r, n = tp.rank, tp.size
    with torch.no_grad():
        m.embed.copy_(full.embed)
        m.norm.copy_(full.norm)
        if cfg.hidden_size_per_layer_input:
            for nm in ("ple_embed", "ple_model_proj", "ple_proj_norm"):
                getattr(m, nm).copy_(getattr(full, nm))
        for L, Fl in zip(m.layers, full.layers):
            D, H = L.D, cfg.hidden_size
            q, k, v = Fl.w_qkv.split([Fl.n_q * D, Fl.n_kv * D, Fl.n_kv * D], 0)
            kv0 = (r * Fl.n_kv) // n if Fl.n_kv >= n else 0
            L.w_qkv.copy_(torch.cat([q.view(Fl.n_q, D, H)[r * L.n_q:(r + 1) * L.n_q].reshape(-1, H),
                                     k.view(Fl.n_kv, D, H)[kv0:kv0 + L.n_kv].reshape(-1, H),
                                     v.view(Fl.n_kv, D, H)[kv0:kv0 + L.n_kv].reshape(-1, H)], 0))
            L.w_o.copy_(Fl.w_o[:, r * L.n_q * D:(r + 1) * L.n_q * D])
            g, u = Fl.w_gu[:Fl.F], Fl.w_gu[Fl.F:]
            L.w_gu.copy_(torch.cat([g[r * L.F:(r + 1) * L.F], u[r * L.F:(r + 1) * L.F]], 0))
            L.w_down.copy_(Fl.w_down[:, r * L.F:(r + 1) * L.F])
            names = ["q_norm", "k_norm", "ln_in", "ln_post_attn", "ln_pre_ffn", "ln_post_ffn"]
            if L.ple:
                names += ["ple_gate", "ple_proj", "ln_post_ple"]
            if L.moe:
                names += ["router_proj", "router_scale", "per_expert_scale", "ln_post_ffn_1", "ln_post_ffn_2", "ln_pre_ffn_2"]
                L.ex_gate_up.copy_(Fl.ex_gate_up[r * L.e_local:(r + 1) * L.e_local])
                L.ex_down.copy_(Fl.ex_down[r * L.e_local:(r + 1) * L.e_local])
            for nm in names:
                getattr(L, nm).copy_(getattr(Fl, nm))
            L.layer_scalar = Fl.layer_scalar
    return m
