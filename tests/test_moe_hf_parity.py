"""The K3-class decoder (latent attention with absorbed projections and a latent cache, sigmoid router with a selection-only bias and
group-limited top-k, shared expert, leading dense layer) against the Hugging Face DeepSeek-V3 implementation of the same
architecture: an independent oracle with an EXPANDED key / value cache and a different formulation of every block.  The experts'
weights are the de-quantised NVFP4 values on both sides; activation quantisation is switched off here so that the comparison is about
the architecture (the quantised pipeline has its own bit-exact tests)."""
import pytest
import torch

from mary_b200.models.moe import MoEDecoder, init_random_, tiny_moe_config
from mary_b200.models.moe import model as moe_model
from mary_b200.runtime.batch import BatchMeta
from mary_b200.runtime.kv_cache import PagedKVCache


def _dense_experts(x, idx, w, ex, shared=None, nt=None):
    out = torch.zeros(x.shape[0], ex.H, dtype=torch.float32)
    for e in idx.unique().tolist():
        if e < 0:
            continue
        t, j = (idx == e).nonzero(as_tuple=True)
        w13, w2 = ex.dense("w13", e), ex.dense("w2", e)
        g, u = (x[t].float() @ w13.T).chunk(2, -1)
        out.index_add_(0, t, ((torch.nn.functional.silu(g) * u) @ w2.T) * w[t, j].float()[:, None])
    if shared is not None:
        out = out + shared.float()
    return out.to(x.dtype)


@pytest.mark.parametrize("n_tokens", [21, 70])          # below / above the length from which prefill expands K and V from the latent rows
def test_logits_match_huggingface_deepseek_v3(monkeypatch, n_tokens):
    transformers = pytest.importorskip("transformers")
    from transformers.models.deepseek_v3 import DeepseekV3Config, DeepseekV3ForCausalLM
    monkeypatch.setattr(moe_model, "experts_forward", _dense_experts)
    cfg = tiny_moe_config("mla", num_mtp_layers=0, hidden_size=256, q_lora_rank=128, dense_intermediate_size=384, moe_intermediate_size=128,
                          vocab_size=300, num_attention_heads=4)
    m = MoEDecoder(cfg, dtype=torch.float32)
    init_random_(m, 0, std=0.05)
    g = torch.Generator().manual_seed(5)
    with torch.no_grad():
        for L in m.layers:
            if not L.dense:
                L.ffn.router_bias.copy_(0.3 * torch.randn(cfg.n_routed_experts, generator=g))       # moves the selection, not the weights
                L.ffn.w_router.mul_(20.0)                                                           # decisive routing
            for p in (L.ln_attn, L.ln_ffn, L.attn.qa_norm, L.attn.kv_norm):
                p.copy_(1.0 + 0.1 * torch.randn(p.shape, generator=g))
    hc = DeepseekV3Config(vocab_size=cfg.vocab_size, hidden_size=cfg.hidden_size, intermediate_size=cfg.dense_intermediate_size,
                          moe_intermediate_size=cfg.moe_intermediate_size, num_hidden_layers=cfg.num_hidden_layers,
                          num_attention_heads=cfg.num_attention_heads, num_key_value_heads=cfg.num_attention_heads, n_shared_experts=1,
                          n_routed_experts=cfg.n_routed_experts, routed_scaling_factor=cfg.routed_scaling_factor, kv_lora_rank=512,
                          q_lora_rank=cfg.q_lora_rank, qk_rope_head_dim=64, v_head_dim=128, qk_nope_head_dim=128, n_group=cfg.n_group,
                          topk_group=cfg.topk_group, num_experts_per_tok=cfg.num_experts_per_tok, first_k_dense_replace=cfg.first_k_dense,
                          norm_topk_prob=True, hidden_act="silu", rms_norm_eps=cfg.rms_norm_eps, rope_interleave=False,
                          rope_parameters={"rope_type": "default", "rope_theta": cfg.rope_theta}, max_position_embeddings=512,
                          tie_word_embeddings=False, attention_bias=False)
    hc._attn_implementation = "eager"
    hf = DeepseekV3ForCausalLM(hc).eval().float()
    sd = {"model.embed_tokens.weight": m.embed, "model.norm.weight": m.norm, "lm_head.weight": m.lm_head}
    ql = cfg.q_lora_rank
    for i, L in enumerate(m.layers):
        p, a = f"model.layers.{i}.", L.attn
        kvb = torch.cat([torch.cat([a.w_uk[h].T, a.w_uv[h]], 0) for h in range(cfg.num_attention_heads)], 0)      # per head [k_nope ; v] rows
        sd.update({p + "input_layernorm.weight": L.ln_attn, p + "post_attention_layernorm.weight": L.ln_ffn,
                   p + "self_attn.q_a_proj.weight": a.w_qa_kva[:ql], p + "self_attn.q_a_layernorm.weight": a.qa_norm,
                   p + "self_attn.q_b_proj.weight": a.w_qb, p + "self_attn.kv_a_proj_with_mqa.weight": a.w_qa_kva[ql:],
                   p + "self_attn.kv_a_layernorm.weight": a.kv_norm, p + "self_attn.kv_b_proj.weight": kvb, p + "self_attn.o_proj.weight": a.w_o})
        if L.dense:
            F = L.ffn.w_gu.shape[0] // 2
            sd.update({p + "mlp.gate_proj.weight": L.ffn.w_gu[:F], p + "mlp.up_proj.weight": L.ffn.w_gu[F:], p + "mlp.down_proj.weight": L.ffn.w_down})
        else:
            f, ex = L.ffn, L.ffn.experts
            Fs = f.shared.w_gu.shape[0] // 2
            sd.update({p + "mlp.gate.weight": f.w_router, p + "mlp.gate.e_score_correction_bias": f.router_bias,
                       p + "mlp.experts.gate_up_proj": torch.stack([ex.dense("w13", e) for e in range(ex.E)]),
                       p + "mlp.experts.down_proj": torch.stack([ex.dense("w2", e) for e in range(ex.E)]),
                       p + "mlp.shared_experts.gate_proj.weight": f.shared.w_gu[:Fs], p + "mlp.shared_experts.up_proj.weight": f.shared.w_gu[Fs:],
                       p + "mlp.shared_experts.down_proj.weight": f.shared.w_down})
    missing, unexpected = hf.load_state_dict({k: v.detach().float() for k, v in sd.items()}, strict=False)
    assert not unexpected and all("rotary" in k or "inv_freq" in k for k in missing), (missing, unexpected)
    ids = torch.randint(0, cfg.vocab_size, (n_tokens,), generator=g)
    with torch.no_grad():
        want = hf(ids[None]).logits[0]
    spec = m.kv_spec()
    cache = PagedKVCache(spec["num_layers"], n_tokens // 16 + 2, 16, spec["kv_heads"], spec["head_dim"], dtype=torch.float32, latent_dim=576)
    cache.alloc.extend(0, n_tokens)
    table, lens = cache.alloc.page_table([0])
    with torch.no_grad():
        got = m(ids.int(), BatchMeta.build([n_tokens], lens, table, 16), cache)
    row_err = (got - want).abs().amax(-1) / want.abs().max()
    assert (row_err < 2e-4).float().mean() >= 0.95, row_err                      # a router near-tie may move a row; the rest must be exact
    # decode over the latent cache continues the same sequence: one more token equals the library's full forward of n + 1 tokens
    nxt = torch.randint(0, cfg.vocab_size, (1,), generator=g)
    cache.alloc.extend(0, 1)
    table, lens = cache.alloc.page_table([0])
    with torch.no_grad():
        step = m(nxt.int(), BatchMeta.build([1], lens, table, 16), cache)[0]
        want1 = hf(torch.cat([ids, nxt])[None]).logits[0, -1]
    assert float((step - want1).abs().max() / want1.abs().max()) < 2e-4


def test_gqa_softmax_moe_decoder_matches_huggingface_mixtral(monkeypatch):
    """The Inkling-style workload's decoder shape (GQA attention, softmax router over all experts with renormalised top-k, SwiGLU
    experts, no shared expert here) against the Hugging Face Mixtral implementation."""
    pytest.importorskip("transformers")
    from transformers import MixtralConfig, MixtralForCausalLM
    monkeypatch.setattr(moe_model, "experts_forward", _dense_experts)
    cfg = tiny_moe_config("gqa", hidden_size=256, num_attention_heads=4, num_key_value_heads=2, head_dim=64, n_shared_experts=0,
                          first_k_dense=0, moe_intermediate_size=128, vocab_size=300, rope_theta=1e4)
    m = MoEDecoder(cfg, dtype=torch.float32)
    init_random_(m, 0, std=0.05)
    g = torch.Generator().manual_seed(7)
    with torch.no_grad():
        for L in m.layers:
            L.ffn.w_router.mul_(20.0)
            for p in (L.ln_attn, L.ln_ffn):
                p.copy_(1.0 + 0.1 * torch.randn(p.shape, generator=g))
    hc = MixtralConfig(vocab_size=cfg.vocab_size, hidden_size=cfg.hidden_size, intermediate_size=cfg.moe_intermediate_size,
                       num_hidden_layers=cfg.num_hidden_layers, num_attention_heads=cfg.num_attention_heads,
                       num_key_value_heads=cfg.num_key_value_heads, head_dim=cfg.head_dim, num_local_experts=cfg.n_routed_experts,
                       num_experts_per_tok=cfg.num_experts_per_tok, rms_norm_eps=cfg.rms_norm_eps, sliding_window=None,
                       rope_parameters={"rope_type": "default", "rope_theta": cfg.rope_theta}, max_position_embeddings=512,
                       tie_word_embeddings=False)
    hc._attn_implementation = "eager"
    hf = MixtralForCausalLM(hc).eval().float()
    D, nq, nkv = cfg.head_dim, cfg.num_attention_heads, cfg.num_key_value_heads
    sd = {"model.embed_tokens.weight": m.embed, "model.norm.weight": m.norm, "lm_head.weight": m.lm_head}
    for i, L in enumerate(m.layers):
        p, ex = f"model.layers.{i}.", L.ffn.experts
        q, k, v = L.attn.w_qkv.split([nq * D, nkv * D, nkv * D], 0)
        sd.update({p + "input_layernorm.weight": L.ln_attn, p + "post_attention_layernorm.weight": L.ln_ffn,
                   p + "self_attn.q_proj.weight": q, p + "self_attn.k_proj.weight": k, p + "self_attn.v_proj.weight": v,
                   p + "self_attn.o_proj.weight": L.attn.w_o, p + "mlp.gate.weight": L.ffn.w_router,
                   p + "mlp.experts.gate_up_proj": torch.stack([ex.dense("w13", e) for e in range(ex.E)]),
                   p + "mlp.experts.down_proj": torch.stack([ex.dense("w2", e) for e in range(ex.E)])})
    missing, unexpected = hf.load_state_dict({k: v.detach().float() for k, v in sd.items()}, strict=False)
    assert not unexpected and not [k for k in missing if "inv_freq" not in k], (missing, unexpected)
    n = 33
    ids = torch.randint(0, cfg.vocab_size, (n,), generator=g)
    with torch.no_grad():
        want = hf(ids[None]).logits[0]
    spec = m.kv_spec()
    cache = PagedKVCache(spec["num_layers"], 4, 16, spec["kv_heads"], spec["head_dim"], dtype=torch.float32)
    cache.alloc.extend(0, n)
    table, lens = cache.alloc.page_table([0])
    with torch.no_grad():
        got = m(ids.int(), BatchMeta.build([n], lens, table, 16), cache)
    row_err = (got - want).abs().amax(-1) / want.abs().max()
    assert (row_err < 2e-4).float().mean() >= 0.95, row_err
