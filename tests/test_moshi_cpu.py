"""Moshi-style speech LM: the stream delay machine, the per-step depformer, and the frame loop."""
import torch

from mary_b200.models.moshi import LmGen, MoshiConfig, StreamCache, init_random_


def test_stream_cache_delays_forcing_and_undelayed_output():
    c = MoshiConfig.tiny()                       # streams: text, agent (semantic, acoustic), user (semantic, acoustic)
    assert c.delays == [0, 0, 1, 0, 1] and c.max_delay == 1 and c.num_streams == 5
    sc = StreamCache(c)
    assert sc.prepare(user_audio=[7, 8]) is None and sc.offset == 1             # offset 0 only seeds
    assert [row[0] for row in sc.cache] == [c.text_card, c.card, c.card, c.card, c.card]
    outs = []
    for f in range(1, 6):
        p = sc.prepare(user_audio=[10 + f, 20 + f])
        # user semantic (stream 3, delay 0) is provided at the target position now; user acoustic (stream 4, delay 1) lands one ahead
        assert p["provided"][3] and p["target"][3] == 10 + f
        if f == 1:
            assert p["input"] == [c.text_card] + [c.card] * 4                   # the seeded initial tokens are fed first
            assert p["provided"][2] and p["target"][2] == c.card                # delayed streams get their initial token at offset <= delay
        if f >= 2:
            assert p["provided"][4] and p["target"][4] == 20 + f - 1            # what the caller gave one frame earlier
        out = sc.commit(p, sampled_text=100 + f, sampled_audio=[200 + f, 300 + f, 400 + f, 500 + f])
        outs.append(out)
    assert outs[0] is None and outs[1] is not None                              # emission starts once offset > max_delay
    # undelayed frame at offset o: stream k shows what sits at (o - max_delay + delay_k); provided tokens win over sampled ones
    o = outs[3]                                                                 # produced at offset 4: base position 3
    assert o[0] == 103 and o[1] == 203 and o[2] == 304                          # acoustic agent codebook taken one position later
    assert o[3] == 13 and o[4] == 23                                            # user tokens: provided values, re-aligned
    sc.reset()
    assert sc.offset == 0 and all(v == -2 for row in sc.cache for v in row)


def test_depformer_forcing_changes_only_later_steps_and_cache_matches_recompute():
    c = MoshiConfig.tiny()
    m = LmGen(c)
    init_random_(m, 0)
    torch.manual_seed(1)
    h = torch.randn(2, c.dim)
    text = torch.tensor([3, 9])
    with torch.no_grad():
        free = m.depformer.generate(h, text)
        forced = m.depformer.generate(h, text, forced=[None, 5, None, None])
        assert torch.equal(free[:, :2], forced[:, :2])                          # step 1's own OUTPUT is not changed by forcing its token
        # cached steps equal recomputing the prefix from scratch
        prev, cache, toks = text, None, []
        for t in range(c.dep_q):
            lg, cache = m.depformer.step(t, h, prev, cache)
            prev2, cache2 = text, None
            for u in range(t + 1):
                lg2, cache2 = m.depformer.step(u, h, prev2, cache2)
                prev2 = lg2.argmax(-1)
            assert torch.allclose(lg, lg2, atol=1e-5)
            prev = lg.argmax(-1)
            toks.append(prev)
        assert torch.equal(torch.stack(toks, 1), free)


def test_frame_loop_is_deterministic_and_respects_provided_tokens():
    c = MoshiConfig.tiny()
    runs = []
    for _ in range(2):
        m = LmGen(c)
        init_random_(m, 0)
        outs = []
        for f in range(8):
            outs.append(m.step(user_audio=[(3 * f) % c.card, (5 * f + 1) % c.card], text=7 if f == 4 else None))
        runs.append(outs)
    assert runs[0] == runs[1]
    frames = [o for o in runs[0] if o is not None]
    assert len(frames) == 8 - 1 - c.max_delay
    for i, o in enumerate(frames):
        f = i + 1                                                               # frame whose tokens are emitted
        assert o[3] == (3 * f) % c.card and o[4] == (5 * f + 1) % c.card       # user streams come back exactly as provided
        assert 0 <= o[1] < c.card and 0 <= o[2] < c.card
    assert frames[3][0] == 7                                                    # the forced text token of frame 4
    m.reset_session()
    assert m.step(user_audio=[0, 1]) is None


def test_depformer_matches_the_huggingface_depth_decoder():
    """Same weights: per-codebook (flexible) linears for the input projection, q / k / v / o, the gated MLP and the heads; no rotary;
    step t is conditioned on the token of step t - 1 (the text token at t = 0)."""
    import pytest
    pytest.importorskip("transformers")
    from transformers.models.moshi.configuration_moshi import MoshiDepthConfig
    from transformers.models.moshi.modeling_moshi import MoshiDepthDecoder
    c = MoshiConfig.tiny()
    torch.manual_seed(0)
    hc = MoshiDepthConfig(vocab_size=c.text_card, hidden_size=c.dep_dim, input_size=c.dim, num_hidden_layers=c.dep_layers,
                          num_attention_heads=c.dep_heads, audio_vocab_size=c.card, ffn_dim=2 * c.dep_ffn, rms_norm_eps=c.eps,
                          num_codebooks=c.dep_q, max_position_embeddings=c.dep_q + 1, sliding_window=c.dep_q)
    hc._attn_implementation = "eager"
    hf = MoshiDepthDecoder(hc).eval()
    with torch.no_grad():
        for n, p in hf.named_parameters():
            p.copy_(1.0 + 0.1 * torch.randn_like(p) if "layernorm" in n else 0.15 * torch.randn_like(p))
    sd = {k: v.detach() for k, v in hf.state_dict().items()}
    m = LmGen(c)
    init_random_(m, 0)
    d = m.depformer
    with torch.no_grad():
        d.w_in.copy_(sd["input_projections.weight"]), d.text_emb.copy_(sd["text_embed_tokens.weight"]), d.heads.copy_(sd["lm_heads.weight"])
        for t in range(c.dep_q - 1):
            d.audio_emb[t].copy_(sd[f"embed_tokens.{t}.weight"])
        for li in range(c.dep_layers):
            p = f"layers.{li}."
            d.w_qkv[li].copy_(torch.cat([sd[p + f"self_attn.{x}_proj.linear.weight"] for x in "qkv"], 1))
            d.w_o[li].copy_(sd[p + "self_attn.o_proj.linear.weight"])
            d.w_gu[li].copy_(sd[p + "mlp.fc1.weight"]), d.w_down[li].copy_(sd[p + "mlp.fc2.weight"])
            d.norm1[li].copy_(sd[p + "input_layernorm.weight"]), d.norm2[li].copy_(sd[p + "post_attention_layernorm.weight"])
    B = 3
    h = torch.randn(B, c.dim)
    ids = torch.cat([torch.randint(0, c.text_card, (B, 1)), torch.randint(0, c.card, (B, c.dep_q - 1))], 1)
    with torch.no_grad():
        # the library builds its causal mask only when an attention mask is passed
        want = hf(input_ids=ids, last_hidden_state=h[:, None, :], attention_mask=torch.ones(B, c.dep_q, dtype=torch.long)).logits
        cache, got = None, []
        for t in range(c.dep_q):
            lg, cache = d.step(t, h, ids[:, t], cache)
            got.append(lg)
    got = torch.stack(got, 1)
    assert torch.allclose(got, want, atol=2e-4), float((got - want).abs().max())


def test_whole_speech_lm_loaded_by_name_matches_huggingface_moshi():
    """Temporal transformer + text head + depth decoder filled by ``load_into`` from the library's state-dict names; the frame
    embedding is the sum of the text and the sixteen audio stream embeddings, as the library's conditional-generation model forms it."""
    import pytest
    pytest.importorskip("transformers")
    from transformers.models.moshi.configuration_moshi import MoshiConfig as HFConfig, MoshiDepthConfig
    from transformers.models.moshi.modeling_moshi import MoshiDepthDecoder, MoshiForCausalLM
    from mary_b200.models.moshi import load_into
    from mary_b200.runtime.batch import BatchMeta
    from mary_b200 import ops
    c = MoshiConfig.tiny()
    torch.manual_seed(1)
    depth = dict(vocab_size=c.text_card, hidden_size=c.dep_dim, input_size=c.dim, num_hidden_layers=c.dep_layers,
                 num_attention_heads=c.dep_heads, audio_vocab_size=c.card, ffn_dim=2 * c.dep_ffn, rms_norm_eps=c.eps,
                 num_codebooks=c.dep_q, max_position_embeddings=c.dep_q + 1, sliding_window=c.dep_q)
    hc = HFConfig(vocab_size=c.text_card, hidden_size=c.dim, num_hidden_layers=c.layers, num_attention_heads=c.heads,
                  num_key_value_heads=c.heads, audio_vocab_size=c.card, max_position_embeddings=c.context, rope_theta=c.rope_theta,
                  head_dim=c.dim // c.heads, ffn_dim=2 * c.ffn, rms_norm_eps=c.eps, num_codebooks=c.dep_q // 2, sliding_window=c.context,
                  depth_decoder_config=dict(depth))
    hc._attn_implementation = "eager"
    lm = MoshiForCausalLM(hc).eval()
    dc = MoshiDepthConfig(**depth)
    dc._attn_implementation = "eager"
    dd = MoshiDepthDecoder(dc).eval()
    with torch.no_grad():
        for mod in (lm, dd):
            for n, p in mod.named_parameters():
                p.copy_(1.0 + 0.1 * torch.randn_like(p) if "norm" in n else 0.15 * torch.randn_like(p))
    audio_tables = [0.15 * torch.randn(c.card + 1, c.dim) for _ in range(c.dep_q)]
    sd = {"decoder." + k: v.detach() for k, v in lm.state_dict().items()}
    sd.update({"depth_decoder." + k: v.detach() for k, v in dd.state_dict().items()})
    sd.update({f"embed_tokens.{s}.weight": t for s, t in enumerate(audio_tables)})

    class L:
        def load_tensor(self, n, dtype):
            return sd[n].to(dtype)
    m = LmGen(c)
    init_random_(m, 5)
    load_into(m, L())
    T = 7
    text = torch.randint(0, c.text_card, (T,))
    audio = torch.randint(0, c.card, (T, c.dep_q))
    with torch.no_grad():
        emb = lm.model.embed_tokens(text) + sum(audio_tables[s][audio[:, s]] for s in range(c.dep_q))
        out = lm(inputs_embeds=emb[None], attention_mask=torch.ones(1, T, dtype=torch.long))
        want_logits, want_h = out.logits[0], out.last_hidden_state[0]
        x = torch.cat([m.embed_frame([int(text[t])] + [int(a) for a in audio[t]]) for t in range(T)])
        assert torch.allclose(x, emb, atol=1e-6)
        meta = BatchMeta.build([T], [T], m.table, 16, m.dev)
        h = m.temporal.hidden_from_embeds(x, meta, m.cache)
        got_logits = ops.linear(h, m.text_head).float()
    assert torch.allclose(h, want_h, atol=3e-4, rtol=1e-3), float((h - want_h).abs().max())
    assert torch.allclose(got_logits, want_logits, atol=3e-4, rtol=1e-3), float((got_logits - want_logits).abs().max())
    # the depth decoder, conditioned on the temporal state the two models agree on
    ids = torch.cat([torch.randint(0, c.text_card, (T, 1)), torch.randint(0, c.card, (T, c.dep_q - 1))], 1)
    with torch.no_grad():
        want = dd(input_ids=ids, last_hidden_state=want_h[:, None, :], attention_mask=torch.ones(T, c.dep_q, dtype=torch.long)).logits
        cache, got = None, []
        for t in range(c.dep_q):
            lg, cache = m.depformer.step(t, h, ids[:, t], cache)
            got.append(lg)
    got = torch.stack(got, 1)
    assert torch.allclose(got, want, atol=5e-4, rtol=1e-3), float((got - want).abs().max())
