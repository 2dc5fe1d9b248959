"""Qwen3-TTS frame generator on a tiny configuration: the predictor's cached steps equal one uncached pass, the logits
processor follows the reference rules, and the frame loop is deterministic, streams and stops."""
import numpy as np
import pytest
import torch

from mary_b200 import ops
from mary_b200.models.qwen3tts import (CodePredictor, Qwen3TTSConfig, SamplingParams, Talker, generate_frames, init_random_,
                                       process_talker_logits)
from mary_b200.runtime.batch import BatchMeta
from mary_b200.runtime.kv_cache import PagedKVCache


def _models(seed=0):
    cfg = Qwen3TTSConfig.tiny()
    t, p = Talker(cfg), CodePredictor(cfg)
    init_random_(t, p, seed, std=0.2)
    return cfg, t, p


def test_predictor_cached_steps_equal_full_recompute():
    cfg, t, p = _models()
    torch.manual_seed(1)
    h, e0 = torch.randn(cfg.talker_hidden), torch.randn(cfg.talker_hidden)
    with torch.no_grad():
        codes, esum = p.predict_frame(h, e0, temperature=0.0)
        # uncached: feed the whole prefix again for every codebook
        xs = [p.project(torch.stack([h, e0]))]
        want = []
        for i in range(cfg.num_code_groups - 1):
            x = torch.cat(xs)
            spec = p.stack.kv_spec()
            cache = PagedKVCache(spec["num_layers"], 3, 16, spec["kv_heads"], spec["head_dim"], dtype=torch.float32)
            cache.alloc.extend(0, x.shape[0])
            table, lens = cache.alloc.page_table([0])
            hid = p.stack.hidden_from_embeds(x, BatchMeta.build([x.shape[0]], lens, table, 16), cache)[-1:]
            tok = int(ops.linear(hid, p.heads[i]).argmax())
            want.append(tok)
            xs.append(p.project(ops.embed(torch.tensor([tok], dtype=torch.int32), p.embeddings[i])))
    assert codes.tolist() == want
    assert torch.allclose(esum, p.accumulate_frame(want), atol=1e-5)


def test_logits_processing_rules():
    cfg = Qwen3TTSConfig.tiny()
    lg = torch.linspace(-1, 1, cfg.codec_vocab)
    out = process_talker_logits(lg, [3, 60, 3], 0, 2.0, cfg)
    assert out[3] == lg[3] * 2.0 and out[60] == lg[60] / 2.0          # negative logits are multiplied, positive divided
    assert out[cfg.codec_eos] == float("-inf")                          # no end of speech in the first two frames
    assert torch.isinf(out[cfg.pred_vocab:]).all()
    out2 = process_talker_logits(lg, [], 2, 2.0, cfg)
    assert out2[cfg.codec_eos] == lg[cfg.codec_eos]
    assert torch.isinf(out2[cfg.pred_vocab:cfg.codec_eos]).all() and torch.isinf(out2[cfg.codec_eos + 1:]).all()
    assert torch.equal(out2[:cfg.pred_vocab], lg[:cfg.pred_vocab])


def test_frame_loop_is_deterministic_streams_and_stops():
    cfg, t, p = _models(3)
    text = torch.randint(0, cfg.text_vocab, (9,), dtype=torch.int32)
    with torch.no_grad():
        prefill = t.embed_text(text[:6]) + t.embed_codec(torch.full((6,), cfg.codec_pad, dtype=torch.int32))
        trailing = t.embed_text(text[6:])
        pad = t.embed_text(torch.tensor([0], dtype=torch.int32))[0]
    params = SamplingParams(max_frames=7, seed=5)
    a = generate_frames(t, p, prefill, trailing, pad, params)
    b = generate_frames(t, p, prefill, trailing, pad, params)
    assert a.shape[1] == cfg.num_code_groups and 1 <= a.shape[0] <= 7 and np.array_equal(a, b)
    assert (a[:, 0] < cfg.codec_vocab).all() and (a[:, 1:] < cfg.pred_vocab).all() and (a >= 0).all()
    c = generate_frames(t, p, prefill, trailing, pad, SamplingParams(max_frames=7, seed=6))
    assert a.shape != c.shape or not np.array_equal(a, c)                # another seed, another utterance
    seen = []
    d = generate_frames(t, p, prefill, trailing, pad, params, on_frame=lambda f: (seen.append(f), len(seen) < 3)[1])
    assert len(seen) == min(3, a.shape[0]) and d.shape[0] == min(2, a.shape[0])
    assert np.array_equal(d, a[:d.shape[0]])


def test_speaker_mel_matches_the_library_filterbank_and_ecapa_pooling_rules():
    import math

    import numpy as np
    from mary_b200.models.qwen3tts.speaker import Ecapa, EcapaConfig, slaney_mel_filters, speaker_mel
    audio_utils = pytest.importorskip("transformers.audio_utils")
    want = audio_utils.mel_filter_bank(num_frequency_bins=513, num_mel_filters=128, min_frequency=0.0, max_frequency=12000.0, sampling_rate=24000,
                                       norm="slaney", mel_scale="slaney")
    got = slaney_mel_filters(128, 1024, 24000, 0.0, 12000.0)
    assert np.allclose(got.numpy().T, want, atol=1e-6)
    wave = torch.randn(256 * 20)
    mel = speaker_mel(wave)
    assert mel.shape == (128, 20) and mel.min() >= math.log(1e-5) - 1e-6
    # against torch.stft with the same padding convention
    x = torch.nn.functional.pad(wave[None, None], (384, 384), mode="reflect")[0, 0]
    spec = torch.stft(x, 1024, 256, window=torch.hann_window(1024), center=False, return_complex=True)
    ref = (got @ torch.sqrt(spec.real ** 2 + spec.imag ** 2 + 1e-9)).clamp_min(1e-5).log()
    assert torch.allclose(mel, ref, atol=2e-3)

    c = EcapaConfig.tiny()
    m = Ecapa(c)
    g = torch.Generator().manual_seed(0)
    for n, p in m.named_parameters():
        p.data.normal_(0.0, 0.2, generator=g)
    feats = torch.randn(c.n_mels, 37)
    v = m(feats)
    assert v.shape == (c.out_dim,) and torch.isfinite(v).all()
    assert m.tdnn0(feats).shape[1] == 37 and m.blocks[2](torch.randn(c.channels, 37)).shape == (c.channels, 37)     # "same" by reflection
    # zero attention weights: uniform attention, so the pooled statistics are the plain mean and standard deviation
    x = torch.randn(c.channels * 3, 11)
    m.att2.w.data.zero_(), m.att2.b.data.zero_()
    p = m.pool(x)
    assert torch.allclose(p[:x.shape[0], 0], x.mean(1), atol=1e-5) and torch.allclose(p[x.shape[0]:, 0], x.std(1, unbiased=False), atol=1e-5)
    # Res2Net: the first channel group passes through the middle stage untouched
    b = m.blocks[0]
    h = torch.randn(c.channels, 9)
    grp = c.channels // c.res2net_scale
    saved = b.tdnn2.w.data.clone()
    b.tdnn2.w.data.zero_()
    b.tdnn2.w.data[:grp, :grp, 0] = torch.eye(grp)
    b.tdnn2.b.data.zero_()
    b.se2.w.data.zero_(), b.se2.b.data.fill_(20.0)                      # gate = 1
    assert torch.allclose((b(h) - h)[:grp], torch.relu(b.tdnn1(h)[:grp]), atol=1e-5)
    b.tdnn2.w.data.copy_(saved)


def test_ecapa_loads_by_released_names_and_gates_attention_through_relu_then_tanh():
    from mary_b200.models.qwen3tts import speaker
    from mary_b200.models.qwen3tts.speaker import Ecapa, EcapaConfig
    c = EcapaConfig.tiny()
    g = torch.Generator().manual_seed(4)
    names = {"blocks.0.conv": (c.channels, c.n_mels, c.kernel0)}
    grp, n = c.channels // c.res2net_scale, c.channels * len(c.dilations)
    for i in range(1, len(c.dilations) + 1):
        names[f"blocks.{i}.tdnn1.conv"] = names[f"blocks.{i}.tdnn2.conv"] = (c.channels, c.channels, 1)
        for j in range(c.res2net_scale - 1):
            names[f"blocks.{i}.res2net_block.blocks.{j}.conv"] = (grp, grp, 3)
        names[f"blocks.{i}.se_block.conv1"], names[f"blocks.{i}.se_block.conv2"] = (c.se_channels, c.channels, 1), (c.channels, c.se_channels, 1)
    names.update({"mfa.conv": (n, n, 1), "asp.tdnn.conv": (c.att_channels, 3 * n, 1), "asp.conv": (n, c.att_channels, 1), "fc": (c.out_dim, 2 * n, 1)})
    sd = {}
    for k, s in names.items():
        sd["speaker_encoder." + k + ".weight"] = torch.randn(s, generator=g) * 0.2
        sd["speaker_encoder." + k + ".bias"] = torch.randn(s[0], generator=g) * 0.1

    class L:
        def load_tensor(self, n, dtype):
            return sd[n].to(dtype)
    m = Ecapa(c)
    speaker.load_into(m, L())
    assert sum(p.numel() for p in m.parameters()) == sum(v.numel() for v in sd.values())          # every parameter came from a name
    feats = torch.randn(c.n_mels, 29)
    v = m(feats)
    # the same network restated with functional calls straight from the dictionary
    import torch.nn.functional as F

    def conv(x, name, d=1, relu=True):
        w, b = sd["speaker_encoder." + name + ".weight"], sd["speaker_encoder." + name + ".bias"]
        tot = d * (w.shape[2] - 1)
        x = F.pad(x[None], (tot // 2, tot - tot // 2), mode="reflect") if tot else x[None]
        y = F.conv1d(x, w, b, dilation=d)[0]
        return F.relu(y) if relu else y
    h = conv(feats, "blocks.0.conv")
    hs = []
    for i, d in enumerate(c.dilations, start=1):
        res = h
        t = conv(h, f"blocks.{i}.tdnn1.conv")
        outs = []
        for j in range(c.res2net_scale):
            part = t[j * grp:(j + 1) * grp]
            outs.append(part if j == 0 else conv(part if j == 1 else part + outs[-1], f"blocks.{i}.res2net_block.blocks.{j - 1}.conv", d))
        t = conv(torch.cat(outs), f"blocks.{i}.tdnn2.conv")
        s = torch.sigmoid(conv(conv(t.mean(1, keepdim=True), f"blocks.{i}.se_block.conv1"), f"blocks.{i}.se_block.conv2", relu=False))
        h = t * s + res
        hs.append(h)
    h = conv(torch.cat(hs), "mfa.conv")
    T = h.shape[1]
    mean, std = h.mean(1, keepdim=True), h.var(1, unbiased=False, keepdim=True).clamp_min(1e-12).sqrt()
    a = conv(torch.tanh(conv(torch.cat([h, mean.expand(-1, T), std.expand(-1, T)]), "asp.tdnn.conv")), "asp.conv", relu=False).softmax(1)
    mu = (h * a).sum(1, keepdim=True)
    sg = ((h - mu) ** 2 * a).sum(1, keepdim=True).clamp_min(1e-12).sqrt()
    want = conv(torch.cat([mu, sg]), "fc", relu=False)[:, 0]
    assert torch.allclose(v, want, atol=1e-5), float((v - want).abs().max())
    bad = dict(sd)
    bad["speaker_encoder.fc.weight"] = torch.zeros(c.out_dim + 1, 2 * n, 1)

    class LB(L):
        def load_tensor(self, n, dtype):
            return bad[n].to(dtype)
    with pytest.raises(ValueError, match="speaker_encoder.fc.weight"):
        speaker.load_into(Ecapa(c), LB())
