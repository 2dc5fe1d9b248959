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
