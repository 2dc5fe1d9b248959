"""Voxtral realtime against the Hugging Face implementation (random tiny weights loaded by name): full-utterance logits, the
streaming path chunk by chunk equal to the full pass, the delay conditioning, and the mel front end against the library's
feature extractor."""
import numpy as np
import pytest
import torch

from mary_b200.models.voxtral import VoxtralConfig, VoxtralListener, VoxtralModel, load_into, log_mel


class _DictLoader:
    def __init__(self, sd):
        self.sd = sd

    def load_tensor(self, n, dtype):
        return self.sd[n].to(dtype)


def _pair():
    transformers = pytest.importorskip("transformers")
    from transformers.models.voxtral_realtime import VoxtralRealtimeConfig, VoxtralRealtimeForConditionalGeneration
    c = VoxtralConfig.tiny()
    torch.manual_seed(0)
    rope = lambda th: {"rope_type": "default", "rope_theta": th}  # noqa: E731
    hf_cfg = VoxtralRealtimeConfig(
        audio_config=dict(hidden_size=c.a_hidden, intermediate_size=c.a_ffn, num_hidden_layers=c.a_layers, num_attention_heads=c.a_heads,
                          num_key_value_heads=c.a_heads, head_dim=c.a_head_dim, num_mel_bins=c.n_mels, sliding_window=c.a_window, rms_norm_eps=c.eps,
                          rope_parameters=rope(c.a_theta), max_position_embeddings=256, vocab_size=c.vocab),
        text_config=dict(vocab_size=c.vocab, hidden_size=c.hidden, intermediate_size=c.ffn, num_hidden_layers=c.layers,
                         num_attention_heads=c.heads, num_key_value_heads=c.kv_heads, head_dim=c.head_dim, rms_norm_eps=c.eps,
                         rope_parameters=rope(c.theta), sliding_window=c.window, max_position_embeddings=256, tie_word_embeddings=True),
        downsample_factor=c.downsample, default_num_delay_tokens=c.delay_tokens)
    for cc in (hf_cfg, hf_cfg.audio_config, hf_cfg.text_config):
        cc._attn_implementation = "eager"
    hf = VoxtralRealtimeForConditionalGeneration(hf_cfg).eval()
    with torch.no_grad():
        for n, p in hf.named_parameters():
            if p.dim() == 1:
                p.copy_((1.0 if "norm" in n else 0.0) + 0.1 * torch.randn_like(p))
            elif "ada_rms_norm" in n:
                p.copy_(0.3 * torch.randn_like(p))
    m = VoxtralModel(c)
    load_into(m, _DictLoader({k: v.detach() for k, v in hf.state_dict().items()}))
    return c, hf, m


def test_full_utterance_logits_match_huggingface_and_streaming_matches_full():
    c, hf, m = _pair()
    T = 20                                                    # 20 text positions = 160 mel frames = 80 encoder frames (window 12)
    mel = torch.randn(c.n_mels, 8 * T)
    ids = torch.randint(6, c.vocab, (T,))
    ids[0] = c.bos
    with torch.no_grad():
        want = hf(input_ids=ids[None], input_features=mel[None], num_delay_tokens=c.delay_tokens).logits[0]
        got = m(ids.tolist(), mel)
    assert torch.allclose(got, want, atol=3e-4, rtol=3e-4), float((got - want).abs().max())
    with torch.no_grad():
        other = m(ids.tolist(), mel, delay_tokens=5.0)
    assert (other - got).abs().max() > 1e-3                   # the delay code reaches the logits

    lis = VoxtralListener(m)
    toks = []
    for lo, hi in ((0, 3), (3, 4), (4, 11), (11, 20)):        # uneven chunks of whole text positions
        toks += lis.feed(mel[:, 8 * lo:8 * hi], forced=ids.tolist()[1:] + [0])
    assert toks == got.argmax(-1).tolist()


def test_free_running_listener_holds_the_pad_token_during_the_delay():
    c, hf, m = _pair()
    mel = torch.randn(c.n_mels, 8 * 7)
    lis = VoxtralListener(m, delay_tokens=3)
    out = lis.feed(mel[:, :24]) + lis.feed(mel[:, 24:])
    assert len(out) == 7 and lis.tokens == out
    # the same stream with the inputs spelled out: bos, the pad token while the position is inside the delay, then the model's
    # own previous choice
    forced = [c.pad, c.pad, c.pad] + out[3:6] + [0]
    again = VoxtralListener(m, delay_tokens=3).feed(mel, forced=forced)
    assert again == out
    wrong = VoxtralListener(m, delay_tokens=3).feed(mel, forced=[c.pad + 1] * 7)
    assert wrong[0] == out[0] and wrong != out


def test_log_mel_matches_the_library_feature_extractor():
    pytest.importorskip("transformers")
    from transformers.models.voxtral_realtime import VoxtralRealtimeFeatureExtractor
    fe = VoxtralRealtimeFeatureExtractor()
    rng = np.random.default_rng(0)
    wave = (0.1 * rng.standard_normal(16000)).astype(np.float32)
    want = torch.as_tensor(fe(wave, sampling_rate=16000, return_tensors="pt")["input_features"][0])
    got = log_mel(wave, n_mels=fe.feature_size, n_fft=fe.n_fft, hop=fe.hop_length, global_max=getattr(fe, "global_log_mel_max", 1.5))
    n = min(got.shape[1], want.shape[1])
    assert abs(got.shape[1] - want.shape[1]) <= 1
    assert torch.allclose(got[:, :n], want[:, :n], atol=2e-3), float((got[:, :n] - want[:, :n]).abs().max())
