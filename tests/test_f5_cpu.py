"""F5-TTS pieces: spectral transforms as matrix products against torch.stft / istft, the Vocos head, ConvNeXt-V2 global response
normalisation, AdaLN-zero gating, classifier-free guidance, the sway grid and the end-to-end text + reference -> waveform path."""
import math

import torch

from mary_b200.models.f5 import CFM, DiT, F5Config, Vocos, VocosConfig, istft_matmul, mel_spectrogram, stft_matmul, sway_times
from mary_b200.models.f5.dit import ConvNeXtV2Block, init_random_, rope_interleaved


def test_stft_and_istft_by_matrix_products_match_torch():
    torch.manual_seed(0)
    x = torch.randn(2000)
    for n_fft, hop in ((64, 16), (128, 32), (100, 25)):
        want = torch.stft(x, n_fft, hop, window=torch.hann_window(n_fft), return_complex=True)
        got = stft_matmul(x, n_fft, hop)
        assert got.shape == want.shape and torch.allclose(got, want, atol=2e-4)
        back = istft_matmul(got, n_fft, hop, length=2000)
        n = hop * (got.shape[1] - 1)                                    # samples the frames cover
        assert torch.allclose(back[:n], x[:n], atol=1e-4)
        assert torch.allclose(back, torch.istft(want, n_fft, hop, window=torch.hann_window(n_fft), length=2000), atol=1e-4)
    m = mel_spectrogram(x, n_mels=20, n_fft=128, hop=32, sr=8000)
    assert m.shape == (20, 2000 // 32 + 1) and m.min() >= math.log(1e-5) - 1e-6


def test_vocos_turns_mel_frames_into_hop_samples_each():
    c = VocosConfig.tiny()
    v = Vocos(c)
    init_random_(v, 0, 0.2)
    mel = torch.randn(c.n_mels, 9)
    wav = v(mel)
    assert wav.shape == (9 * c.hop,) and torch.isfinite(wav).all()
    spec = v.spectrum(mel)
    assert spec.shape == (c.n_fft // 2 + 1, 9) and spec.abs().max() <= 100.0 + 1e-3


def test_global_response_normalisation_and_rotary_pairs():
    b = ConvNeXtV2Block(8, 16)
    init_random_(b, 1, 0.3)
    x = torch.randn(11, 8)
    with torch.no_grad():
        b.grn_gamma.zero_()                       # gamma = beta = 0: GRN is the identity inside the MLP
        plain = b(x)
        b.grn_gamma.fill_(1.0)
        scaled = b(x)
    assert not torch.allclose(plain, scaled)
    q = torch.randn(5, 2, 8)
    inv = 1.0 / (10000.0 ** (torch.arange(0, 8, 2).float() / 8))
    r = rope_interleaved(q, torch.arange(5), inv)
    assert torch.allclose(r[0], q[0]) and torch.allclose(r.norm(dim=-1), q.norm(dim=-1), atol=1e-5)
    # pair (0, 1) at position 3 turns by 3 * inv[0] radians
    ang = math.atan2(r[3, 0, 1], r[3, 0, 0]) - math.atan2(q[3, 0, 1], q[3, 0, 0])
    assert math.isclose((ang - 3.0 + math.pi) % (2 * math.pi) - math.pi, 0.0, abs_tol=1e-4)


def _dit():
    m = DiT(F5Config.tiny())
    init_random_(m, 0, 0.2)
    return m


def test_adaln_zero_gates_text_and_reference_conditioning():
    m = _dit()
    c = m.c
    T = 14
    x, cond = torch.randn(T, c.n_mels), torch.randn(T, c.n_mels)
    text = [3, 5, 7, 2]
    with torch.no_grad():
        v = m(x, cond, text, 0.3)
        assert v.shape == (T, c.n_mels)
        assert not torch.allclose(m(x, cond, text, 0.7), v)                          # the flow time reaches the output
        assert not torch.allclose(m(x, cond, [3, 5, 8, 2], 0.3), v)                  # so does the text
        assert torch.allclose(m(x, cond, text, 0.3, drop_text=True), m(x, cond, [], 0.3))
        assert torch.allclose(m(x, cond, text, 0.3, drop_cond=True), m(x, torch.zeros_like(cond), text, 0.3))
        # zero modulation weights (the AdaLN-zero initialisation): gates are 0, every block is the identity
        saved = [(b.mod_w.clone(), b.mod_b.clone()) for b in m.blocks]
        for b in m.blocks:
            b.mod_w.zero_(), b.mod_b.zero_()
        base = m(x, cond, text, 0.3)
        for b in m.blocks:
            b.w_o.normal_()
        assert torch.allclose(m(x, cond, text, 0.3), base)
        for b, (w, bb) in zip(m.blocks, saved):
            b.mod_w.copy_(w), b.mod_b.copy_(bb)
    first = DiT(F5Config(**{**F5Config.tiny().__dict__, "pe_attn_head": 1}))
    first.load_state_dict(m.state_dict())
    with torch.no_grad():
        assert not torch.allclose(first(x, cond, text, 0.3), m(x, cond, text, 0.3))  # rotating one head only is a different model


def test_guidance_sway_grid_and_sampling_pipeline():
    m = _dit()
    c = m.c
    ts = sway_times(8, -1.0)
    assert ts[0] == 0 and math.isclose(float(ts[-1]), 1.0, abs_tol=1e-6) and (ts[1:] > ts[:-1]).all()
    assert float(ts[4]) < 0.5                                                        # the warp spends more steps near t = 0
    assert torch.allclose(sway_times(8, None), torch.linspace(0, 1, 9))
    T = 12
    x, cond = torch.randn(T, c.n_mels), torch.randn(T, c.n_mels)
    with torch.no_grad():
        v_c = m(x, cond, [1, 2], 0.4)
        v_u = m(x, cond, [1, 2], 0.4, drop_cond=True, drop_text=True)
        assert torch.allclose(CFM(m, cfg_strength=0.0).velocity(x, cond, [1, 2], 0.4), v_c)
        assert torch.allclose(CFM(m, cfg_strength=2.0).velocity(x, cond, [1, 2], 0.4), v_c + 2.0 * (v_c - v_u), atol=1e-5)
    ref = torch.randn(5, c.n_mels)
    g = torch.Generator().manual_seed(0)
    mel = CFM(m, nfe=4).sample(ref, [1, 2, 3, 4, 5, 6], 16, generator=g)
    assert mel.shape == (16, c.n_mels) and torch.equal(mel[:5], ref) and torch.isfinite(mel).all()
    voc = Vocos(VocosConfig(n_mels=c.n_mels, dim=16, ffn=32, layers=1, n_fft=64, hop=16))
    init_random_(voc, 2, 0.1)
    wav = voc(mel[5:].T.contiguous())
    assert wav.shape == (11 * 16,)


def test_mel_front_end_matches_torchaudio():
    """The reference mel of F5-TTS / Vocos is torchaudio's MelSpectrogram (magnitude, HTK scale, no normalisation) followed by
    log(clamp(1e-5)); the matrix-product version must agree with it."""
    import pytest
    ta = pytest.importorskip("torchaudio")
    torch.manual_seed(0)
    wave = torch.randn(24000 // 2) * 0.2
    want = ta.transforms.MelSpectrogram(sample_rate=24000, n_fft=1024, win_length=1024, hop_length=256, n_mels=100, power=1, center=True,
                                        normalized=False, norm=None)(wave).clamp_min(1e-5).log()
    got = mel_spectrogram(wave, n_mels=100, n_fft=1024, hop=256, sr=24000)
    assert got.shape == want.shape
    assert torch.allclose(got, want, atol=2e-3), float((got - want).abs().max())
