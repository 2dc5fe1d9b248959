"""STFT / inverse STFT as matrix products (src/models/f5: "STFT/ISTFT as DFT-matmul + conv"), so the spectral front and back ends
run on the same GEMM kernels as everything else.

Forward: frames (a strided view of the reflect-padded signal) times a ``[n_fft, 2 (n_fft / 2 + 1)]`` windowed DFT basis.
Inverse: the one-sided spectrum times the windowed inverse basis gives one ``n_fft``-sample frame per column; frames are
overlap-added (``fold``) and divided by the overlap-added squared window."""
from __future__ import annotations

import math

import torch
import torch.nn.functional as F


def _basis(n_fft: int, device, dtype=torch.float32):
    n = torch.arange(n_fft, dtype=torch.float64, device=device)
    k = torch.arange(n_fft // 2 + 1, dtype=torch.float64, device=device)
    ang = 2.0 * math.pi * n[:, None] * k[None, :] / n_fft
    return ang.cos().to(dtype), ang.sin().to(dtype)


def stft_matmul(wave, n_fft: int, hop: int, window=None):
    """``wave [L]`` -> complex ``[n_fft / 2 + 1, frames]`` (centred, reflect padding: the convention of ``torch.stft``)."""
    window = torch.hann_window(n_fft, device=wave.device) if window is None else window
    x = F.pad(wave[None, None].float(), (n_fft // 2, n_fft // 2), mode="reflect")[0, 0]
    frames = x.unfold(0, n_fft, hop) * window                                  # [frames, n_fft]
    cos, sin = _basis(n_fft, wave.device)
    return torch.complex(frames @ cos, -(frames @ sin)).T


def istft_matmul(spec, n_fft: int, hop: int, window=None, length: int | None = None):
    """Inverse of ``stft_matmul``: complex ``[n_fft / 2 + 1, frames]`` -> ``[L]``."""
    window = torch.hann_window(n_fft, device=spec.device) if window is None else window
    cos, sin = _basis(n_fft, spec.device)
    w = torch.full((n_fft // 2 + 1,), 2.0, device=spec.device)
    w[0] = 1.0
    if n_fft % 2 == 0:
        w[-1] = 1.0
    re, im = spec.real.T.float() * w, spec.imag.T.float() * w
    frames = (re @ cos.T - im @ sin.T) / n_fft * window                        # [frames, n_fft]
    T = frames.shape[0]
    total = n_fft + hop * (T - 1)
    y = F.fold(frames.T[None], (1, total), (1, n_fft), stride=(1, hop))[0, 0, 0]
    env = F.fold((window ** 2)[:, None].expand(-1, T)[None], (1, total), (1, n_fft), stride=(1, hop))[0, 0, 0]
    y = y / env.clamp_min(1e-11)
    if length is None:
        return y[n_fft // 2: total - n_fft // 2]
    y = y[n_fft // 2:][:length]                          # samples past the last hop still lie inside the last frames
    return F.pad(y, (0, length - y.shape[0]))


def mel_filterbank_htk(n_mels: int, n_fft: int, sr: int, fmin: float = 0.0, fmax: float | None = None):
    """Triangular filters on the HTK mel scale between ``fmin`` and ``fmax``, unnormalised, ``[n_mels, n_fft / 2 + 1]``."""
    def to_mel(f):
        return 2595.0 * math.log10(1.0 + f / 700.0)
    pts = torch.linspace(to_mel(fmin), to_mel(sr / 2 if fmax is None else fmax), n_mels + 2, dtype=torch.float64)
    hz = 700.0 * (10.0 ** (pts / 2595.0) - 1.0)
    freqs = torch.linspace(0, sr / 2, n_fft // 2 + 1, dtype=torch.float64)
    lo, mid, hi = hz[:-2, None], hz[1:-1, None], hz[2:, None]
    return torch.minimum((freqs - lo) / (mid - lo), (hi - freqs) / (hi - mid)).clamp_min(0.0).float()


def mel_spectrogram(wave, n_mels: int = 100, n_fft: int = 1024, hop: int = 256, sr: int = 24000):
    """Log-magnitude mel ``[n_mels, frames]``: ``log(clamp(mel_fb @ |STFT|, 1e-5))`` (24 kHz, 100 bins, hop 256 for F5 / Vocos)."""
    mag = stft_matmul(wave, n_fft, hop).abs()
    return (mel_filterbank_htk(n_mels, n_fft, sr).to(wave.device) @ mag).clamp_min(1e-5).log()
