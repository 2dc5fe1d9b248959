"""``say``: text -> waveform in a reference voice, in process (src/say.rs:148-211: ``synthesize`` / ``synthesize_to_wav``).

``Voice`` loads the DiT, the vocoder and the reference recording ONCE (what the warm server of ``say_serve`` keeps between
requests); every ``synthesize`` call then costs the flow sampler and the vocoder only.  Duration rule of the reference front
end: target frames = reference frames x (target characters / reference characters) / speed."""
from __future__ import annotations

import numpy as np
import torch


class Voice:
    def __init__(self, dit, vocoder, ref_wave: np.ndarray, sample_rate: int, ref_text: str, n_fft: int = 1024, hop: int = 256, nfe: int = 32,
                 cfg_strength: float = 2.0, speed: float = 1.0):
        from ..models.f5 import CFM, mel_spectrogram
        self.dit, self.voc, self.sr, self.ref_text, self.speed = dit, vocoder, sample_rate, ref_text, speed
        self.ref = mel_spectrogram(torch.as_tensor(ref_wave, dtype=torch.float32), n_mels=dit.c.n_mels, n_fft=n_fft, hop=hop, sr=sample_rate).T.contiguous()
        self.cfm = CFM(dit, nfe=nfe, cfg_strength=cfg_strength)

    @staticmethod
    def from_pile(pile_path: str, ref_wav_path: str, ref_text: str, model: str = "f5", vocoder: str = "vocos", **kw) -> "Voice":
        from ..cli.families import _loader, read_wav
        from ..models.f5 import DiT, F5Config, Vocos, VocosConfig
        from ..models.f5 import dit as f5
        from ..models.f5.vocos import load_into as load_vocos
        dit, voc = DiT(F5Config()), Vocos(VocosConfig())
        f5.load_into(dit, _loader(pile_path, model))
        load_vocos(voc, _loader(pile_path, vocoder))
        wav, sr = read_wav(ref_wav_path)
        return Voice(dit, voc, wav, sr, ref_text, **kw)

    def synthesize(self, text: str, seed: int = 0) -> np.ndarray:
        c = self.dit.c
        chars = [ord(ch) % (c.text_vocab - 1) for ch in self.ref_text + " " + text]      # byte-level ids when the pile holds no vocabulary
        total = self.ref.shape[0] + max(1, int(self.ref.shape[0] * len(text) / max(1, len(self.ref_text)) / self.speed))
        with torch.no_grad():
            mel = self.cfm.sample(self.ref, chars, total, generator=torch.Generator().manual_seed(seed))
            return self.voc(mel[self.ref.shape[0]:].T.contiguous()).float().cpu().numpy()


def synthesize(weights_pile: str, ref_wav: str, ref_text: str, gen_text: str, **kw) -> np.ndarray:
    """One-shot form: load, synthesise, return the samples (src/say.rs:148)."""
    return Voice.from_pile(weights_pile, ref_wav, ref_text, **kw).synthesize(gen_text)


def synthesize_to_wav(weights_pile: str, ref_wav: str, ref_text: str, gen_text: str, out_path: str, **kw) -> float:
    """Writes the waveform; returns its duration in seconds (src/say.rs:201)."""
    from ..cli.families import write_wav
    v = Voice.from_pile(weights_pile, ref_wav, ref_text, **kw)
    pcm = v.synthesize(gen_text)
    write_wav(out_path, pcm, v.sr)
    return pcm.shape[0] / v.sr
