"""``speak``: streaming text-to-speech in process (src/speak.rs:417-485: ``SpeakStream``, ``synthesize_stream``, ``synthesize``).

The talker and the code predictor produce one frame of codebook tokens at a time; every frame goes to the streaming codec
decoder at once, so the first audio leaves after one frame instead of after the utterance (time to first audio is the number
the reference tunes, PORT_NOTES.md:165-166)."""
from __future__ import annotations

import numpy as np
import torch


class Speaker:
    """Talker + code predictor + codec, loaded once."""

    def __init__(self, talker, predictor, codec, cfg):
        self.talker, self.pred, self.codec, self.cfg = talker, predictor, codec, cfg

    @staticmethod
    def from_pile(pile_path: str, model: str = "qwen3tts", codec_name: str = "codec") -> "Speaker":
        from ..cli.families import _loader
        from ..models.codec.mimi import MimiCodec, MimiConfig
        from ..models.codec.mimi import load_into as load_codec
        from ..models.qwen3tts.model import CodePredictor, Qwen3TTSConfig, Talker
        from ..models.qwen3tts.model import load_into as load_tts
        cfg = Qwen3TTSConfig()
        talker, pred = Talker(cfg), CodePredictor(cfg)
        load_tts(talker, pred, _loader(pile_path, model))
        mc = MimiConfig()
        mc.num_codebooks, mc.codebook_size = cfg.num_code_groups, cfg.pred_vocab
        codec = MimiCodec(mc)
        load_codec(codec, _loader(pile_path, codec_name))
        return Speaker(talker, pred, codec, cfg)

    def synthesize_stream(self, text_ids, max_frames: int = 200, seed: int = 0, prefill: int = 4):
        """Generator of PCM chunks (float32 arrays), one per codec frame, in generation order."""
        from ..models.qwen3tts.model import SamplingParams, generate_frames
        cfg, talker, codec = self.cfg, self.talker, self.codec
        text = torch.as_tensor(list(text_ids), dtype=torch.int32)
        n0 = max(1, min(len(text), prefill))
        with torch.no_grad():
            pre = talker.embed_text(text[:n0]) + talker.embed_codec(torch.full((n0,), cfg.codec_pad, dtype=torch.int32))
            trailing = talker.embed_text(text[n0:]) if len(text) > n0 else torch.zeros(0, pre.shape[1])
            pad = talker.embed_text(torch.tensor([0], dtype=torch.int32))[0]
        chunks, state = [], [None]

        def sink(frame):
            codes = (torch.tensor(frame[:codec.c.num_codebooks], dtype=torch.long) % codec.c.codebook_size)[None]
            pcm, state[0] = codec.decode_step(codes, state[0])
            chunks.append(pcm.reshape(-1).float().cpu().numpy())
            return True
        # the frame loop calls the sink synchronously; handing the chunks out as a generator keeps the caller's loop simple
        generate_frames(talker, self.pred, pre, trailing, pad, SamplingParams(max_frames=max_frames, seed=seed), on_frame=sink)
        yield from chunks

    def synthesize(self, text_ids, **kw) -> np.ndarray:
        parts = list(self.synthesize_stream(text_ids, **kw))
        return np.concatenate(parts) if parts else np.zeros(0, dtype=np.float32)


def synthesize_stream(pile_path: str, text_ids, **kw):
    return Speaker.from_pile(pile_path).synthesize_stream(text_ids, **kw)


def synthesize(pile_path: str, text_ids, **kw) -> np.ndarray:
    return Speaker.from_pile(pile_path).synthesize(text_ids, **kw)


def synthesize_to_wav(pile_path: str, text_ids, out_path: str, **kw) -> float:
    from ..cli.families import write_wav
    sp = Speaker.from_pile(pile_path)
    pcm = sp.synthesize(text_ids, **kw)
    write_wav(out_path, pcm, sp.codec.c.sample_rate)
    return pcm.shape[0] / sp.codec.c.sample_rate
