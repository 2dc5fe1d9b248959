"""Packaged voice prompts and the system-prompt flow of a Moshi-family dialogue model.

Reference: src/models/personaplex/voice_prompt.rs (the ``.pt`` package), prompt.rs (assembly), pipeline.rs:117-160 (the phases).
A packaged voice is ``{"embeddings": [N, 1, 1, dim], "cache": [1, streams, ring]}``: the temporal stack's INPUT embeddings of every
voice frame, replayed one step at a time in place of the embedding tables, and the token-ring snapshot that replaces the stream
cache after the replay.  Stock voices store bf16 (widening to f32 is exact), locally built ones f32.  The file is read with
:mod:`mary_b200.format.torch_pt`, which builds tensors and containers only and never runs the pickle.

Prompt phases (``run_prompt``): voice replay -> silence spacer -> text system prompt (one SentencePiece token per step, agent
silence and the user's reference sine alongside) -> silence spacer."""
from __future__ import annotations

from dataclasses import dataclass

import torch

from ...format.torch_pt import load_pt

SILENCE_TOKENS = [948, 243, 1178, 546, 1736, 1030, 1978, 2008]      # one frame of agent silence (codec tokens)
SINE_TOKENS = [430, 1268, 381, 1611, 1095, 1495, 56, 472]           # one frame of the user's reference sine
TEXT_PAD_TOKEN = 3
SILENCE_FRAMES = 6                                                  # int(0.5 * 12.5 Hz)


@dataclass
class VoicePrompt:
    embeddings: torch.Tensor          # [N, dim] f32
    cache: torch.Tensor               # [streams, ring] int64

    @property
    def n_frames(self) -> int:
        return self.embeddings.shape[0]

    @staticmethod
    def load(src, cfg) -> "VoicePrompt":
        obj = load_pt(src)
        if not isinstance(obj, dict) or "embeddings" not in obj or "cache" not in obj:
            raise ValueError("voice prompt: expected a dict with 'embeddings' and 'cache'")
        emb, cache = obj["embeddings"], obj["cache"]
        if emb.dim() != 4 or tuple(emb.shape[1:]) != (1, 1, cfg.dim) or not emb.is_floating_point():
            raise ValueError(f"voice prompt: embeddings {tuple(emb.shape)} {emb.dtype}, expected [N, 1, 1, {cfg.dim}] floating point")
        ring = cfg.max_delay + 3
        if tuple(cache.shape) != (1, cfg.num_streams, ring) or cache.dtype != torch.int64:
            raise ValueError(f"voice prompt: cache {tuple(cache.shape)} {cache.dtype}, expected [1, {cfg.num_streams}, {ring}] int64")
        return VoicePrompt(emb.reshape(-1, cfg.dim).float(), cache[0].clone())

    def save(self, path, dtype=torch.float32) -> None:
        """Write the package the way the upstream flow does (``torch.save`` of the two tensors)."""
        torch.save({"embeddings": self.embeddings.to(dtype).reshape(-1, 1, 1, self.embeddings.shape[1]), "cache": self.cache[None].clone()}, path)


def wrap_with_system_tags(text: str) -> str:
    """Add ``<system>`` tags unless present.  The tags are plain text to the tokenizer, not special tokens (prompt.rs:28-37)."""
    t = text.strip()
    return t if t.startswith("<system>") and t.endswith("<system>") else f"<system> {t} <system>"


@dataclass
class Prompt:
    voice: VoicePrompt
    text_tokens: list
    silence_frames: int = SILENCE_FRAMES

    @staticmethod
    def build(voice_src, spm, system_text: str, cfg) -> "Prompt":
        toks = spm.encode(wrap_with_system_tags(system_text)) if system_text else []
        return Prompt(VoicePrompt.load(voice_src, cfg), toks)

    def total_steps(self) -> int:
        return self.voice.n_frames + 2 * self.silence_frames + len(self.text_tokens)
