"""``LocalTextEngine``: chat turns in, one generation out (src/local.rs:1-260).

The playground side of the reference talks to a text model through this one trait, so that any local decoder can stand behind
it.  Gemma has no system turn: system content is folded into the NEXT user turn (a trailing system gets a user turn of its own);
a thinking model's output is split into channels — the last ``final`` / ``answer`` channel is the text, the others the reasoning —
and stop strings cut the final text only, after the split (src/local.rs:83-236)."""
from __future__ import annotations

import enum
from dataclasses import dataclass, field


class LocalRole(enum.Enum):
    SYSTEM = "system"
    USER = "user"
    ASSISTANT = "assistant"


@dataclass
class LocalChatTurn:
    role: LocalRole
    content: str


@dataclass
class LocalGenParams:
    """``temperature`` / ``top_p`` / ``seed`` are carried for callers that set them; decoding is greedy at temperature 0."""
    max_tokens: int = 128
    temperature: float = 0.0
    top_p: float | None = None
    stop: list = field(default_factory=list)
    seed: int | None = None


@dataclass
class LocalGeneration:
    text: str
    reasoning: str | None
    prompt_tokens: int
    completion_tokens: int


class LocalTextEngine:
    """The seam: anything with ``generate(turns, params) -> LocalGeneration``."""

    def generate(self, turns: list[LocalChatTurn], params: LocalGenParams) -> LocalGeneration:
        raise NotImplementedError


_MARKERS = ("<|channel>", "<channel|>", "<|think|>", "<|turn>", "<turn|>", "<bos>", "<eos>")


def strip_markers(s: str) -> str:
    for m in _MARKERS:
        s = s.replace(m, "")
    return s


def split_channels(raw: str) -> tuple[str, str | None]:
    """``(final text, reasoning | None)`` of a raw completion (src/local.rs:98-134)."""
    if "<|channel>" not in raw:
        return strip_markers(raw).strip(), None
    channels = []
    for seg in raw.split("<|channel>")[1:]:
        if "<channel|>" in seg:
            name, content = seg.split("<channel|>", 1)
            channels.append((name.strip().lower(), strip_markers(content).strip()))
        else:
            channels.append(("", strip_markers(seg).strip()))          # a header without its close marker: all of it is content
    if not channels:
        return strip_markers(raw).strip(), None
    final = max((i for i, (n, _) in enumerate(channels) if "final" in n or "answer" in n), default=len(channels) - 1)
    reasoning = [c for i, (_, c) in enumerate(channels) if i != final and c]
    return channels[final][1], ("\n".join(reasoning) if reasoning else None)


def apply_stop(text: str, stop: list[str]) -> str:
    cuts = [text.find(s) for s in stop if s and s in text]
    return text[:min(cuts)] if cuts else text


def build_chat(turns: list[LocalChatTurn]) -> str:
    s, sys_buf = "<bos>", ""
    for t in turns:
        if t.role is LocalRole.SYSTEM:
            sys_buf += t.content + "\n"
        elif t.role is LocalRole.USER:
            s += "<|turn>user\n" + sys_buf + t.content + "<turn|>\n"
            sys_buf = ""
        else:
            s += "<|turn>model\n" + t.content + "<turn|>\n"
    if sys_buf:
        s += "<|turn>user\n" + sys_buf + "<turn|>\n"
    return s + "<|turn>model\n"


class GemmaEngine(LocalTextEngine):
    def __init__(self, lm):
        self.lm = lm

    def generate(self, turns, params: LocalGenParams) -> LocalGeneration:
        chat = build_chat(turns)
        tok = self.lm.tokenizer
        if tok is None:
            raise RuntimeError("this pile holds no tokenizer")
        ids = tok.encode(chat, add_special_tokens=False).ids
        # generated in full (no early stop string), so that a thinking model's channels complete; the stop strings apply to the
        # FINAL channel after the split
        out = [t for t in self.lm.engine.generate([ids], params.max_tokens)[0] if t not in self.lm.engine.eos]
        text, reasoning = split_channels(tok.decode(out, skip_special_tokens=False))
        return LocalGeneration(apply_stop(text, params.stop), reasoning, len(ids), len(out))


def load_gemma4_from_pile(path, device="cpu", dtype=None, **kw) -> GemmaEngine:
    """Open a persisted Gemma-4 pile config-free and put it behind the seam (``load_gemma4_from_persisted_pile[_f16]``)."""
    import torch
    from ..models.gemma4.lm import GemmaLM
    dtype = dtype or (torch.bfloat16 if str(device).startswith("cuda") else torch.float32)
    return GemmaEngine(GemmaLM.from_pile(path, device=device, dtype=dtype, **kw))
