"""Byte-level BPE in the tiktoken style, for the Kimi-K3 vocabulary (src/tiktoken.rs).

The rank table is the merge order: a pair may merge iff its concatenation is in the table, lowest rank
first.  Text is first split by a regular expression (``KIMI_K3_PAT_STR``, :52-61) and long inputs are
chunked before the regex runs (:67-68)."""
from __future__ import annotations

import regex

# Kimi-style pattern: Han runs, contractions-aware words, numbers of up to 3 digits, punctuation, whitespace.
KIMI_K3_PAT_STR = "|".join([
    r"[\p{Han}]+",
    r"[^\r\n\p{L}\p{N}]?[\p{Lu}\p{Lt}\p{Lm}\p{Lo}\p{M}&&[^\p{Han}]]*[\p{Ll}\p{Lm}\p{Lo}\p{M}&&[^\p{Han}]]+(?i:'s|'t|'re|'ve|'m|'ll|'d)?",
    r"[^\r\n\p{L}\p{N}]?[\p{Lu}\p{Lt}\p{Lm}\p{Lo}\p{M}&&[^\p{Han}]]+[\p{Ll}\p{Lm}\p{Lo}\p{M}&&[^\p{Han}]]*(?i:'s|'t|'re|'ve|'m|'ll|'d)?",
    r"\p{N}{1,3}",
    r" ?[^\s\p{L}\p{N}]+[\r\n]*",
    r"\s*[\r\n]+",
    r"\s+(?!\S)",
    r"\s+",
])
MAX_CHUNK_CHARS = 400_000
MAX_NO_WHITESPACE_CHARS = 25_000


class TikToken:
    def __init__(self, ranks: dict[bytes, int], pattern: str = KIMI_K3_PAT_STR, special: dict[str, int] | None = None):
        self.ranks = ranks
        self.special = dict(special or {})
        self.decoder = {i: t for t, i in ranks.items()}
        self.decoder.update({i: s.encode("utf-8") for s, i in self.special.items()})
        self._re = regex.compile(pattern, flags=regex.V1)
        self._special_re = regex.compile("|".join(regex.escape(s) for s in sorted(self.special, key=len, reverse=True))) \
            if self.special else None
        for b in range(256):
            if bytes([b]) not in ranks:
                raise ValueError(f"rank table lacks the single byte {b:#04x}")

    def _bpe(self, piece: bytes) -> list[int]:
        if piece in self.ranks:
            return [self.ranks[piece]]
        parts = [bytes([b]) for b in piece]
        while len(parts) > 1:
            best, best_i = None, -1
            for i in range(len(parts) - 1):
                r = self.ranks.get(parts[i] + parts[i + 1])
                if r is not None and (best is None or r < best):
                    best, best_i = r, i
            if best is None:
                break
            parts[best_i:best_i + 2] = [parts[best_i] + parts[best_i + 1]]
        return [self.ranks[p] for p in parts]

    def _chunks(self, text: str):
        for i in range(0, len(text), MAX_CHUNK_CHARS):
            yield text[i:i + MAX_CHUNK_CHARS]

    def encode_ordinary(self, text: str) -> list[int]:
        out: list[int] = []
        for chunk in self._chunks(text):
            for m in self._re.finditer(chunk):
                out.extend(self._bpe(m.group().encode("utf-8")))
        return out

    def encode(self, text: str, allow_special: bool = True) -> list[int]:
        if not allow_special or self._special_re is None:
            return self.encode_ordinary(text)
        out, pos = [], 0
        for m in self._special_re.finditer(text):
            out.extend(self.encode_ordinary(text[pos:m.start()]))
            out.append(self.special[m.group()])
            pos = m.end()
        out.extend(self.encode_ordinary(text[pos:]))
        return out

    def decode_bytes(self, ids) -> bytes:
        return b"".join(self.decoder[int(i)] for i in ids)

    def decode(self, ids) -> str:
        return self.decode_bytes(ids).decode("utf-8", errors="replace")
