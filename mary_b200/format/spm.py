"""SentencePiece UNIGRAM tokenizer read straight from a ``.model`` file (or from the typed piece table of a pile).

Reference: src/models/personaplex/spm.rs.  The model file is a proto2 ``ModelProto``; a read-only wire-format walker pulls out
what the tokenizer needs and REFUSES what this implementation does not restate, so that a different model file fails loudly
instead of tokenising differently (spm.rs:143-224): ``model_type`` must be UNIGRAM, the normaliser's ``precompiled_charsmap`` must
be empty (identity normalisation: prepend one dummy-prefix space when asked, escape U+0020 to U+2581, nothing else),
``remove_extra_whitespaces`` false, ``escape_whitespaces`` true, no USER_DEFINED pieces.

Encoding is Viterbi over UTF-8 character boundaries (spm.rs:272-383): every NORMAL piece that matches at a position is an edge
scored by its log-probability; a position that no single-character piece covers gets a one-character UNK edge at
``min score - 10``; ties keep the first best (strict ``>``).  On the way back UNK edges become the ``<0xXX>`` BYTE pieces of the
character's UTF-8 bytes (``byte_fallback``), or the unknown piece when the model has none.  Decoding concatenates raw piece bytes
(one byte for a BYTE piece), un-escapes U+2581 and only then decodes UTF-8, so a character split over byte pieces reassembles
(spm.rs:420-458)."""
from __future__ import annotations

import struct

META = "▁".encode("utf-8")
UNK_PENALTY = 10.0
NORMAL, UNKNOWN, CONTROL, USER_DEFINED, UNUSED, BYTE = 1, 2, 3, 4, 5, 6


def _fields(b: bytes):
    """``(field number, wire type, value)`` of one protobuf message; value is an int (varint) or bytes."""
    i, n = 0, len(b)

    def varint():
        nonlocal i
        x = s = 0
        while True:
            if i >= n:
                raise ValueError("spm proto: truncated varint")
            c = b[i]
            i += 1
            x |= (c & 0x7F) << s
            if not c & 0x80:
                return x
            s += 7
    while i < n:
        tag = varint()
        f, wt = tag >> 3, tag & 7
        if wt == 0:
            yield f, wt, varint()
        elif wt in (1, 5):
            w = 8 if wt == 1 else 4
            if i + w > n:
                raise ValueError("spm proto: truncated fixed field")
            yield f, wt, b[i:i + w]
            i += w
        elif wt == 2:
            ln = varint()
            if i + ln > n:
                raise ValueError("spm proto: truncated bytes field")
            yield f, wt, b[i:i + ln]
            i += ln
        else:
            raise ValueError(f"spm proto: unsupported wire type {wt}")


def parse_model(data: bytes):
    """``(pieces [(bytes, score, type)], add_dummy_prefix, byte_fallback)`` of a SentencePiece ``.model`` file."""
    pieces, trainer, normalizer = [], None, None
    for f, wt, v in _fields(data):
        if f == 1 and wt == 2:                       # ModelProto.pieces: {1 piece, 2 score (float), 3 type (default NORMAL)}
            piece, score, typ = b"", 0.0, NORMAL
            for pf, pwt, pv in _fields(v):
                if pf == 1:
                    piece = bytes(pv)
                elif pf == 2:
                    (score,) = struct.unpack("<f", pv)
                elif pf == 3:
                    typ = pv
            pieces.append((piece, score, typ))
        elif f == 2:
            trainer = v
        elif f == 3:
            normalizer = v
    if trainer is None or normalizer is None:
        raise ValueError("spm: the model file carries no trainer_spec / normalizer_spec")
    model_type, byte_fallback = 1, False              # TrainerSpec: 3 model_type (1 = UNIGRAM), 35 byte_fallback
    for f, _wt, v in _fields(trainer):
        if f == 3:
            model_type = v
        elif f == 35:
            byte_fallback = v != 0
    if model_type != 1:
        raise ValueError(f"spm: model_type {model_type}: only UNIGRAM is implemented")
    # NormalizerSpec: 2 precompiled_charsmap, 3 add_dummy_prefix, 4 remove_extra_whitespaces (proto2 default TRUE),
    # 5 escape_whitespaces (default true)
    charsmap, add_dummy_prefix, remove_extra, escape_ws = 0, True, True, True
    for f, _wt, v in _fields(normalizer):
        if f == 2:
            charsmap = len(v)
        elif f == 3:
            add_dummy_prefix = v != 0
        elif f == 4:
            remove_extra = v != 0
        elif f == 5:
            escape_ws = v != 0
    if charsmap:
        raise ValueError("spm: a precompiled_charsmap (NFKC-style normaliser) is not implemented")
    if remove_extra:
        raise ValueError("spm: remove_extra_whitespaces=true is not implemented")
    if not escape_ws:
        raise ValueError("spm: escape_whitespaces=false is not implemented")
    return pieces, add_dummy_prefix, byte_fallback


class SpmTokenizer:
    def __init__(self, pieces, add_dummy_prefix: bool = True):
        """``pieces``: rows ``(bytes, score, type)`` in id order (the table a pile's typed unigram graph gives back)."""
        self.add_dummy_prefix = add_dummy_prefix
        self.map: dict[bytes, tuple[int, float]] = {}
        self.byte_id = [-1] * 256
        self.surface: list[bytes] = []
        self.is_byte: list[bool] = []
        self.unk_id = -1
        self.max_len, min_score = 0, float("inf")
        for i, (piece, score, typ) in enumerate(pieces):
            piece = bytes(piece)
            if typ == NORMAL:
                self.max_len = max(self.max_len, len(piece))
                min_score = min(min_score, score)
                self.map.setdefault(piece, (i, float(score)))
                self.surface.append(piece)
                self.is_byte.append(False)
            elif typ == BYTE:                                            # "<0xAB>"
                s = piece.decode("ascii")
                if len(s) != 6 or not (s.startswith("<0x") and s.endswith(">")):
                    raise ValueError(f"spm: malformed byte piece {piece!r}")
                b = int(s[3:5], 16)
                self.byte_id[b] = i
                self.surface.append(bytes([b]))
                self.is_byte.append(True)
            elif typ == USER_DEFINED:
                raise ValueError("spm: USER_DEFINED pieces (always-match semantics) are not implemented")
            else:                                                       # UNKNOWN, CONTROL, UNUSED never match from text
                if typ == UNKNOWN and self.unk_id < 0:
                    self.unk_id = i
                self.surface.append(piece)
                self.is_byte.append(False)
        self.byte_fallback = all(b >= 0 for b in self.byte_id)
        if not self.byte_fallback and any(b >= 0 for b in self.byte_id):
            raise ValueError("spm: some but not all 256 byte pieces are present")
        if not self.byte_fallback and self.unk_id < 0:
            raise ValueError("spm: neither byte pieces nor an unknown piece: unknown characters cannot be encoded")
        self.unk_score = (min_score if self.map else 0.0) - UNK_PENALTY

    @staticmethod
    def load(path) -> "SpmTokenizer":
        with open(path, "rb") as f:
            pieces, prefix, _ = parse_model(f.read())
        return SpmTokenizer(pieces, prefix)

    def vocab_size(self) -> int:
        return len(self.surface)

    def piece_bytes(self, i: int) -> bytes:
        return self.surface[i]

    def encode(self, text: str) -> list[int]:
        if not text:
            return []
        norm = (META if self.add_dummy_prefix else b"") + text.replace(" ", "▁").encode("utf-8")
        n = len(norm)

        def clen(p):
            b = norm[p]
            return 1 if b < 0x80 else 4 if b >= 0xF0 else 3 if b >= 0xE0 else 2 if b >= 0xC0 else 0
        NEG = float("-inf")
        best = [NEG] * (n + 1)
        back = [(0, -2)] * (n + 1)
        best[0] = 0.0
        pos = 0
        while pos < n:
            cl = clen(pos)
            if cl == 0:
                raise ValueError("spm: lattice node on a continuation byte")
            if best[pos] > NEG:
                single, end = False, pos
                while end < n and end - pos < self.max_len:
                    c = clen(end)
                    if c == 0:
                        break
                    end += c
                    if end > n:
                        break
                    hit = self.map.get(norm[pos:end])
                    if hit is not None:
                        if best[pos] + hit[1] > best[end]:
                            best[end], back[end] = best[pos] + hit[1], (pos, hit[0])
                        if end - pos == cl:
                            single = True
                if not single and best[pos] + self.unk_score > best[pos + cl]:
                    best[pos + cl], back[pos + cl] = best[pos] + self.unk_score, (pos, -1)
            pos += cl
        if best[n] == NEG:
            raise ValueError("spm: the end of the text is unreachable")
        rev, pos = [], n
        while pos > 0:
            start, i = back[pos]
            if i >= 0:
                rev.append(i)
            elif self.byte_fallback:
                rev.extend(self.byte_id[b] for b in reversed(norm[start:pos]))
            else:
                rev.append(self.unk_id)
            pos = start
        return rev[::-1]

    @staticmethod
    def _unescape(raw: bytes) -> str:
        return raw.replace(META, b" ").decode("utf-8", errors="replace")

    def decode_token(self, i: int) -> str:
        return self._unescape(self.surface[i])

    def decode(self, ids) -> str:
        s = self._unescape(b"".join(self.surface[i] for i in ids))
        return s[1:] if self.add_dummy_prefix and s.startswith(" ") else s
