"""Tokenizers stored as a graph of facts, and rebuilt from facts without a JSON side file.

Reference: src/tokenizer.rs — vocab entries, merges and added tokens are entities; the normalizer /
pre-tokenizer / decoder / post-processor pipeline is a tagged AST (ids :95-180, attrs :181-270);
``build_tokenizer`` constructs a HF ``tokenizers.Tokenizer`` from the facts (:1049-1290);
``save_tokenizer_json`` (:294) ingests a ``tokenizer.json``; ``CountingBlobs`` meters put rate (:52-93).

Layout: one tokenizer entity ``{tokenizer_name, pipeline document}``; the pipeline (everything in
``tokenizer.json`` except ``model.vocab``, ``model.merges`` and ``added_tokens``) is stored with
:mod:`jsonfacts` as a tagged tree; each vocab entry is ``{tok_of, token, token_id[, score]}``, each merge
``{merge_of, merge_rank, merge_left, merge_right}``, each added token ``{added_of, token, token_id, flags}``.
Token text is a ShortString when it fits in 32 bytes without NUL, else a blob handle.
"""
from __future__ import annotations

import json
import time

from ..pile.trible import (TribleBuilder, TribleSet, derived_id, fresh_id, r_f64, r_genid, r_shortstring, r_u256,
                           v_f64, v_genid, v_handle, v_shortstring, v_u256)
from . import jsonfacts
from .model import get_text, put_text

_A = lambda n: derived_id(b"mary_b200.tokenizer", n.encode())  # noqa: E731
TOKENIZER_NAME = _A("tokenizer_name")
TOKENIZER_KIND = _A("tokenizer_kind")
TOK_OF = _A("tok_of")
TOKEN_SHORT = _A("token_short")
TOKEN_LONG = _A("token_long")
TOKEN_ID = _A("token_id")
TOKEN_SCORE = _A("token_score")
MERGE_OF = _A("merge_of")
MERGE_RANK = _A("merge_rank")
MERGE_LEFT_S, MERGE_LEFT_L = _A("merge_left_short"), _A("merge_left_long")
MERGE_RIGHT_S, MERGE_RIGHT_L = _A("merge_right_short"), _A("merge_right_long")
ADDED_OF = _A("added_of")
ADDED_FLAGS = _A("added_flags")
RANK_B64 = _A("tiktoken_rank_bytes")      # tiktoken: token BYTES (not text) as a blob handle / short value
PATTERN = _A("tiktoken_pattern")

_FLAG_NAMES = ("single_word", "lstrip", "rstrip", "normalized", "special")


class CountingBlobs:
    """Store wrapper that counts puts and bytes, with a puts-per-second meter (src/tokenizer.rs:52-93)."""

    def __init__(self, inner):
        self.inner, self.puts, self.bytes, self._t0 = inner, 0, 0, time.time()

    def put(self, data):
        self.puts += 1
        self.bytes += len(memoryview(data).cast("B"))
        return self.inner.put(data)

    def rate(self) -> float:
        return self.puts / max(time.time() - self._t0, 1e-9)

    def __getattr__(self, k):
        return getattr(self.inner, k)


def _text_pair(store, s: str, short_attr: bytes, long_attr: bytes):
    b = s.encode("utf-8")
    if len(b) <= 32 and b"\x00" not in b and (not b or b[-1] != 0):
        return short_attr, v_shortstring(s)
    return long_attr, put_text(store, s)


def _read_text(store, facts: TribleSet, e: bytes, short_attr: bytes, long_attr: bytes) -> str:
    v = facts.maybe(e, short_attr)
    if v is not None:
        return r_shortstring(v)
    return get_text(store, facts.one(e, long_attr))


def save_tokenizer_json(store, tb: TribleBuilder, name: str, tokenizer_json: dict | str, owner: bytes | None = None) -> bytes:
    """Ingest a HF ``tokenizer.json`` (dict or text) as facts; returns the tokenizer entity id."""
    doc = json.loads(tokenizer_json) if isinstance(tokenizer_json, str) else json.loads(json.dumps(tokenizer_json))
    tid = derived_id(b"tokenizer", (owner or b""), name.encode())
    model = doc.get("model", {})
    vocab = model.pop("vocab", None)
    merges = model.pop("merges", None)
    added = doc.pop("added_tokens", None) or []
    kind = model.get("type", "BPE")
    jsonfacts.save_document(store, tb, f"tokenizer:{name}", doc, owner=tid)
    pairs = [(TOKENIZER_NAME, put_text(store, name)), (TOKENIZER_KIND, v_shortstring(kind))]
    if owner is not None:
        from . import schema as S
        pairs.append((S.OWNER, v_genid(owner)))
    tb.entity(pairs, id=tid)
    if isinstance(vocab, dict):                       # BPE / WordPiece: token -> id
        for tok, i in vocab.items():
            a, v = _text_pair(store, tok, TOKEN_SHORT, TOKEN_LONG)
            tb.entity([(TOK_OF, v_genid(tid)), (a, v), (TOKEN_ID, v_u256(i))])
    elif isinstance(vocab, list):                     # Unigram: [[piece, score], ...]
        for i, (tok, score) in enumerate(vocab):
            a, v = _text_pair(store, tok, TOKEN_SHORT, TOKEN_LONG)
            tb.entity([(TOK_OF, v_genid(tid)), (a, v), (TOKEN_ID, v_u256(i)), (TOKEN_SCORE, v_f64(score))])
    for r, m in enumerate(merges or []):
        l, rt = m.split(" ", 1) if isinstance(m, str) else m
        la, lv = _text_pair(store, l, MERGE_LEFT_S, MERGE_LEFT_L)
        ra, rv = _text_pair(store, rt, MERGE_RIGHT_S, MERGE_RIGHT_L)
        tb.entity([(MERGE_OF, v_genid(tid)), (MERGE_RANK, v_u256(r)), (la, lv), (ra, rv)])
    for t in added:
        flags = sum((1 << i) for i, f in enumerate(_FLAG_NAMES) if t.get(f))
        a, v = _text_pair(store, t["content"], TOKEN_SHORT, TOKEN_LONG)
        tb.entity([(ADDED_OF, v_genid(tid)), (a, v), (TOKEN_ID, v_u256(t["id"])), (ADDED_FLAGS, v_u256(flags))])
    return tid


def list_tokenizers(store, facts: TribleSet) -> dict[str, bytes]:
    return {get_text(store, v): e for e, v in facts.with_attr(TOKENIZER_NAME)}


def select_tokenizer(store, facts: TribleSet, name: str | None = None) -> bytes:
    """Exact-cardinality tokenizer selection (``TokenizerSelector``, src/selection.rs:36-43)."""
    toks = list_tokenizers(store, facts)
    if name is None:
        if len(toks) != 1:
            raise LookupError(f"{len(toks)} tokenizers in the pile, expected exactly 1")
        return next(iter(toks.values()))
    if name not in toks:
        raise LookupError(f"tokenizer {name!r} not found")
    return toks[name]


def load_tokenizer_json(store, facts: TribleSet, tid: bytes) -> dict:
    """Rebuild the ``tokenizer.json`` dict from facts."""
    name = get_text(store, facts.one(tid, TOKENIZER_NAME))
    doc = jsonfacts.load_document(store, facts, f"tokenizer:{name}", owner=tid)
    kind = r_shortstring(facts.one(tid, TOKENIZER_KIND))
    entries = []
    for e in facts.entities_where(TOK_OF, v_genid(tid)):
        i = r_u256(facts.one(e, TOKEN_ID))
        sc = facts.maybe(e, TOKEN_SCORE)
        entries.append((i, _read_text(store, facts, e, TOKEN_SHORT, TOKEN_LONG), r_f64(sc) if sc is not None else None))
    entries.sort()
    if kind == "Unigram":
        doc["model"]["vocab"] = [[t, s] for _, t, s in entries]
    else:
        doc["model"]["vocab"] = {t: i for i, t, _ in entries}
    merges = []
    for e in facts.entities_where(MERGE_OF, v_genid(tid)):
        merges.append((r_u256(facts.one(e, MERGE_RANK)), _read_text(store, facts, e, MERGE_LEFT_S, MERGE_LEFT_L),
                       _read_text(store, facts, e, MERGE_RIGHT_S, MERGE_RIGHT_L)))
    if merges or kind == "BPE":
        doc["model"]["merges"] = [[l, r] for _, l, r in sorted(merges)]
    added = []
    for e in facts.entities_where(ADDED_OF, v_genid(tid)):
        fl = r_u256(facts.one(e, ADDED_FLAGS))
        d = {"id": r_u256(facts.one(e, TOKEN_ID)), "content": _read_text(store, facts, e, TOKEN_SHORT, TOKEN_LONG)}
        d.update({f: bool(fl >> i & 1) for i, f in enumerate(_FLAG_NAMES)})
        added.append(d)
    doc["added_tokens"] = sorted(added, key=lambda d: d["id"])
    return doc


def build_tokenizer(store, facts: TribleSet, tid: bytes | None = None):
    """HF ``tokenizers.Tokenizer`` constructed from facts — no JSON file on disk."""
    from tokenizers import Tokenizer
    if tid is None:
        tid = select_tokenizer(store, facts)
    return Tokenizer.from_str(json.dumps(load_tokenizer_json(store, facts, tid)))


# --------------------------------------------------------------------------- tiktoken rank tables
def save_tiktoken(store, tb: TribleBuilder, name: str, ranks: dict[bytes, int], pattern: str,
                  special: dict[str, int] | None = None, owner: bytes | None = None) -> bytes:
    """Byte-level BPE rank table (the rank IS the merge order; src/tokenizer.rs:459, src/tiktoken.rs)."""
    tid = derived_id(b"tokenizer", (owner or b""), name.encode())
    tb.entity([(TOKENIZER_NAME, put_text(store, name)), (TOKENIZER_KIND, v_shortstring("tiktoken")),
               (PATTERN, put_text(store, pattern))], id=tid)
    # one blob holds the table (length-prefixed byte strings in rank order): 200k+ entities would add nothing
    import struct
    ordered = sorted(ranks.items(), key=lambda kv: kv[1])
    if [r for _, r in ordered] != list(range(len(ordered))):
        raise ValueError("tiktoken ranks must be 0..n-1 without gaps")
    blob = b"".join(struct.pack("<H", len(t)) + t for t, _ in ordered)
    tb.add(tid, RANK_B64, v_handle(store.put(blob)))
    for s, i in (special or {}).items():
        a, v = _text_pair(store, s, TOKEN_SHORT, TOKEN_LONG)
        tb.entity([(ADDED_OF, v_genid(tid)), (a, v), (TOKEN_ID, v_u256(i)), (ADDED_FLAGS, v_u256(1 << 4))])
    return tid


def load_tiktoken(store, facts: TribleSet, tid: bytes):
    import struct
    from .tiktoken import TikToken
    blob = bytes(store.get(facts.one(tid, RANK_B64)))
    ranks, o, i = {}, 0, 0
    while o < len(blob):
        (n,) = struct.unpack_from("<H", blob, o)
        ranks[blob[o + 2:o + 2 + n]] = i
        o += 2 + n
        i += 1
    special = {}
    for e in facts.entities_where(ADDED_OF, v_genid(tid)):
        special[_read_text(store, facts, e, TOKEN_SHORT, TOKEN_LONG)] = r_u256(facts.one(e, TOKEN_ID))
    return TikToken(ranks, get_text(store, facts.one(tid, PATTERN)), special)


def save_spm_unigram(store, tb: TribleBuilder, name: str, pieces: list[tuple[str, float]], unk_id: int = 0,
                     owner: bytes | None = None) -> bytes:
    """SentencePiece unigram model as facts (src/tokenizer.rs:1794): pieces with scores, metaspace pipeline."""
    doc = {"version": "1.0", "truncation": None, "padding": None, "added_tokens": [],
           "normalizer": None,
           "pre_tokenizer": {"type": "Metaspace", "replacement": "▁", "prepend_scheme": "always", "split": True},
           "post_processor": None,
           "decoder": {"type": "Metaspace", "replacement": "▁", "prepend_scheme": "always", "split": True},
           "model": {"type": "Unigram", "unk_id": unk_id, "vocab": [[p, float(s)] for p, s in pieces], "byte_fallback": False}}
    return save_tokenizer_json(store, tb, name, doc, owner)
