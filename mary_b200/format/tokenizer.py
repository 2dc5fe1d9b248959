"""Tokenizers stored as a typed graph of facts, and rebuilt from facts without a JSON side file.

Reference: src/tokenizer.rs.  The attribute and tag ids below are the reference's own (tags :95-180, attributes :181-270), so a
pile written here answers the reference's queries and the other way round:

* a vocab entry is ``{piece, token_id}`` (a Unigram entry adds ``piece_score`` and a piece-type tag), a merge is
  ``{merge_left, merge_right, index = rank}``, an added token ``{piece, token_id, index = order}`` with ``SPECIAL`` /
  ``NORMALIZED`` flag tags; entries are content-derived entities that the tokenizer points at through ``vocab`` / ``merge`` /
  ``added`` edges (:294-526);
* the tokenizer entity carries its model type as a tag (``WORD_PIECE`` / ``BPE`` / ``UNIGRAM`` / ``TIKTOKEN``), ``model_name``,
  the flat model knobs and one edge per pipeline role (``normalizer``, ``pre_tokenizer``, ``decoder``, ``post_processor``);
* a pipeline node is a tagged entity: its type and its true booleans are tags, regex / behaviour / prefix are flat attributes and a
  ``Sequence`` lists its children through ``member`` edges that carry an ``index`` (``save_config_node``, :533-638);
* a tiktoken rank table is ``{piece_bytes, token_id = rank}`` per entry plus one ``TIKTOKEN_PRE_TOKENIZER`` node (:459-526); a
  SentencePiece unigram model is its scored, typed piece table (:1794-1857).

What the reference's schema has no place for is kept so that ``tokenizer.json`` round-trips exactly.  A pipeline node that the
typed form cannot restate field for field (``Metaspace``, ``TemplateProcessing``, ``NFKC`` ...) is stored as an ``OPAQUE`` node
over a :mod:`jsonfacts` subtree; the remaining top-level and model fields (``version``, ``truncation``, ``dropout`` ...) are one
small :mod:`jsonfacts` document owned by the tokenizer; the added-token booleans the reference defers (``single_word``,
``lstrip``, ``rstrip``) are extension flag tags.  The extension ids are minted in this package's namespace and never collide
with the reference's.  ``build_tokenizer`` constructs a HF ``tokenizers.Tokenizer`` from the facts (:1049-1290);
``CountingBlobs`` meters the put rate (:52-93)."""
from __future__ import annotations

import json
import time

from ..pile.trible import (TribleBuilder, TribleSet, derived_id, id_hex, r_bool, r_f64, r_genid, r_shortstring, r_u256, v_bool,
                           v_f64, v_genid, v_handle, v_shortstring, v_u256)
from . import jsonfacts
from .model import get_text, put_text
from .schema import INDEX, MEMBER, META_TAG, MODEL_NAME


class ty:
    """Node and model type tags (src/tokenizer.rs:95-138)."""
    BERT_NORMALIZER = id_hex("AC009EBADB3488042EDCD3D2C8648342")
    SEQUENCE = id_hex("33E6588376EEEDCBD4CD16DA197B7F90")
    NFC = id_hex("4D9204FC08700571D2407B74C0348DE0")
    REPLACE = id_hex("48927BD29F9321104585A69B1B541812")
    LOWERCASE = id_hex("C670B7A8105E77D2F6EF0DA05A8F5C99")
    BERT_PRE_TOKENIZER = id_hex("A6259970638C680F95F061D9EA7F2975")
    SPLIT = id_hex("B39A4D683D9B44F7D72BE118DA8E46BD")
    BYTE_LEVEL = id_hex("4FDB5C7C0999B4DECA894AD75E5A94C6")
    WORD_PIECE = id_hex("85A060015E6E94F70479E0E6B6BE0D98")
    BPE = id_hex("71F4DAC1D6392375923D7A2A9FA53650")
    TIKTOKEN = id_hex("BB88D3A2CAFF2AAA7DC00CA78945CC2E")
    TIKTOKEN_PRE_TOKENIZER = id_hex("AF6D6B71213E710F92E434D451540805")
    UNIGRAM = id_hex("AAC02E8BB835F423DF9EA5C0BAA3CAD6")
    PIECE_NORMAL = id_hex("EEEA86BCCE689C062D7C26EF1EEF936A")
    PIECE_UNKNOWN = id_hex("8F7B8C418D447BA7E45CEA8BB4914AC2")
    PIECE_CONTROL = id_hex("3EE7240B7CB58403D1DF30E39277CFF2")
    PIECE_USER_DEFINED = id_hex("9796A2F548F7C646D1798EFE7E8B4001")
    PIECE_BYTE = id_hex("9D9E4D16DD83083B49D34056344FD082")
    PIECE_UNUSED = id_hex("DD28C23E8DE557BC00F0451A8ED7C1C6")
    # extension: a pipeline node kept as a JSON subtree because the typed form cannot restate it
    OPAQUE = derived_id(b"mary_b200.tokenizer", b"ty.opaque")


class flag:
    """Boolean options as tags, presence = true (src/tokenizer.rs:144-178)."""
    CLEAN_TEXT = id_hex("C3A27148CDE4AC009B47E1EE141D477B")
    HANDLE_CHINESE_CHARS = id_hex("56D740D98D843D6E9B3E7CEB09B1949D")
    LOWERCASE = id_hex("46D626BCA9C575916A51DAAF0D4A3E16")
    INVERT = id_hex("1C84B18C4CD06F912C6FAF93FD64C48A")
    ADD_PREFIX_SPACE = id_hex("19B8979BAED4ADF439A7C8867ABC8727")
    TRIM_OFFSETS = id_hex("E7CC5D08B8995F31A4736B1482124071")
    CLEANUP = id_hex("42A792CDD8594CE881541C784C65B03F")
    FUSE_UNK = id_hex("39F4E0AF4C309CB77AADD1EB33495967")
    SPECIAL = id_hex("BBB4BCA9CA25CAB5F2ECABF787B0A638")
    NORMALIZED = id_hex("266A99918C6951D5C9F2D0A961C05D4A")
    USE_REGEX = id_hex("32F9C0904E02BC40F2FF723966A88D8E")
    IGNORE_MERGES = id_hex("22B7385E0FFC80CFAB80AE750557F784")
    # extensions: what the reference defers or folds away
    SINGLE_WORD = derived_id(b"mary_b200.tokenizer", b"flag.single_word")
    LSTRIP = derived_id(b"mary_b200.tokenizer", b"flag.lstrip")
    RSTRIP = derived_id(b"mary_b200.tokenizer", b"flag.rstrip")
    PATTERN_IS_STRING = derived_id(b"mary_b200.tokenizer", b"flag.pattern_is_string")
    STRIP_ACCENTS = derived_id(b"mary_b200.tokenizer", b"flag.strip_accents")
    KEEP_ACCENTS = derived_id(b"mary_b200.tokenizer", b"flag.keep_accents")


# attributes (src/tokenizer.rs:181-270); INDEX, MEMBER and MODEL_NAME are shared with the model schema
TOKENIZER = id_hex("E7014108A8F9512B19E3E8272E8A71F9")
VOCAB = id_hex("E839AA8F549C0D608FB86476A1EF3416")
MERGE = id_hex("E229769197BB035A2D6F61BC6A7D44BC")
ADDED = id_hex("B2553118F4CAAF1D028619956DE7F145")
NORMALIZER = id_hex("53BAF87A0E7F1410F8212B3EDF2A498C")
PRE_TOKENIZER = id_hex("6EEBF39CADD11B7CFBB624019AE21585")
POST_PROCESSOR = id_hex("98EC58B28F4D0BB43965DF7C5FF22713")
DECODER = id_hex("F3AAA4CD8EE04E5592059564A21FE953")
PIECE = id_hex("AE7FE29F2F38153F58C542D5CA4A9356")
TOKEN_ID = id_hex("F0E2E782F7BB62F52B1186DDE0EB5388")
PIECE_BYTES = id_hex("714AE13F801202EB27C83E3AB2290669")
MERGE_LEFT = id_hex("5723ECE1FF426C58879B79D5669A7CF1")
MERGE_RIGHT = id_hex("5C78FEB151F35A2C5D07BEC92E860752")
UNK_TOKEN = id_hex("68F1A9E6ED735E7C3ADCCA076AFF1742")
CONTINUING_SUBWORD_PREFIX = id_hex("11F76A2C0856C16CB030C4327D5A3B93")
END_OF_WORD_SUFFIX = id_hex("6FB969E8A3EDD1A657C721DD5A7D42EA")
MAX_INPUT_CHARS = id_hex("DF3F88DBFA2B44A7783169C9640014AF")
PIECE_SCORE = id_hex("3BCB70478942DB710ED2A4FB023F3457")
BYTE_FALLBACK = id_hex("EE4C6647619A836326196F0DBF84FA98")
PATTERN = id_hex("C8262D5668B8A1F541B3C35D54201BEC")
REPLACE_CONTENT = id_hex("3AC7574C07D02D389B4E7AD3B3B084D9")
BEHAVIOR = id_hex("964B4FCF7477E7E4436F0325F89B7CB5")
OPAQUE_VALUE = derived_id(b"mary_b200.tokenizer", b"opaque_value")     # extension: OPAQUE node -> jsonfacts root
MERGE_RANK = INDEX                                                      # a merge's rank is its ``index``

MODEL_TAGS = {"WordPiece": ty.WORD_PIECE, "BPE": ty.BPE, "Unigram": ty.UNIGRAM, "tiktoken": ty.TIKTOKEN}
_MODEL_OF_TAG = {v: k for k, v in MODEL_TAGS.items()}
_ROLES = (("normalizer", NORMALIZER, "normalizers"), ("pre_tokenizer", PRE_TOKENIZER, "pretokenizers"),
          ("post_processor", POST_PROCESSOR, "processors"), ("decoder", DECODER, "decoders"))
_SPM_TAGS = {1: ty.PIECE_NORMAL, 2: ty.PIECE_UNKNOWN, 3: ty.PIECE_CONTROL, 4: ty.PIECE_USER_DEFINED, 5: ty.PIECE_UNUSED,
             6: ty.PIECE_BYTE}
_SPM_OF_TAG = {v: k for k, v in _SPM_TAGS.items()}
_ADDED_FLAGS = (("single_word", flag.SINGLE_WORD), ("lstrip", flag.LSTRIP), ("rstrip", flag.RSTRIP),
                ("normalized", flag.NORMALIZED), ("special", flag.SPECIAL))


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


class _Intern:
    """Every distinct string is put ONCE per ingest: all merge halves are vocab pieces already, so a 200k-piece tokenizer would
    otherwise ask the store a million times for the same handles (src/tokenizer.rs:305-338)."""

    def __init__(self, store):
        self.store, self.memo = store, {}

    def __call__(self, s: str) -> bytes:
        h = self.memo.get(s)
        if h is None:
            h = self.memo[s] = put_text(self.store, s)
        return h


def _short_ok(s) -> bool:
    if not isinstance(s, str) or not s:
        return False
    b = s.encode("utf-8")
    return len(b) <= 32 and b"\x00" not in b


def _tags(facts: TribleSet, e: bytes) -> set:
    return {r_genid(v) for v in facts.values(e, META_TAG)}


def node_tags(facts: TribleSet, node: bytes) -> list[bytes]:
    """The tag ids a node carries (src/tokenizer.rs:795-800)."""
    return sorted(_tags(facts, node))


def ordered_members(facts: TribleSet, node: bytes) -> list[bytes]:
    """A ``Sequence`` node's children in ``index`` order; a child without exactly one index is an error
    (``ordered_members_strict``, src/tokenizer.rs:817-851)."""
    kids = []
    for v in facts.values(node, MEMBER):
        c = r_genid(v)
        idx = facts.values(c, INDEX)
        if len(idx) != 1:
            raise ValueError(f"sequence member {c.hex()} carries {len(idx)} index facts, expected 1")
        kids.append((r_u256(idx[0]), c))
    kids.sort()
    if [i for i, _ in kids] != list(range(len(kids))):
        raise ValueError(f"sequence members are not numbered 0..{len(kids) - 1}: {[i for i, _ in kids]}")
    return [c for _, c in kids]


# --------------------------------------------------------------------------- pipeline nodes
def _typed_pairs(v: dict, intern) -> list | None:
    """The reference's typed form of one pipeline node (children excluded), or None when it has no type tag for it."""
    t = v.get("type")

    def flags(*names):
        return [(META_TAG, v_genid(f)) for key, f in names if v.get(key) is True]

    def pattern():
        p = v.get("pattern")
        if not isinstance(p, dict) or len(p) != 1:
            return None
        (kind, s), = p.items()
        if kind not in ("Regex", "String") or not isinstance(s, str):
            return None
        return [(PATTERN, intern(s))] + ([(META_TAG, v_genid(flag.PATTERN_IS_STRING))] if kind == "String" else [])

    if t == "BertNormalizer":
        sa = v.get("strip_accents")
        extra = [] if sa is None else [(META_TAG, v_genid(flag.STRIP_ACCENTS if sa else flag.KEEP_ACCENTS))]
        return [(META_TAG, v_genid(ty.BERT_NORMALIZER))] + extra + flags(
            ("clean_text", flag.CLEAN_TEXT), ("handle_chinese_chars", flag.HANDLE_CHINESE_CHARS), ("lowercase", flag.LOWERCASE))
    if t in ("NFC", "Lowercase", "BertPreTokenizer"):
        return [(META_TAG, v_genid({"NFC": ty.NFC, "Lowercase": ty.LOWERCASE, "BertPreTokenizer": ty.BERT_PRE_TOKENIZER}[t]))]
    if t == "Replace":
        p = pattern()
        if p is None or not _short_ok(v.get("content")):
            return None
        return [(META_TAG, v_genid(ty.REPLACE)), (REPLACE_CONTENT, v_shortstring(v["content"]))] + p
    if t == "Split":
        p = pattern()
        if p is None or not _short_ok(v.get("behavior")):
            return None
        return [(META_TAG, v_genid(ty.SPLIT)), (BEHAVIOR, v_shortstring(v["behavior"]))] + p + flags(("invert", flag.INVERT))
    if t == "ByteLevel":
        # an absent ``use_regex`` means true (the HF default): reading only an explicit true would turn every tokenizer that omits
        # the field into a ``use_regex: false`` one (src/tokenizer.rs:611-616)
        ur = [(META_TAG, v_genid(flag.USE_REGEX))] if v.get("use_regex", True) else []
        return [(META_TAG, v_genid(ty.BYTE_LEVEL))] + ur + flags(("add_prefix_space", flag.ADD_PREFIX_SPACE),
                                                                 ("trim_offsets", flag.TRIM_OFFSETS))
    if t == "WordPiece":                                       # the decoder role; the model WordPiece is the tokenizer entity
        if not _short_ok(v.get("prefix")):
            return None
        return [(META_TAG, v_genid(ty.WORD_PIECE)), (CONTINUING_SUBWORD_PREFIX, v_shortstring(v["prefix"]))] + flags(
            ("cleanup", flag.CLEANUP))
    return None


def _node_json(store, facts: TribleSet, node: bytes, seq_key: str) -> dict:
    """The ``tokenizer.json`` form of one pipeline node (the inverse of :func:`save_config_node`)."""
    tags = _tags(facts, node)

    def pat():
        return {"String" if flag.PATTERN_IS_STRING in tags else "Regex": get_text(store, facts.one(node, PATTERN))}

    if ty.OPAQUE in tags:
        return jsonfacts.load_json(store, facts, r_genid(facts.one(node, OPAQUE_VALUE)))
    if ty.SEQUENCE in tags:
        return {"type": "Sequence", seq_key: [_node_json(store, facts, c, seq_key) for c in ordered_members(facts, node)]}
    if ty.BERT_NORMALIZER in tags:
        sa = True if flag.STRIP_ACCENTS in tags else False if flag.KEEP_ACCENTS in tags else None
        return {"type": "BertNormalizer", "clean_text": flag.CLEAN_TEXT in tags, "handle_chinese_chars": flag.HANDLE_CHINESE_CHARS in tags,
                "strip_accents": sa, "lowercase": flag.LOWERCASE in tags}
    if ty.NFC in tags:
        return {"type": "NFC"}
    if ty.LOWERCASE in tags:
        return {"type": "Lowercase"}
    if ty.BERT_PRE_TOKENIZER in tags:
        return {"type": "BertPreTokenizer"}
    if ty.REPLACE in tags:
        return {"type": "Replace", "pattern": pat(), "content": r_shortstring(facts.one(node, REPLACE_CONTENT))}
    if ty.SPLIT in tags:
        return {"type": "Split", "pattern": pat(), "behavior": r_shortstring(facts.one(node, BEHAVIOR)), "invert": flag.INVERT in tags}
    if ty.BYTE_LEVEL in tags:
        return {"type": "ByteLevel", "add_prefix_space": flag.ADD_PREFIX_SPACE in tags, "trim_offsets": flag.TRIM_OFFSETS in tags,
                "use_regex": flag.USE_REGEX in tags}
    if ty.WORD_PIECE in tags:
        return {"type": "WordPiece", "prefix": r_shortstring(facts.one(node, CONTINUING_SUBWORD_PREFIX)), "cleanup": flag.CLEANUP in tags}
    if ty.TIKTOKEN_PRE_TOKENIZER in tags:
        return {"type": "Split", "pattern": {"Regex": get_text(store, facts.one(node, PATTERN))}, "behavior": "Isolated", "invert": False}
    raise ValueError(f"pipeline node {node.hex()} carries no known type tag")


def save_config_node(store, tb: TribleBuilder, v: dict, seq_key: str, intern=None, index: int | None = None) -> bytes:
    """Ingest one pipeline subtree; returns its entity id (src/tokenizer.rs:533-638).  ``seq_key`` is the name a ``Sequence`` of
    this role gives its children; ``index`` is the node's position under its parent, part of the node's identity so that two equal
    steps of one sequence stay two nodes."""
    intern = intern or _Intern(store)
    pos = [] if index is None else [(INDEX, v_u256(index))]
    if v.get("type") == "Sequence" and isinstance(v.get(seq_key), list) and set(v) == {"type", seq_key}:
        kids = [save_config_node(store, tb, c, seq_key, intern, i) for i, c in enumerate(v[seq_key])]
        return tb.entity([(META_TAG, v_genid(ty.SEQUENCE))] + pos + [(MEMBER, v_genid(k)) for k in kids])
    pairs = _typed_pairs(v, intern)
    if pairs is not None:
        # typed only when the typed form restates the node field for field; a node with fields the schema has no place for
        # (or defaults that differ) keeps every field as an opaque subtree instead of losing some
        probe = TribleBuilder()
        nid = probe.entity(pairs)
        if _node_json(store, probe.build(), nid, seq_key) == v:
            return tb.entity(pairs + pos)
    root = jsonfacts.save_json(store, tb, v)
    return tb.entity([(META_TAG, v_genid(ty.OPAQUE)), (OPAQUE_VALUE, v_genid(root))] + pos)


# --------------------------------------------------------------------------- tokenizer.json
def _merge_pair(m):
    """A merge is ``["a", "b"]`` in newer files and ``"a b"`` in older ones (src/tokenizer.rs:274-292)."""
    if isinstance(m, str):
        l, _, r = m.partition(" ")
        return l, r
    l, r = m
    return l, r


def _residual_name(name: str) -> str:
    return f"tokenizer:{name}"


def _link(tb: TribleBuilder, tid: bytes, owner: bytes | None) -> None:
    if owner is not None:
        tb.add(owner, TOKENIZER, v_genid(tid))


def save_tokenizer_json(store, tb: TribleBuilder, name: str, tokenizer_json: dict | str, owner: bytes | None = None) -> bytes:
    """Ingest a HF ``tokenizer.json`` (dict or text) as facts; returns the tokenizer entity id (src/tokenizer.rs:294-526).  With
    ``owner`` the model root gains a ``tokenizer`` edge to it."""
    doc = json.loads(tokenizer_json) if isinstance(tokenizer_json, str) else json.loads(json.dumps(tokenizer_json))
    intern = _Intern(store)
    model = dict(doc.pop("model", None) or {})
    kind = model.pop("type", "BPE")
    if kind not in ("WordPiece", "BPE", "Unigram"):
        raise ValueError(f"unsupported tokenizer model type: {kind!r}")
    vocab, merges = model.pop("vocab", None), model.pop("merges", None)
    added = doc.pop("added_tokens", None) or []
    pairs = [(META_TAG, v_genid(MODEL_TAGS[kind])), (MODEL_NAME, intern(name))]

    if isinstance(vocab, dict):                       # BPE / WordPiece: piece -> id
        for tok, i in vocab.items():
            pairs.append((VOCAB, v_genid(tb.entity([(PIECE, intern(tok)), (TOKEN_ID, v_u256(i))]))))
    elif isinstance(vocab, list):                     # Unigram: [[piece, score], ...]; the id is the position
        unk, bf = model.get("unk_id"), bool(model.get("byte_fallback"))
        for i, (tok, score) in enumerate(vocab):
            typ = 2 if i == unk else 6 if bf and len(tok) == 6 and tok.startswith("<0x") and tok.endswith(">") else 1
            pairs.append((VOCAB, v_genid(tb.entity([(META_TAG, v_genid(_SPM_TAGS[typ])), (PIECE, intern(tok)), (TOKEN_ID, v_u256(i)),
                                                    (PIECE_SCORE, v_f64(float(score)))]))))
    for rank, m in enumerate(merges or []):
        l, r = _merge_pair(m)
        pairs.append((MERGE, v_genid(tb.entity([(MERGE_LEFT, intern(l)), (MERGE_RIGHT, intern(r)), (INDEX, v_u256(rank))]))))
    for order, t in enumerate(added):
        fl = [(META_TAG, v_genid(f)) for key, f in _ADDED_FLAGS if t.get(key) is True]
        pairs.append((ADDED, v_genid(tb.entity([(PIECE, intern(t["content"])), (TOKEN_ID, v_u256(t["id"])),
                                                (INDEX, v_u256(order))] + fl))))

    # flat model knobs: typed when the schema can hold the value, else they stay in the residual document
    for key, attr in (("unk_token", UNK_TOKEN), ("continuing_subword_prefix", CONTINUING_SUBWORD_PREFIX),
                      ("end_of_word_suffix", END_OF_WORD_SUFFIX)):
        if _short_ok(model.get(key)):
            pairs.append((attr, v_shortstring(model.pop(key))))
    if isinstance(model.get("max_input_chars_per_word"), int):
        pairs.append((MAX_INPUT_CHARS, v_u256(model.pop("max_input_chars_per_word"))))
    if isinstance(model.get("byte_fallback"), bool):
        pairs.append((BYTE_FALLBACK, v_bool(model.pop("byte_fallback"))))
    for key, f in (("ignore_merges", flag.IGNORE_MERGES), ("fuse_unk", flag.FUSE_UNK)):
        if model.get(key) is True:
            model.pop(key)
            pairs.append((META_TAG, v_genid(f)))
    for key, attr, seq_key in _ROLES:
        if isinstance(doc.get(key), dict):            # an explicit null is a statement of the file too; the residual keeps it
            pairs.append((attr, v_genid(save_config_node(store, tb, doc.pop(key), seq_key, intern))))

    tid = tb.entity(pairs)
    doc["model"] = model
    jsonfacts.save_document(store, tb, _residual_name(name), doc, owner=tid)
    _link(tb, tid, owner)
    return tid


def find_tokenizers(facts: TribleSet) -> list[bytes]:
    """Entities that carry a model type tag AND a ``model_name``: the name keeps the WordPiece DECODER node, which shares the
    ``WORD_PIECE`` tag, out of the answer (src/tokenizer.rs:767-793)."""
    named = {e for e, _ in facts.with_attr(MODEL_NAME)}
    return sorted(e for e in named if _tags(facts, e) & set(_MODEL_OF_TAG))


def list_tokenizers(store, facts: TribleSet) -> dict[str, bytes]:
    return {get_text(store, facts.one(e, MODEL_NAME)): e for e in find_tokenizers(facts)}


def tokenizer_kind(facts: TribleSet, tid: bytes) -> str:
    kinds = [_MODEL_OF_TAG[t] for t in _tags(facts, tid) if t in _MODEL_OF_TAG]
    if len(kinds) != 1:
        raise ValueError(f"tokenizer {tid.hex()} carries {len(kinds)} model type tags, expected 1")
    return kinds[0]


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


def load_vocab(store, facts: TribleSet, tid: bytes) -> list[tuple[int, str, float | None]]:
    """``(id, piece, score)`` rows in id order; two entries with one id are an error (``load_vocab_strict``, :877-917)."""
    rows = []
    for v in facts.values(tid, VOCAB):
        e = r_genid(v)
        sc = facts.maybe(e, PIECE_SCORE)
        rows.append((r_u256(facts.one(e, TOKEN_ID)), get_text(store, facts.one(e, PIECE)), r_f64(sc) if sc is not None else None))
    rows.sort(key=lambda r: r[0])
    for a, b in zip(rows, rows[1:]):
        if a[0] == b[0]:
            raise ValueError(f"token id {a[0]} names two pieces: {a[1]!r} and {b[1]!r}")
    return rows


def load_merges(store, facts: TribleSet, tid: bytes) -> list[tuple[str, str]]:
    """Merges in rank order; the ranks must be ``0..n-1`` without gaps or repeats (``load_merges_strict``, :919-958): a missing
    merge silently changes every encoding that would have used it."""
    rows = []
    for v in facts.values(tid, MERGE):
        e = r_genid(v)
        rows.append((r_u256(facts.one(e, INDEX)), get_text(store, facts.one(e, MERGE_LEFT)), get_text(store, facts.one(e, MERGE_RIGHT))))
    rows.sort(key=lambda r: r[0])
    if [k for k, _, _ in rows] != list(range(len(rows))):
        raise ValueError(f"merge ranks are not 0..{len(rows) - 1} without gaps or repeats")
    return [(l, r) for _, l, r in rows]


def load_added(store, facts: TribleSet, tid: bytes) -> list[dict]:
    """Added tokens in their original order, with every boolean restated (:700-719, :960-1047)."""
    rows = []
    for v in facts.values(tid, ADDED):
        e = r_genid(v)
        tags = _tags(facts, e)
        d = {"id": r_u256(facts.one(e, TOKEN_ID)), "content": get_text(store, facts.one(e, PIECE))}
        d.update({key: f in tags for key, f in _ADDED_FLAGS})
        rows.append((r_u256(facts.one(e, INDEX)), d))
    rows.sort(key=lambda r: r[0])
    return [d for _, d in rows]


def load_tokenizer_json(store, facts: TribleSet, tid: bytes) -> dict:
    """Rebuild the ``tokenizer.json`` dict from facts: the residual document first, then everything the typed graph states."""
    name = get_text(store, facts.one(tid, MODEL_NAME))
    kind = tokenizer_kind(facts, tid)
    tags = _tags(facts, tid)
    try:
        doc = jsonfacts.load_document(store, facts, _residual_name(name), owner=tid)
    except LookupError:
        doc = {"version": "1.0", "truncation": None, "padding": None, "normalizer": None, "pre_tokenizer": None,
               "post_processor": None, "decoder": None, "model": {}}
    model = doc.setdefault("model", {})
    model["type"] = kind
    rows = load_vocab(store, facts, tid)
    if kind == "Unigram":
        if [i for i, _, _ in rows] != list(range(len(rows))):
            raise ValueError("unigram piece ids must be 0..n-1 without gaps")
        model["vocab"] = [[t, s] for _, t, s in rows]
        if "unk_id" not in model:
            unk = [r_u256(facts.one(r_genid(v), TOKEN_ID)) for v in facts.values(tid, VOCAB)
                   if ty.PIECE_UNKNOWN in _tags(facts, r_genid(v))]
            model["unk_id"] = unk[0] if unk else None
    else:
        model["vocab"] = {t: i for i, t, _ in rows}
    merges = load_merges(store, facts, tid)
    if merges or kind == "BPE":
        model["merges"] = [[l, r] for l, r in merges]
    for key, attr in (("unk_token", UNK_TOKEN), ("continuing_subword_prefix", CONTINUING_SUBWORD_PREFIX),
                      ("end_of_word_suffix", END_OF_WORD_SUFFIX)):
        v = facts.maybe(tid, attr)
        if v is not None:
            model[key] = r_shortstring(v)
    v = facts.maybe(tid, MAX_INPUT_CHARS)
    if v is not None:
        model["max_input_chars_per_word"] = r_u256(v)
    v = facts.maybe(tid, BYTE_FALLBACK)
    if v is not None:
        model["byte_fallback"] = r_bool(v)
    for key, f in (("ignore_merges", flag.IGNORE_MERGES), ("fuse_unk", flag.FUSE_UNK)):
        if f in tags:
            model[key] = True
    for key, attr, seq_key in _ROLES:
        v = facts.maybe(tid, attr)
        if v is not None:
            doc[key] = _node_json(store, facts, r_genid(v), seq_key)
    if kind == "Unigram" and flag.ADD_PREFIX_SPACE in tags and doc.get("pre_tokenizer") is None:
        # a graph written from a SentencePiece model states the dummy prefix as a flag, not as a pipeline node
        meta = {"type": "Metaspace", "replacement": "▁", "prepend_scheme": "always", "split": True}
        doc["pre_tokenizer"], doc["decoder"] = dict(meta), dict(meta)
    doc["added_tokens"] = load_added(store, facts, tid)
    return doc


def build_tokenizer(store, facts: TribleSet, tid: bytes | None = None):
    """HF ``tokenizers.Tokenizer`` constructed from facts — no JSON file on disk (src/tokenizer.rs:1049-1290).  A merge table
    with a gap is refused here rather than silently encoding differently."""
    from tokenizers import Tokenizer
    if tid is None:
        tid = select_tokenizer(store, facts)
    return Tokenizer.from_str(json.dumps(load_tokenizer_json(store, facts, tid)))


# --------------------------------------------------------------------------- tiktoken rank tables
def save_tiktoken(store, tb: TribleBuilder, name: str, ranks: dict[bytes, int], pattern: str,
                  special: dict[str, int] | None = None, owner: bytes | None = None, unk_token: str | None = None,
                  not_special: tuple = ()) -> bytes:
    """Byte-level BPE rank table (src/tokenizer.rs:459-526, src/tiktoken.rs): one ``{piece_bytes, token_id = rank}`` entity per
    entry (the rank IS the merge order; the pieces are raw bytes because mid-codepoint fragments are no strings), the reserved
    slots as added tokens, and one pre-tokenizer node that holds the pattern.  Names in ``not_special`` are added tokens the
    encoder still isolates but that do not carry the ``SPECIAL`` flag."""
    ordered = sorted(ranks.items(), key=lambda kv: kv[1])
    if [r for _, r in ordered] != list(range(len(ordered))):
        raise ValueError("tiktoken ranks must be 0..n-1 without gaps")
    pairs = [(META_TAG, v_genid(ty.TIKTOKEN)), (MODEL_NAME, put_text(store, name))]
    for tok, r in ordered:
        pairs.append((VOCAB, v_genid(tb.entity([(PIECE_BYTES, v_handle(store.put(bytes(tok)))), (TOKEN_ID, v_u256(r))]))))
    for order, (s, i) in enumerate(sorted((special or {}).items(), key=lambda kv: kv[1])):
        fl = [] if s in not_special else [(META_TAG, v_genid(flag.SPECIAL))]
        pairs.append((ADDED, v_genid(tb.entity([(PIECE, put_text(store, s)), (TOKEN_ID, v_u256(i)), (INDEX, v_u256(order))] + fl))))
    pairs.append((PRE_TOKENIZER, v_genid(tb.entity([(META_TAG, v_genid(ty.TIKTOKEN_PRE_TOKENIZER)), (PATTERN, put_text(store, pattern))]))))
    if _short_ok(unk_token):
        pairs.append((UNK_TOKEN, v_shortstring(unk_token)))
    tid = tb.entity(pairs)
    _link(tb, tid, owner)
    return tid


def load_tiktoken_ranks(store, facts: TribleSet, tid: bytes) -> dict[bytes, int]:
    """``piece bytes -> rank`` (src/tokenizer.rs:721-741); the ranks must be ``0..n-1``."""
    ranks = {}
    for v in facts.values(tid, VOCAB):
        e = r_genid(v)
        ranks[bytes(store.get(facts.one(e, PIECE_BYTES)))] = r_u256(facts.one(e, TOKEN_ID))
    if sorted(ranks.values()) != list(range(len(ranks))):
        raise ValueError("tiktoken rank table has gaps or repeats")
    return ranks


def load_pre_tokenizer_pattern(store, facts: TribleSet, tid: bytes) -> str:
    """The pattern of the tokenizer's pre-tokenizer node (src/tokenizer.rs:743-765)."""
    node = r_genid(facts.one(tid, PRE_TOKENIZER))
    return get_text(store, facts.one(node, PATTERN))


def load_tiktoken(store, facts: TribleSet, tid: bytes):
    from .tiktoken import TikToken
    if tokenizer_kind(facts, tid) != "tiktoken":
        raise ValueError("not a tiktoken tokenizer")
    special = {d["content"]: d["id"] for d in load_added(store, facts, tid)}
    return TikToken(load_tiktoken_ranks(store, facts, tid), load_pre_tokenizer_pattern(store, facts, tid), special)


# --------------------------------------------------------------------------- SentencePiece unigram
def save_spm_unigram(store, tb: TribleBuilder, name: str, pieces: list[tuple], unk_id: int = 0, owner: bytes | None = None,
                     add_dummy_prefix: bool = True, byte_fallback: bool = False) -> bytes:
    """SentencePiece unigram model as facts (src/tokenizer.rs:1794-1837): the scored piece table IS the model, so every entry
    carries ``piece_score`` and a piece-type tag and the ``.model`` file itself is not stored.  ``pieces`` rows are
    ``(text, score)`` or ``(text, score, type)`` with SentencePiece's type numbers (1 normal, 2 unknown, 3 control,
    4 user-defined, 5 unused, 6 byte); without a type, row ``unk_id`` is the unknown piece and the rest are normal."""
    pairs = [(META_TAG, v_genid(ty.UNIGRAM)), (MODEL_NAME, put_text(store, name)), (BYTE_FALLBACK, v_bool(byte_fallback))]
    if add_dummy_prefix:
        pairs.append((META_TAG, v_genid(flag.ADD_PREFIX_SPACE)))
    for i, row in enumerate(pieces):
        text, score = row[0], row[1]
        typ = row[2] if len(row) > 2 else 2 if i == unk_id else 1
        if isinstance(text, bytes):
            text = text.decode("utf-8")
        pairs.append((VOCAB, v_genid(tb.entity([(META_TAG, v_genid(_SPM_TAGS[typ])), (PIECE, put_text(store, text)),
                                                (TOKEN_ID, v_u256(i)), (PIECE_SCORE, v_f64(float(score)))]))))
    tid = tb.entity(pairs)
    _link(tb, tid, owner)
    return tid


def load_spm_pieces(store, facts: TribleSet, tid: bytes) -> list[tuple[bytes, float, int]]:
    """``(bytes, score, type)`` rows in id order (src/tokenizer.rs:1839-1857)."""
    rows = []
    for v in facts.values(tid, VOCAB):
        e = r_genid(v)
        typ = [_SPM_OF_TAG[t] for t in _tags(facts, e) if t in _SPM_OF_TAG]
        if len(typ) != 1:
            raise ValueError(f"unigram entry {e.hex()} carries {len(typ)} piece-type tags, expected 1")
        rows.append((r_u256(facts.one(e, TOKEN_ID)), get_text(store, facts.one(e, PIECE)).encode("utf-8"),
                     r_f64(facts.one(e, PIECE_SCORE)), typ[0]))
    rows.sort(key=lambda r: r[0])
    return [(b, s, t) for _, b, s, t in rows]


def has_add_prefix_space(facts: TribleSet, tid: bytes) -> bool:
    """Whether the tokenizer node carries the ``ADD_PREFIX_SPACE`` flag (src/tokenizer.rs:1859-1861)."""
    return flag.ADD_PREFIX_SPACE in _tags(facts, tid)
