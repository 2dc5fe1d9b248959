"""JSON documents (``config.json``, ``hf_quant_config.json``, chat templates) stored as facts.

The node model is the reference's (src/jsonfacts.rs): one content-derived entity per JSON node whose attribute set holds

* its type tag for containers and ``null`` (``metadata::tag`` = ``JSON_OBJECT`` / ``JSON_ARRAY`` / ``JSON_NULL``; scalars need
  none, their value attribute is the discriminant, :53-70),
* its POSITION — ``json_key`` for an object member, ``index`` for an array element — folded into the identity at construction,
  so ``[1, 1]`` is two nodes and equal subtrees under the same key still collapse (:24-38, :166-190),
* one of ``json_string`` / ``json_int`` / ``json_float`` / ``json_bool``; integers and floats stay apart so ``4096`` does not
  come back as ``4096.0`` (:40-46, :131-147), an integer beyond 64 bits is refused (:137-141),
* ``member`` edges to its children.

A named document is a node tagged ``JSON_DOCUMENT`` with ``metadata::name`` and ``document_root`` (:200-216); a model root may be
attached as owner label so two models in one pile can hold different ``config.json`` files."""
from __future__ import annotations

from ..pile.trible import (TribleBuilder, TribleSet, r_bool, r_f64, r_genid, r_i256, r_u256, v_bool, v_f64, v_genid, v_i256, v_u256)
from . import schema as S
from .model import get_text, put_text


def save_json(store, tb: TribleBuilder, value, _pos=None) -> bytes:
    """Ingest a parsed JSON value; returns the root node's id (src/jsonfacts.rs:113-196)."""
    pairs = []
    if _pos is not None:
        kind, p = _pos
        pairs.append((S.JSON_KEY, put_text(store, p)) if kind == "key" else (S.INDEX, v_u256(p)))
    if value is None:
        pairs.append((S.META_TAG, v_genid(S.JSON_NULL)))
    elif isinstance(value, bool):
        pairs.append((S.JSON_BOOL, v_bool(value)))
    elif isinstance(value, int):
        if not -(1 << 63) <= value < (1 << 63):
            raise ValueError(f"integer {value} does not fit in i64")
        pairs.append((S.JSON_INT, v_i256(value)))
    elif isinstance(value, float):
        pairs.append((S.JSON_FLOAT, v_f64(value)))
    elif isinstance(value, str):
        pairs.append((S.JSON_STRING, put_text(store, value)))
    elif isinstance(value, dict):
        pairs.append((S.META_TAG, v_genid(S.JSON_OBJECT)))
        for k, v in value.items():
            pairs.append((S.MEMBER, v_genid(save_json(store, tb, v, ("key", str(k))))))
    elif isinstance(value, (list, tuple)):
        pairs.append((S.META_TAG, v_genid(S.JSON_ARRAY)))
        for i, v in enumerate(value):
            pairs.append((S.MEMBER, v_genid(save_json(store, tb, v, ("index", i)))))
    else:
        raise TypeError(f"not a JSON value: {type(value)}")
    return tb.entity(pairs)


def save_document(store, tb: TribleBuilder, name: str, doc, owner: bytes | None = None) -> bytes:
    """Store ``doc`` (a parsed JSON value) under the document name; returns the root node id."""
    root = save_json(store, tb, doc)
    pairs = [(S.META_TAG, v_genid(S.JSON_DOCUMENT)), (S.META_NAME, put_text(store, name)), (S.DOCUMENT_ROOT, v_genid(root))]
    if owner is not None:
        pairs.append((S.OWNER, v_genid(owner)))
    tb.entity(pairs)
    return root


def list_documents(store, facts: TribleSet) -> list[tuple[str, bytes, bytes | None]]:
    out = []
    for e in facts.entities_where(S.META_TAG, v_genid(S.JSON_DOCUMENT)):
        owner = facts.maybe(e, S.OWNER)
        out.append((get_text(store, facts.one(e, S.META_NAME)), r_genid(facts.one(e, S.DOCUMENT_ROOT)), r_genid(owner) if owner else None))
    return sorted(out, key=lambda t: (t[0], t[1]))


def load_json(store, facts: TribleSet, node: bytes):
    """Rebuild the JSON value under ``node`` (src/jsonfacts.rs:258-340): members of an object keep their stored order by key
    lookup, array elements are ordered by ``index``.  Objects come back with their keys sorted — the canonical form in which
    the reference compares a document with its round trip (:40-46)."""
    tags = {r_genid(v) for v in facts.values(node, S.META_TAG)}
    if S.JSON_NULL in tags:
        return None
    if S.JSON_OBJECT in tags:
        kids = sorted((get_text(store, facts.one(r_genid(m), S.JSON_KEY)), r_genid(m)) for m in facts.values(node, S.MEMBER))
        return {k: load_json(store, facts, c) for k, c in kids}      # canonical: keys in sorted order, as the reference's object map
    if S.JSON_ARRAY in tags:
        kids = sorted((r_u256(facts.one(r_genid(m), S.INDEX)), r_genid(m)) for m in facts.values(node, S.MEMBER))
        return [load_json(store, facts, c) for _, c in kids]
    for attr, rd in ((S.JSON_BOOL, r_bool), (S.JSON_INT, r_i256), (S.JSON_FLOAT, r_f64)):
        v = facts.maybe(node, attr)
        if v is not None:
            return rd(v)
    v = facts.maybe(node, S.JSON_STRING)
    if v is not None:
        return get_text(store, v)
    raise LookupError("JSON node without a value or a type tag")


def load_document(store, facts: TribleSet, name: str, owner: bytes | None = None):
    """Exactly one document of that name (and owner, when given) must exist."""
    hits = [(n, r, o) for n, r, o in list_documents(store, facts) if n == name and (owner is None or o == owner)]
    if len(hits) != 1:
        have = sorted({n for n, _, _ in list_documents(store, facts)})
        raise LookupError(f"document {name!r}: found {len(hits)}, expected exactly 1; this pile has {have}")
    return load_json(store, facts, hits[0][1])
