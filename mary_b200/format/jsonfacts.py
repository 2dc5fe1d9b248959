"""JSON documents (``config.json``, ``hf_quant_config.json``, chat templates) stored as facts.

Reference: src/jsonfacts.rs.  One entity per JSON node; the node id folds in its position (path from
the document root) so equal scalars at different places stay distinct (:24-38,120-198); ints and floats
are kept apart so a round trip is exact (:40-46); ``save_document`` / ``load_document`` (:200-256).
Nine attributes: key, string, int, float, bool, parent, position, type, document root (+ name label)."""
from __future__ import annotations

import json

from ..pile.trible import (TribleBuilder, TribleSet, derived_id, r_bool, r_f64, r_genid, r_i256, r_shortstring,
                           v_bool, v_f64, v_genid, v_i256, v_shortstring, v_u256, r_u256)
from . import schema as S
from .model import get_text, put_text

_TYPES = ("object", "array", "string", "int", "float", "bool", "null")


def _node_id(doc_salt: bytes, path: tuple) -> bytes:
    return derived_id(b"jsonnode", doc_salt, json.dumps(path).encode())


def save_document(store, tb: TribleBuilder, name: str, doc, owner: bytes | None = None) -> bytes:
    """Store ``doc`` (a parsed JSON value) under the document name; returns the root node id.
    ``owner`` (e.g. a model root) salts the ids so two models can hold different ``config.json``."""
    salt = (owner or b"") + name.encode()

    def put(value, path, parent, key, pos):
        nid = _node_id(salt, path)
        pairs = []
        if parent is not None:
            pairs.append((S.JSON_PARENT, v_genid(parent)))
            pairs.append((S.JSON_POS, v_u256(pos)))
        if key is not None:
            pairs.append((S.JSON_KEY, put_text(store, key)))
        if isinstance(value, bool):
            pairs += [(S.JSON_TYPE, v_shortstring("bool")), (S.JSON_BOOL, v_bool(value))]
        elif isinstance(value, int):
            pairs += [(S.JSON_TYPE, v_shortstring("int")), (S.JSON_INT, v_i256(value))]
        elif isinstance(value, float):
            pairs += [(S.JSON_TYPE, v_shortstring("float")), (S.JSON_FLOAT, v_f64(value))]
        elif isinstance(value, str):
            pairs += [(S.JSON_TYPE, v_shortstring("string")), (S.JSON_STRING, put_text(store, value))]
        elif value is None:
            pairs += [(S.JSON_TYPE, v_shortstring("null"))]
        elif isinstance(value, dict):
            pairs += [(S.JSON_TYPE, v_shortstring("object"))]
            for i, (k, v) in enumerate(value.items()):
                put(v, path + (str(k),), nid, str(k), i)
        elif isinstance(value, (list, tuple)):
            pairs += [(S.JSON_TYPE, v_shortstring("array"))]
            for i, v in enumerate(value):
                put(v, path + (i,), nid, None, i)
        else:
            raise TypeError(f"not a JSON value: {type(value)}")
        tb.entity(pairs, id=nid)
        return nid

    root = put(doc, (), None, None, 0)
    labels = [(S.DOCUMENT_ROOT, v_genid(root)), (S.DOCUMENT_NAME, put_text(store, name))]
    if owner is not None:
        labels.append((S.OWNER, v_genid(owner)))
    tb.entity(labels, id=derived_id(b"jsondoc", salt))
    return root


def list_documents(store, facts: TribleSet) -> list[tuple[str, bytes, bytes | None]]:
    out = []
    for e, v in facts.with_attr(S.DOCUMENT_ROOT):
        name = get_text(store, facts.one(e, S.DOCUMENT_NAME))
        owner = facts.maybe(e, S.OWNER)
        out.append((name, r_genid(v), r_genid(owner) if owner else None))
    return out


def load_document(store, facts: TribleSet, name: str, owner: bytes | None = None):
    """Exactly one document of that name (and owner, when given) must exist."""
    hits = [(n, r, o) for n, r, o in list_documents(store, facts) if n == name and (owner is None or o == owner)]
    if len(hits) != 1:
        raise LookupError(f"document {name!r}: found {len(hits)}, expected exactly 1")
    root = hits[0][1]
    children: dict[bytes, list[tuple[int, bytes]]] = {}
    for e, v in facts.with_attr(S.JSON_PARENT):
        children.setdefault(r_genid(v), []).append((r_u256(facts.one(e, S.JSON_POS)), e))

    def build(nid):
        t = r_shortstring(facts.one(nid, S.JSON_TYPE))
        if t == "bool":
            return r_bool(facts.one(nid, S.JSON_BOOL))
        if t == "int":
            return r_i256(facts.one(nid, S.JSON_INT))
        if t == "float":
            return r_f64(facts.one(nid, S.JSON_FLOAT))
        if t == "string":
            return get_text(store, facts.one(nid, S.JSON_STRING))
        if t == "null":
            return None
        kids = sorted(children.get(nid, []))
        if t == "array":
            return [build(k) for _, k in kids]
        return {get_text(store, facts.one(k, S.JSON_KEY)): build(k) for _, k in kids}

    return build(root)
