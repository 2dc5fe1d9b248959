"""Pile maintenance that rewrites representations without touching meaning (src/bin/pile_leaf_migrate.rs,
src/bin/pile_loader_equiv.rs, and the separate ``model-migration`` crate).

* ``migrate_leaves``: pile to pile, into a NEW file; the source is only read.  Substitution, not reconstruction: every fact is
  carried over verbatim except the ``data`` / ``data_f16`` / ``shape`` facts of the leaves that are converted; each converted leaf
  KEEPS ITS OWN ENTITY ID and gains one typed-tensor fact; every blob a carried fact refers to is copied, the superseded data and
  shape blobs are not.  Leaves in encodings this tool has no typed form for (q4 / q8) pass through whole, shape included.
* ``branch_to_collection``: facts that live on a legacy named branch are published once into the model-graph collection.
* ``loader_equiv``: prove the converted pile equal through the PUBLIC loader (``WeightLoader.load_host_f32`` for every tensor name)
  and assert that the converted side really reads typed leaves — a check that passes because both sides fell back to the legacy
  path would prove nothing."""
from __future__ import annotations

import numpy as np

from ..nn.weight_loader import WeightLoader
from ..pile import Pile
from ..pile.trible import TribleBuilder, TribleSet, v_handle
from . import schema as S
from .leaf import Elem, LeafError, leaf_attr, read_blob, tensor_blob
from .persist import LEGACY_BRANCHES, publish_fragment, read_model_pile
from .selection import ModelSelector, SelectedModelIndex

_LEGACY = (S.DATA, S.DATA_F16)


def migrate_leaves(src: Pile, dst: Pile, key, message: str = "typed leaves") -> dict:
    facts = read_model_pile(src)
    by_entity: dict[bytes, list] = {}
    for e, a, v in facts:
        by_entity.setdefault(e, []).append((a, v))
    tb = TribleBuilder()
    stats = {"converted": 0, "passed_through": 0, "blobs_copied": 0, "blobs_dropped": 0}
    dropped: set[bytes] = set()
    for e, pairs in by_entity.items():
        attrs = {a for a, _ in pairs}
        legacy = [(a, v) for a, v in pairs if a in _LEGACY]
        convertible = len(legacy) == 1 and S.SHAPE in attrs and not ({S.DATA_Q4, S.DATA_Q8} & attrs)
        if not convertible:
            for a, v in pairs:
                tb.add(e, a, v)
            if legacy:
                stats["passed_through"] += 1
            continue
        a_data, h_data = legacy[0]
        h_shape = next(v for a, v in pairs if a == S.SHAPE)
        dims = tuple(int(d) for d in np.frombuffer(src.get(h_shape), dtype=np.uint64))
        elem = Elem.F16 if a_data == S.DATA_F16 else Elem.F32
        payload = src.get(h_data)
        blob = tensor_blob(elem, dims, payload)
        back = read_blob(blob)
        if back.dims != dims or bytes(back.payload) != bytes(payload):          # compared as it encodes, like the original tool
            raise LeafError(f"leaf {e.hex()}: typed blob does not reproduce the legacy payload")
        tb.add(e, leaf_attr(elem, len(dims)), v_handle(dst.put(blob)))
        for a, v in pairs:
            if a not in _LEGACY and a != S.SHAPE:
                tb.add(e, a, v)
        dropped.update((bytes(h_data), bytes(h_shape)))
        stats["converted"] += 1
    out = tb.build()
    for _, _, v in out:                                                          # blobs that carried facts refer to
        h = bytes(v)
        if h in dropped:
            continue
        try:
            blob = src.get(h)
        except Exception:                                                        # a value that is not a handle
            continue
        dst.put(blob)
        stats["blobs_copied"] += 1
    stats["blobs_dropped"] = len(dropped)
    publish_fragment(dst, key, out, message)
    return stats


def branch_to_collection(pile: Pile, key) -> int:
    """Publish the facts of the first legacy branch that has any into the model-graph collection; returns the number of facts
    (0 when the collection already serves the pile)."""
    from ..pile.repo import Repository
    repo = Repository(pile)
    names = repo.branches()
    for b in LEGACY_BRANCHES:
        for bid in names.get(b, []):
            head = repo.head(bid)
            if head:
                facts = repo.checkout(bid)
                publish_fragment(pile, key, facts, f"from branch {b}"[:32])
                return len(facts)
    return 0


def loader_equiv(original: Pile, converted: Pile, selector: ModelSelector = ModelSelector.only()) -> dict:
    fa, fb = read_model_pile(original), read_model_pile(converted)
    la = WeightLoader.from_pile(SelectedModelIndex.from_snapshot(original, fa, selector))
    lb = WeightLoader.from_pile(SelectedModelIndex.from_snapshot(converted, fb, selector))
    if sorted(la.names()) != sorted(lb.names()):
        raise AssertionError(f"tensor names differ: {sorted(set(la.names()) ^ set(lb.names()))[:5]} ...")
    typed = 0
    for n in la.names():
        a, b = la.load_host_f32(n), lb.load_host_f32(n)
        if a.shape != b.shape or not np.array_equal(a, b):
            raise AssertionError(f"{n}: loaders disagree")
        typed += int(_reads_typed(converted, fb, lb, n))
    if typed != len(la.names()):
        raise AssertionError(f"only {typed} of {len(la.names())} tensors of the converted pile are typed leaves")
    return {"tensors": len(la.names()), "typed": typed}


def _reads_typed(pile, facts: TribleSet, loader: WeightLoader, name: str) -> bool:
    from .model import index_keymap
    from .selection import model_roots
    for r in model_roots(facts):
        km = index_keymap(pile, facts, r)
        if name in km:
            leaf_entity = facts.one(km[name], S.WEIGHT)
            from ..pile.trible import r_genid
            ent = r_genid(leaf_entity)
            return not any(a in _LEGACY for a, _ in facts.of_entity(ent))
    return False
