"""Exact-cardinality model selection and the strict ``name -> Leaf`` index.

Reference: src/selection.rs.  ``ModelSelector::{Only, Root, Name, Source{source, quantization}}`` (:19-32);
zero or many matches is an error, never "first" (:173-257); tensor names are unique per root (:259-292);
shards are sibling roots merged by tensor name with a disjointness check (:319-345)."""
from __future__ import annotations

from dataclasses import dataclass

from ..pile.trible import TribleSet, r_genid, r_shortstring
from . import schema as S
from .leaf import Leaf, resolve
from .model import get_text, index_keymap, load_module_leaf


class SelectionError(LookupError):
    pass


@dataclass(frozen=True)
class ModelSelector:
    kind: str                      # "only" | "root" | "name" | "source"
    root: bytes | None = None
    name: str | None = None
    source: str | None = None
    quantization: str | None = None

    @staticmethod
    def only():
        return ModelSelector("only")

    @staticmethod
    def by_root(root: bytes):
        return ModelSelector("root", root=root)

    @staticmethod
    def by_name(name: str):
        return ModelSelector("name", name=name)

    @staticmethod
    def by_source(source: str, quantization: str | None = None):
        return ModelSelector("source", source=source, quantization=quantization)


def model_roots(facts: TribleSet) -> list[bytes]:
    return sorted({e for e, _ in facts.with_attr(S.MODEL_ROOT)})


def select_model_roots(store, facts: TribleSet, sel: ModelSelector) -> list[bytes]:
    """All roots that match (a sharded model matches with several roots under ``name``/``source``)."""
    roots = model_roots(facts)
    if sel.kind == "only":
        return roots
    if sel.kind == "root":
        return [r for r in roots if r == sel.root]
    out = []
    for r in roots:
        if sel.kind == "name":
            v = facts.maybe(r, S.MODEL_NAME)
            if v is not None and get_text(store, v) == sel.name:
                out.append(r)
        elif sel.kind == "source":
            v = facts.maybe(r, S.SOURCE)
            if v is None or get_text(store, v) != sel.source:
                continue
            q = facts.maybe(r, S.QUANTIZATION)
            qs = r_shortstring(q) if q is not None else None
            if qs == sel.quantization:
                out.append(r)
    return out


def select_model_root(store, facts: TribleSet, sel: ModelSelector) -> bytes:
    roots = select_model_roots(store, facts, sel)
    if len(roots) != 1:
        raise SelectionError(f"selector {sel} matched {len(roots)} model roots, expected exactly 1")
    return roots[0]


class SelectedModelIndex:
    """``name -> module`` over one root or over disjoint shard roots; leaves are resolved lazily."""

    def __init__(self, store, facts: TribleSet, roots: list[bytes]):
        if not roots:
            raise SelectionError("no model root selected")
        self.store, self.facts, self.roots = store, facts, list(roots)
        self.keymap: dict[str, bytes] = {}
        for r in roots:
            km = index_keymap(store, facts, r)
            clash = self.keymap.keys() & km.keys()
            if clash:
                raise SelectionError(f"shard roots overlap on {len(clash)} tensor names, e.g. {sorted(clash)[0]!r}")
            self.keymap.update(km)

    @staticmethod
    def from_snapshot(store, facts: TribleSet, sel: ModelSelector = ModelSelector.only(), shards: bool = False):
        roots = select_model_roots(store, facts, sel)
        if not shards and len(roots) != 1:
            raise SelectionError(f"selector {sel} matched {len(roots)} model roots, expected exactly 1")
        return SelectedModelIndex(store, facts, roots)

    def names(self) -> list[str]:
        return sorted(self.keymap)

    def has(self, name: str) -> bool:
        return name in self.keymap

    def leaf(self, name: str, role: bytes = S.WEIGHT) -> Leaf:
        try:
            m = self.keymap[name]
        except KeyError:
            raise SelectionError(f"tensor {name!r} is not in the selected model") from None
        return load_module_leaf(self.store, self.facts, m, role)

    def module(self, name: str) -> bytes:
        return self.keymap[name]

    def experts_in_layers(self, lo: int, hi: int) -> dict[tuple[int, int], list[str]]:
        """Placement is a QUERY over ``layer`` / ``expert_index`` facts, not a file layout
        (src/models/inkling/pile.rs:514-549).  Returns ``(layer, expert) -> tensor names``."""
        from ..pile.trible import r_i256
        inv = {m: n for n, m in self.keymap.items()}
        out: dict[tuple[int, int], list[str]] = {}
        for m, v in self.facts.with_attr(S.LAYER):
            if m not in inv:
                continue
            layer = r_i256(v)
            if not (lo <= layer < hi):
                continue
            ex = self.facts.maybe(m, S.EXPERT_INDEX)
            if ex is None:
                continue
            out.setdefault((layer, r_i256(ex)), []).append(inv[m])
        for k in out:
            out[k].sort()
        return out
