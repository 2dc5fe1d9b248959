"""The three primitives of the model graph: tensor leaf, module entity, model root.

Reference: src/format.rs:141-326 (put/load helpers), src/ingest.rs:89-262 (import, roots, keymaps).

* module = ``{kind, safetensor_path, weight[, bias][, index]}`` where ``weight``/``bias`` are role edges to
  leaf entities and ``kind`` follows the rank (``vector/matrix/conv/tensor``, src/ingest.rs:142-147);
* model root id = hash of its ``member`` set only; ``model_name``/``source``/``quantization`` are labels
  attached afterwards so they do not change the id (src/ingest.rs:178-205).
"""
from __future__ import annotations

import numpy as np

from ..pile.trible import (TribleBuilder, TribleSet, content_id, r_genid, r_shortstring, v_genid, v_handle,
                           v_shortstring, v_u256)
from . import schema as S
from .leaf import Elem, Leaf, put_array, put_leaf, resolve


def kind_of_rank(rank: int) -> str:
    return {1: "vector", 2: "matrix", 3: "conv"}.get(rank, "tensor")


def put_text(store, text: str) -> bytes:
    return v_handle(store.put(text.encode("utf-8")))


def get_text(store, value: bytes) -> str:
    return bytes(store.get(value)).decode("utf-8")


def put_module(store, tb: TribleBuilder, name: str, weight_leaf: bytes, rank: int,
               bias_leaf: bytes | None = None, index: int | None = None, extra=()) -> bytes:
    pairs = [(S.KIND, v_shortstring(kind_of_rank(rank))), (S.SAFETENSOR_PATH, put_text(store, name)),
             (S.WEIGHT, v_genid(weight_leaf))]
    if bias_leaf is not None:
        pairs.append((S.BIAS, v_genid(bias_leaf)))
    if index is not None:
        pairs.append((S.INDEX, v_u256(index)))
    pairs.extend(extra)
    return tb.entity(pairs)


def put_tensor(store, tb: TribleBuilder, name: str, arr: np.ndarray, elem: Elem | None = None, extra=()) -> bytes:
    """Leaf + module for one named tensor; returns the module entity id."""
    a = np.asarray(arr)
    leaf = put_array(store, tb, a, elem)
    return put_module(store, tb, name, leaf, a.ndim, extra=extra)


def put_fp4_tensor(store, tb: TribleBuilder, name: str, codes: np.ndarray, scales: np.ndarray,
                   scale2: float | None, layer: int | None = None, expert: int | None = None) -> bytes:
    """Block-scaled expert matrix as ONE blob ``[codes][scales][scale2]`` with logical dims
    (src/models/inkling/pile.rs:343-399) plus ``layer`` / ``expert_index`` placement facts (:408-466)."""
    from ..pile.trible import v_i256
    rows, k = codes.shape[0], codes.shape[1] * 2
    if scale2 is not None:
        payload = codes.tobytes() + scales.tobytes() + np.float32(scale2).tobytes()
        elem = Elem.NVFP4
    else:
        payload = codes.tobytes() + scales.tobytes()
        elem = Elem.MXFP4
    leaf = put_leaf(store, tb, elem, (rows, k), payload)
    extra = []
    if layer is not None:
        extra.append((S.LAYER, v_i256(layer)))
    if expert is not None:
        extra.append((S.EXPERT_INDEX, v_i256(expert)))
    return put_module(store, tb, name, leaf, 2, extra=extra)


def put_linear(store, tb: TribleBuilder, name: str, weight: np.ndarray, bias: np.ndarray | None = None) -> bytes:
    wl = put_array(store, tb, weight)
    bl = put_array(store, tb, bias) if bias is not None else None
    return put_module(store, tb, name, wl, np.asarray(weight).ndim, bias_leaf=bl)


def build_model_root(store, tb: TribleBuilder, members: list[bytes], name: str | None = None,
                     source: str | None = None, quantization: str | None = None) -> bytes:
    """Root id = hash(member*) only; labels are attached to that id afterwards."""
    if not members:
        raise ValueError("a model root needs at least one member")
    pairs = [(S.MEMBER, v_genid(m)) for m in sorted(set(members))]
    root = content_id(pairs)
    tb.entity(pairs, id=root)
    labels = [(S.MODEL_ROOT, v_genid(root))]
    if name is not None:
        labels.append((S.MODEL_NAME, put_text(store, name)))
    if source is not None:
        labels.append((S.SOURCE, put_text(store, source)))
    if quantization is not None:
        labels.append((S.QUANTIZATION, v_shortstring(quantization)))
    tb.entity(labels, id=root)
    return root


def root_members(facts: TribleSet, root: bytes) -> list[bytes]:
    return [r_genid(v) for v in facts.values(root, S.MEMBER)]


def module_name(store, facts: TribleSet, module: bytes) -> str:
    return get_text(store, facts.one(module, S.SAFETENSOR_PATH))


def load_module_leaf(store, facts: TribleSet, module: bytes, role: bytes = S.WEIGHT) -> Leaf:
    return resolve(store, facts, r_genid(facts.one(module, role)))


def index_keymap(store, facts: TribleSet, root: bytes) -> dict[str, bytes]:
    """tensor name -> module entity for one root; duplicate names are an error (src/selection.rs:259-292)."""
    out: dict[str, bytes] = {}
    for m in root_members(facts, root):
        n = module_name(store, facts, m)
        if n in out and out[n] != m:
            raise LookupError(f"tensor name {n!r} occurs twice under root {root.hex()}")
        out[n] = m
    return out
