"""Quantised tensor leaves: ``data_q4`` / ``data_q8`` + ``q_scales`` + ``shape`` + ``format_marker`` (src/format.rs:63-87), and sibling
model roots that hold a model's matrices in that form (the reference's derived q4 / q8 piles).

The code blob is the packed quantised payload in block order (Q4_0: 16 nibble bytes per 32 elements, element ``j`` of a block in the low
nibble of byte ``j``, element ``j + 16`` in the high nibble; Q8_0: 32 int8 per block), the scale blob one f16 per block, ``shape`` the
logical ``[rows, cols]`` as u64.  ``format_marker`` versions the layout: a reader refuses a marker it does not know instead of
decoding bytes it would misread.  Vectors and tensors whose last dim is not a multiple of 32 stay typed f32 leaves."""
from __future__ import annotations

import numpy as np

from ..nn.q4 import dequantize_q4, dequantize_q8, quantize_q4, quantize_q8
from ..pile.trible import TribleBuilder, TribleSet, r_genid, v_handle, v_shortstring, r_shortstring
from . import schema as S
from .leaf import Elem, LeafError
from .model import build_model_root, get_text, load_module_leaf, module_name, put_module, put_tensor, root_members

MARKER = {"q4": "q4_0.v1", "q8": "q8_0.v1"}


def put_leaf_q(store, tb: TribleBuilder, weight: np.ndarray, kind: str = "q4", id: bytes | None = None) -> bytes:
    w = np.asarray(weight, dtype=np.float32)
    if w.ndim != 2 or w.shape[1] % 32:
        raise LeafError(f"quantised leaves are matrices with a multiple of 32 columns, got {w.shape}")
    packed = (quantize_q4 if kind == "q4" else quantize_q8)(w)                 # [rows, blocks, 2 + payload]
    scales = np.ascontiguousarray(packed[..., :2]).view(np.float16)[..., 0]
    codes = np.ascontiguousarray(packed[..., 2:])
    pairs = [(S.DATA_Q4 if kind == "q4" else S.DATA_Q8, v_handle(store.put(codes.tobytes()))),
             (S.Q_SCALES, v_handle(store.put(scales.tobytes()))),
             (S.SHAPE, v_handle(store.put(np.asarray(w.shape, dtype=np.uint64).tobytes()))),
             (S.FORMAT_MARKER, v_shortstring(MARKER[kind]))]
    return tb.entity(pairs, id=id)


def is_q_leaf(facts: TribleSet, entity: bytes) -> bool:
    return any(a in (S.DATA_Q4, S.DATA_Q8) for a, _ in facts.of_entity(entity))


def load_leaf_q(store, facts: TribleSet, entity: bytes):
    """``(kind, packed [rows, blocks, 2 + payload] uint8, (rows, cols))`` — the layout ``nn.q4.QLinear`` consumes."""
    kinds = [(a, v) for a, v in facts.of_entity(entity) if a in (S.DATA_Q4, S.DATA_Q8)]
    if len(kinds) != 1:
        raise LeafError(f"leaf {entity.hex()} has {len(kinds)} quantised payloads, expected exactly 1")
    kind = "q4" if kinds[0][0] == S.DATA_Q4 else "q8"
    marker = r_shortstring(facts.one(entity, S.FORMAT_MARKER))
    if marker != MARKER[kind]:
        raise LeafError(f"leaf {entity.hex()}: format marker {marker!r} is not the {MARKER[kind]!r} this reader decodes")
    rows, cols = (int(d) for d in np.frombuffer(store.get(facts.one(entity, S.SHAPE)), dtype=np.uint64))
    nb, width = cols // 32, (16 if kind == "q4" else 32)
    codes = np.frombuffer(store.get(kinds[0][1]), dtype=np.uint8)
    scales = np.frombuffer(store.get(facts.one(entity, S.Q_SCALES)), dtype=np.float16)
    if codes.size != rows * nb * width or scales.size != rows * nb:
        raise LeafError(f"leaf {entity.hex()}: payload sizes do not match shape {(rows, cols)}")
    packed = np.empty((rows, nb, 2 + width), dtype=np.uint8)
    packed[..., :2] = scales.reshape(rows, nb, 1).view(np.uint8)
    packed[..., 2:] = codes.reshape(rows, nb, width)
    return kind, packed, (rows, cols)


def dequantize_leaf_q(store, facts: TribleSet, entity: bytes) -> np.ndarray:
    kind, packed, _ = load_leaf_q(store, facts, entity)
    return (dequantize_q4 if kind == "q4" else dequantize_q8)(packed)


def derive_q_root(pile, key, facts: TribleSet, root: bytes, kind: str = "q4") -> bytes:
    """Sibling root with every eligible matrix quantised (the others kept as f32 leaves), published as one commit."""
    from .persist import publish_fragment
    tb = TribleBuilder()
    members = []
    for m in root_members(facts, root):
        a = load_module_leaf(pile, facts, m).to_f32()
        n = module_name(pile, facts, m)
        if a.ndim == 2 and a.shape[1] % 32 == 0:
            members.append(put_module(pile, tb, n, put_leaf_q(pile, tb, a, kind), 2))
        else:
            members.append(put_tensor(pile, tb, n, a, Elem.F32))
    name, src = facts.maybe(root, S.MODEL_NAME), facts.maybe(root, S.SOURCE)
    new = build_model_root(pile, tb, members, name=get_text(pile, name) if name else None, source=get_text(pile, src) if src else None,
                           quantization=kind)
    publish_fragment(pile, key, tb.build(), f"derive {kind}")
    return new


def module_weight_q(store, facts: TribleSet, module: bytes):
    """The quantised weight of a module entity, or ``None`` when its weight is an ordinary leaf."""
    ent = r_genid(facts.one(module, S.WEIGHT))
    return load_leaf_q(store, facts, ent) if is_q_leaf(facts, ent) else None
