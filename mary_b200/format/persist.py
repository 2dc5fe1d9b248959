"""Pile I/O entry points: import a checkpoint, read a model back, derive half-precision roots.

Reference: src/persist.rs — import (:115-235), f16 derivation (:246-295), filtered component import
(:310-417), branch checkout (:1777-1823), collection-preferring reader (:1733-1769), tokenizer ingest/load
(:1852-2176), JSON sidecar ingest (:2236-2334)."""
from __future__ import annotations

import json
from pathlib import Path

import numpy as np

from ..pile import Collection, MODEL_GRAPH, Pile, Repository, TribleBuilder, TribleSet, signing_key_file
from ..pile.trible import r_genid
from . import jsonfacts, schema as S
from .ingest import f32_to_bf16_bits, ingest_members
from .leaf import Elem
from .model import build_model_root, get_text, module_name, put_tensor, root_members, load_module_leaf
from .selection import ModelSelector, SelectedModelIndex, select_model_root
from .tokenizer import save_tokenizer_json

LEGACY_BRANCHES = ("mary", "main", "inkling")


def ingest_json_documents(store, tb: TribleBuilder, directory, owner: bytes | None,
                          names=("config.json", "hf_quant_config.json", "generation_config.json",
                                 "chat_template.json", "tokenizer_config.json")) -> list[str]:
    done = []
    for n in names:
        p = Path(directory) / n
        if p.is_file():
            jsonfacts.save_document(store, tb, n, json.loads(p.read_text()), owner=owner)
            done.append(n)
    return done


def ingest_hf_tokenizer(store, tb: TribleBuilder, directory, name: str, owner: bytes | None) -> bytes | None:
    p = Path(directory) / "tokenizer.json"
    if not p.is_file():
        return None
    return save_tokenizer_json(store, tb, name, p.read_text(), owner)


def ingest_model_fragment(pile, path, name: str | None = None, source: str | None = None, dtype: str = "f32",
                          name_filter=None) -> tuple[TribleSet, bytes]:
    """checkpoint dir/file -> fact fragment + root id.  The pile is refreshed first and a torn tail refuses
    the import (src/persist.rs:143-151)."""
    pile.refresh()
    tb = TribleBuilder()
    members = ingest_members(pile, tb, path, dtype, name_filter)
    if not members:
        raise ValueError(f"{path}: nothing to import")
    root = build_model_root(pile, tb, members, name=name, source=source or str(path),
                            quantization=None if dtype == "f32" else dtype)
    d = Path(path) if Path(path).is_dir() else Path(path).parent
    ingest_json_documents(pile, tb, d, root)
    ingest_hf_tokenizer(pile, tb, d, name or "tokenizer", root)
    return tb.build(), root


def import_model_to_collection(pile, key, path, name: str | None = None, source: str | None = None,
                               dtype: str = "f32", name_filter=None) -> bytes:
    """Import and publish into the ``mary-model-graph`` collection as one signed commit.  Re-importing the
    same bytes is idempotent: blobs dedupe and the fragment adds no new facts (src/bin/mary.rs:22-30)."""
    frag, root = ingest_model_fragment(pile, path, name, source, dtype, name_filter)
    Collection(Repository(pile, key), MODEL_GRAPH).publish(frag, f"import {name or ''}"[:32])
    pile.flush()
    return root


def publish_fragment(pile, key, fragment: TribleSet, message: str = "fragment") -> bytes:
    c = Collection(Repository(pile, key), MODEL_GRAPH).publish(fragment, message)
    pile.flush()
    return c


def read_model_pile(pile, branch: str | None = None) -> TribleSet:
    """Facts of a pile: an explicit branch, else the model-graph collection, else a legacy branch
    (collection-preferring reader, src/persist.rs:1733-1769)."""
    repo = Repository(pile)
    if branch is not None:
        return repo.checkout_name(branch)
    col = Collection(repo, MODEL_GRAPH)
    if col.exists():
        return col.latest()
    names = repo.branches()
    for b in LEGACY_BRANCHES:
        if b in names:
            return repo.checkout_name(b)
    raise LookupError(f"{getattr(pile, 'path', 'pile')}: no model-graph collection and no legacy branch")


def pile_facts(path, branch: str | None = None):
    pile = Pile.open(str(path), create=False)
    return pile, read_model_pile(pile, branch)


def load_keymap_from_pile(pile, facts: TribleSet | None = None, sel: ModelSelector = ModelSelector.only(),
                          shards: bool = False) -> SelectedModelIndex:
    facts = facts if facts is not None else read_model_pile(pile)
    return SelectedModelIndex.from_snapshot(pile, facts, sel, shards)


def load_config(pile, facts: TribleSet, root: bytes | None = None, name: str = "config.json") -> dict:
    """Model hyper-parameters come from facts in the same pile: ``open(pile) -> model`` needs no side files
    (src/bin/inkling_forward.rs:2841-2854)."""
    return jsonfacts.load_document(pile, facts, name, owner=root)


def derive_half_root(pile, key, facts: TribleSet, root: bytes, dtype: str = "f16") -> bytes:
    """Sibling root holding the same tensors in f16/bf16 (src/persist.rs:246-295)."""
    tb = TribleBuilder()
    members = []
    for m in root_members(facts, root):
        a = load_module_leaf(pile, facts, m).to_f32()
        n = module_name(pile, facts, m)
        if dtype == "f16":
            members.append(put_tensor(pile, tb, n, a.astype(np.float16), Elem.F16))
        else:
            members.append(put_tensor(pile, tb, n, f32_to_bf16_bits(a), Elem.BF16))
    name = facts.maybe(root, S.MODEL_NAME)
    src = facts.maybe(root, S.SOURCE)
    new = build_model_root(pile, tb, members, name=get_text(pile, name) if name else None,
                           source=get_text(pile, src) if src else None, quantization=dtype)
    publish_fragment(pile, key, tb.build(), f"derive {dtype}")
    return new


def default_key(pile_path) -> object:
    return signing_key_file(str(pile_path) + ".key")


def import_file_filtered_to_collection(pile, key, file, dtype: str = "f32", source: str | None = None, quantization: str | None = None,
                                       keep=lambda name: True, name: str | None = None) -> bytes:
    """Import ONE weight file (safetensors, GGUF or a torch pickle), keeping only the tensors ``keep(name)`` accepts, as a model
    root of its own — a component of a larger checkpoint (a vision tower, a codec) becomes selectable by source / quantisation
    without importing the rest (src/persist.rs:296-417).  The file name is recorded as provenance; a filter that selects no float
    tensor is an error, and a torn pile tail refuses the import as always."""
    pile.refresh()
    tb = TribleBuilder()
    members = ingest_members(pile, tb, file, dtype, keep)
    if not members:
        raise ValueError(f"the filtered import selected no supported float tensor from {file}")
    root = build_model_root(pile, tb, members, name=name or Path(file).name, source=source or str(file),
                            quantization=quantization or (None if dtype == "f32" else dtype))
    Collection(Repository(pile, key), MODEL_GRAPH).publish(tb.build(), f"component {Path(file).name}"[:32])
    pile.flush()
    return root


def load_split_index_from_pile(pile, f16_prefix: str, facts: TribleSet | None = None) -> tuple[dict, dict]:
    """``(half-precision leaves, single-precision leaves)`` by tensor name: the roots whose MODEL NAME starts with ``f16_prefix``
    feed the first map, all others the second (src/persist.rs:940-1014).  Serving lanes that keep the large matrices in half
    precision and the small, precision-critical tensors (norm gains, biases) in f32 read both maps from one pile."""
    from .model import index_keymap
    facts = facts if facts is not None else read_model_pile(pile)
    half, single = {}, {}
    for root, v in facts.with_attr(S.MODEL_NAME):
        name = get_text(pile, v)
        target = half if (f16_prefix and name.startswith(f16_prefix)) else single
        for n, module in index_keymap(pile, facts, root).items():
            target[n] = load_module_leaf(pile, facts, module)
    return half, single
