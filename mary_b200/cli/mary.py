"""``mary import <checkpoint dir|file> --pile P --key K [--dtype f16|bf16|f32] [--name N]`` and ``mary keys --pile P``.

The front-door CLI of the reference (src/bin/mary.rs:54-240): import a checkpoint (safetensors > gguf > pickle) with its
``config.json`` and ``tokenizer.json`` into a pile as one signed commit of the model-graph collection (idempotent: re-importing
the same bytes adds nothing), and list what a pile holds."""
from __future__ import annotations

import argparse
import sys

from ..format import schema as S
from ..format.model import get_text, index_keymap
from ..format.persist import import_model_to_collection, read_model_pile
from ..format.selection import model_roots
from ..pile import Pile, signing_key_file
from ..pile.trible import r_shortstring


def cmd_import(a) -> int:
    pile = Pile.open(a.pile)
    key = signing_key_file(a.key)
    root = import_model_to_collection(pile, key, a.source, name=a.name, source=a.source, dtype=a.dtype)
    st = pile.stats()
    print(f"imported root {root.hex()} into {a.pile}: {st['bytes_put']} new bytes, {st['bytes_dedup']} deduplicated")
    pile.close()
    return 0


def cmd_keys(a) -> int:
    pile = Pile.open(a.pile, create=False)
    facts = read_model_pile(pile)
    for r in model_roots(facts):
        name = facts.maybe(r, S.MODEL_NAME)
        q = facts.maybe(r, S.QUANTIZATION)
        km = index_keymap(pile, facts, r)
        print(f"root {r.hex()} name={get_text(pile, name) if name else '-'} quantization={r_shortstring(q) if q else '-'} tensors={len(km)}")
        if a.verbose:
            from ..format.model import load_module_leaf
            for n in sorted(km):
                leaf = load_module_leaf(pile, facts, km[n])
                print(f"  {n}  {leaf.elem.name}{list(leaf.dims)}")
    pile.close()
    return 0


def main(argv=None) -> int:
    ap = argparse.ArgumentParser(prog="mary")
    sub = ap.add_subparsers(dest="cmd", required=True)
    i = sub.add_parser("import")
    i.add_argument("source")
    i.add_argument("--pile", required=True)
    i.add_argument("--key", required=True)
    i.add_argument("--dtype", default="f32", choices=["f32", "f16", "bf16"])
    i.add_argument("--name")
    i.set_defaults(fn=cmd_import)
    k = sub.add_parser("keys")
    k.add_argument("--pile", required=True)
    k.add_argument("-v", "--verbose", action="store_true")
    k.set_defaults(fn=cmd_keys)
    a = ap.parse_args(argv)
    return a.fn(a)


if __name__ == "__main__":
    sys.exit(main())
