"""``mary import <checkpoint dir|file> --pile P --key K [--dtype f16|bf16|f32] [--name N]``, ``mary keys --pile P``, and the pile
maintenance commands ``mary branches|verify|stats|migrate|equiv --pile P`` (the reference's ``pile_branches`` / ``pile_leaf_verify`` /
``pile_leaf_migrate`` / ``pile_loader_equiv`` binaries).

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


def cmd_branches(a) -> int:
    """Branches of a pile with their heads and commit counts (the reference's ``pile_branches`` binary)."""
    from ..pile.repo import Repository
    pile = Pile.open(a.pile, create=False)
    repo = Repository(pile)
    for name, ids in sorted(repo.branches().items()):
        for bid in ids:
            head = repo.head(bid)
            n = len(repo.ancestors(head, verify=not a.no_verify)) if head else 0
            print(f"{name}  id={bid.hex()}  head={head.hex() if head else '-'}  commits={n}")
    pile.close()
    return 0


def cmd_verify(a) -> int:
    """Re-hash every blob record and parse every tensor leaf of every model root (``pile_leaf_verify``): exit 1 on the first
    record whose bytes do not hash to its handle or whose leaf header is inconsistent with its payload."""
    from ..format.model import load_module_leaf
    from ..pile.hashing import blake3
    from ..pile.store import KIND_BLOB
    pile = Pile.open(a.pile, create=False, validate=False)
    n = bad = 0
    for rec in pile.records():
        if rec.kind != KIND_BLOB:
            continue
        n += 1
        if blake3(pile.get(rec.hash)) != rec.hash:
            print(f"CORRUPT blob {rec.hash.hex()} at offset {rec.offset}")
            bad += 1
    facts = read_model_pile(pile)
    leaves = 0
    for r in model_roots(facts):
        for name, ent in index_keymap(pile, facts, r).items():
            try:
                leaf = load_module_leaf(pile, facts, ent)
                leaf.to_f32() if a.deep else None
                leaves += 1
            except Exception as ex:  # report and count every broken leaf
                print(f"BAD leaf {name}: {ex}")
                bad += 1
    print(f"{n} blobs, {leaves} tensor leaves, {bad} problems")
    pile.close()
    return 1 if bad else 0


def cmd_stats(a) -> int:
    pile = Pile.open(a.pile, create=False)
    kinds = {}
    for rec in pile.records():
        k = kinds.setdefault(rec.kind, [0, 0])
        k[0] += 1
        k[1] += rec.length
    print(f"{a.pile}: {pile.size} bytes")
    for kind, (cnt, nbytes) in sorted(kinds.items()):
        print(f"  kind {kind}: {cnt} records, {nbytes} payload bytes")
    pile.close()
    return 0


def cmd_migrate(a) -> int:
    """Legacy two-blob leaves -> typed tensors, pile to pile into a NEW file (``pile_leaf_migrate``); with ``--branch`` the facts of a
    legacy named branch are first published into the model-graph collection (the ``model-migration`` step)."""
    from ..format.migrate import branch_to_collection, migrate_leaves
    src = Pile.open(a.pile, create=False)
    key = signing_key_file(a.key)
    if a.branch:
        print(f"published {branch_to_collection(src, key)} facts from a legacy branch into the collection")
    dst = Pile.open(a.out)
    st = migrate_leaves(src, dst, key)
    print(" ".join(f"{k}={v}" for k, v in st.items()))
    dst.close(), src.close()
    return 0


def cmd_equiv(a) -> int:
    """Compare two piles through the public loader, tensor by tensor (``pile_loader_equiv``); the second must read typed leaves."""
    from ..format.migrate import loader_equiv
    x, y = Pile.open(a.pile, create=False), Pile.open(a.other, create=False)
    try:
        st = loader_equiv(x, y)
    except AssertionError as ex:
        print(f"NOT EQUIVALENT: {ex}")
        return 1
    print(f"{st['tensors']} tensors equal through the loader, {st['typed']} typed")
    return 0


def cmd_k3_gate(a) -> int:
    """The K3 layout gate (tests/k3_layout_gate.rs): the two halves of the name <-> slot mapping against a checkpoint's own headers."""
    from ..models.k3.ckpt import K3Checkpoint
    ck = K3Checkpoint(a.dir)
    g = ck.gate()
    ck.close()
    bad = sum(len(v) for v in g.values())
    print(f"{len(ck)} tensors in {len(ck.shards())} shards; " + ", ".join(f"{k} {len(v)}" for k, v in g.items()))
    for k, v in g.items():
        for item in v[:a.show]:
            print(f"  {k}: {item}")
    return 1 if bad else 0


def cmd_k3_experts(a) -> int:
    """The K3 expert address book (``k3_expert_index``): gate first, bandwidth only when the gate passes."""
    from ..models.k3.ckpt import K3Checkpoint, expert_index, fetch_sweep
    ck = K3Checkpoint(a.dir)
    ix = expert_index(ck)
    print(f"address book: {len(ix['book'])} routed experts (expected {ix['expected']}), {ix['expert_bytes']} bytes each")
    print(f"experts with another size: {len(ix['wrong_size'])}; split or interleaved: {len(ix['split'])}")
    print("resident set (everything that is not a routed expert):")
    for g, n in sorted(ix["resident"].items(), key=lambda kv: -kv[1]):
        print(f"  {g:<32} {n / 2 ** 30:10.4f} GiB")
    if not ix["ok"]:
        print("GATE FAIL: no bandwidth number is reported")
        ck.close()
        return 1
    print("GATE PASS")
    for n, cnt, dt, gbs in fetch_sweep(ck, ix["book"], [int(x) for x in a.sweep.split(",")], a.per_level):
        print(f"  {n:3d} readers: {cnt} experts in {dt * 1e3:.1f} ms = {gbs:.2f} GB/s")
    ck.close()
    return 0


def cmd_fit(a) -> int:
    """Does a sparse-MoE serving configuration fit the GPUs (the question ``gemma31b_fit`` / ``resident_final`` answer by allocating)?
    Prints the per-GPU bill — expert slabs, attention / dense / head weights, paged KV cache for ``batch x ctx`` tokens, activations,
    workspace — against the capacity, and how many expert slabs can stay resident when not all do."""
    from ..models.moe.config import inkling_style_config, k3_class_config
    from ..runtime.budget import AdmissionError, check, moe_bill
    cfg = {"k3": k3_class_config, "inkling": inkling_style_config}[a.model]()
    cap = int(a.capacity_gib * 2 ** 30)
    n_moe = sum(1 for i in range(cfg.num_hidden_layers) if not cfg.is_dense(i)) + cfg.num_mtp_layers
    rc = 0
    for world in [int(x) for x in a.gpus.split(",")]:
        # from 4 GPUs up the serving layout is data-parallel attention + all-to-all experts: a rank caches only its own sequences
        local = a.batch // world if (world >= 4 and not a.replicated_kv) else a.batch
        bill = moe_bill(cfg, world, local, a.ctx, local * (1 + a.spec), cap)
        try:
            check(bill)
            print(f"{world} GPU(s): fits, all {n_moe} expert slabs resident: {bill.lines()}")
            continue
        except AdmissionError:
            pass
        slabs = n_moe
        while slabs > 0:
            b = moe_bill(cfg, world, local, a.ctx, local * (1 + a.spec), cap, expert_slabs=slabs)
            if b.total <= cap * 0.97:
                break
            slabs -= 1
        if slabs:
            print(f"{world} GPU(s): fits only with {slabs} of {n_moe} expert slabs resident (the rest are streamed or shared): {b.lines()}")
        else:
            print(f"{world} GPU(s): does NOT fit even with one resident slab: {bill.lines()}")
            rc = 1
    return rc


def cmd_encode(a) -> int:
    """Text on stdin, an ids file out (``inkling_encode``): stdin is taken VERBATIM (leading space and trailing bytes included; use
    ``printf '%s'``, not ``echo``); ids go out as little-endian i64, the form the serving CLI reads; the decode round trip is printed
    so that a file can be checked against the string it claims to be."""
    import numpy as np
    text = sys.stdin.buffer.read().decode("utf-8")
    if a.tokenizer_json:
        from tokenizers import Tokenizer
        tok = Tokenizer.from_file(a.tokenizer_json)
    else:
        from ..format.tokenizer import build_tokenizer, select_tokenizer
        pile = Pile.open(a.pile, create=False)
        facts = read_model_pile(pile)
        tok = build_tokenizer(pile, facts, select_tokenizer(pile, facts, a.tokenizer))
    ids = tok.encode(text, add_special_tokens=False).ids
    np.asarray(ids, dtype="<i8").tofile(a.out)
    print(f"{len(ids)} ids -> {a.out}")
    print(f"ids: {ids[:32]}{' ...' if len(ids) > 32 else ''}")
    print(f"decode: {tok.decode(ids)!r}")
    return 0


def cmd_flags(a) -> int:
    from ..utils import flags
    for name, kind, default, value, doc in flags.table():
        mark = "" if value == default else "   <- set"
        print(f"{name:<22}{kind:<6}default {default!s:<10} value {value!s:<10}{mark}\n    {doc}")
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
    b = sub.add_parser("branches")
    b.add_argument("--pile", required=True)
    b.add_argument("--no-verify", action="store_true", help="skip the signature check of every commit")
    b.set_defaults(fn=cmd_branches)
    v = sub.add_parser("verify")
    v.add_argument("--pile", required=True)
    v.add_argument("--deep", action="store_true", help="also decode every leaf to f32")
    v.set_defaults(fn=cmd_verify)
    st = sub.add_parser("stats")
    st.add_argument("--pile", required=True)
    st.set_defaults(fn=cmd_stats)
    mg = sub.add_parser("migrate")
    mg.add_argument("--pile", required=True), mg.add_argument("--out", required=True), mg.add_argument("--key", required=True)
    mg.add_argument("--branch", action="store_true", help="first publish a legacy branch's facts into the model-graph collection")
    mg.set_defaults(fn=cmd_migrate)
    eq = sub.add_parser("equiv")
    eq.add_argument("--pile", required=True), eq.add_argument("--other", required=True)
    eq.set_defaults(fn=cmd_equiv)
    kg = sub.add_parser("k3-gate")
    kg.add_argument("dir"), kg.add_argument("--show", type=int, default=10)
    kg.set_defaults(fn=cmd_k3_gate)
    ke = sub.add_parser("k3-experts")
    ke.add_argument("dir"), ke.add_argument("--sweep", default="1,4,16"), ke.add_argument("--per-level", type=int, default=32)
    ke.set_defaults(fn=cmd_k3_experts)
    ft = sub.add_parser("fit")
    ft.add_argument("--model", default="k3", choices=["k3", "inkling"]), ft.add_argument("--gpus", default="1,2,4,8")
    ft.add_argument("--batch", type=int, default=128), ft.add_argument("--ctx", type=int, default=4160), ft.add_argument("--spec", type=int, default=2)
    ft.add_argument("--capacity-gib", type=float, default=178.0)
    ft.add_argument("--replicated-kv", action="store_true", help="every rank caches all sequences (tensor-parallel attention) at any GPU count")
    ft.set_defaults(fn=cmd_fit)
    en = sub.add_parser("encode")
    en.add_argument("out"), en.add_argument("--pile"), en.add_argument("--tokenizer"), en.add_argument("--tokenizer-json")
    en.set_defaults(fn=cmd_encode)
    ga = sub.add_parser("gate", help="run a correctness gate (or 'all'); --mutate runs its positive control")
    ga.add_argument("name"), ga.add_argument("--mutate", action="store_true")
    ga.set_defaults(fn=lambda a: __import__("mary_b200.gates", fromlist=["run"]).run(a.name, a.mutate))
    fl = sub.add_parser("flags", help="the environment flags of the package with the values in effect")
    fl.set_defaults(fn=cmd_flags)
    a = ap.parse_args(argv)
    if argv is None:                                  # run as a program: fail loudly on any thread
        from ..utils import fatal
        fatal.arm()
    return a.fn(a)


if __name__ == "__main__":
    sys.exit(main())
