"""Branches, signed commits and append-only collections on top of a blob store.

Reference behaviour (external crate, usage at src/persist.rs:757-799,1777-1823 and
src/models/inkling/pile.rs:738-763; collections at src/model_collection.rs:27-76,346-900):

* a branch is a named pointer to a head commit; a commit is a small signed fact set that names a
  content blob (a TribleSet archive) and its parent commits; ``checkout`` is the union of the content
  of the head and all its ancestors;
* commits are signed with ed25519;
* a *collection* is an append-only, signed union of fragments published by one team (key); readers
  take either the local latest snapshot or an exact ticket (commit handle).
"""
from __future__ import annotations

import os
from pathlib import Path

from cryptography.hazmat.primitives import serialization
from cryptography.hazmat.primitives.asymmetric.ed25519 import Ed25519PrivateKey, Ed25519PublicKey

from .trible import (TribleBuilder, TribleSet, fresh_id, id_hex, r_shortstring, v_handle, v_shortstring)

# attribute ids of the commit / branch metadata (this build's own namespace)
A_CONTENT = id_hex("4DD4DDD05CC31734B03ABB4E43188B1F")
A_PARENT = id_hex("317044B612C690000D798CA660ECFD2A")
A_MESSAGE = id_hex("B59D147839100B6ED4B165DF76EDF3BB")
A_SIGNED_BY = id_hex("ADB4FFAD247C886848161297EFF5A05B")
A_SIG_R = id_hex("9DF34F84959928F93A3C40AEB6E9E499")
A_SIG_S = id_hex("1ACE03BF70242B289FDF00E4327C3BC6")
A_BRANCH_NAME = id_hex("2E26F8BA886495A8DF04ACF0ED3ACBD4")
A_BRANCH_HEAD = id_hex("272FBC56108F336C4D2E17289468C35F")
A_COLLECTION = id_hex("6C1B0F5A7E0C4B2D9A7F3E21B8D4C5A6")

MODEL_GRAPH = "mary-model-graph"
MODEL_BUNDLES = "mary-model-bundles"


class RepoError(RuntimeError):
    pass


def signing_key_file(path: str | os.PathLike, create: bool = True) -> Ed25519PrivateKey:
    """Load a 32-byte hex seed from ``path``; create it (mode 0600) when absent and ``create``."""
    p = Path(path)
    if p.exists():
        seed = bytes.fromhex(p.read_text().strip())
        if len(seed) != 32:
            raise RepoError(f"{p}: expected 64 hex digits")
        return Ed25519PrivateKey.from_private_bytes(seed)
    if not create:
        raise RepoError(f"{p}: no signing key")
    seed = os.urandom(32)
    p.write_text(seed.hex() + "\n")
    os.chmod(p, 0o600)
    return Ed25519PrivateKey.from_private_bytes(seed)


def public_bytes(key: Ed25519PrivateKey) -> bytes:
    return key.public_key().public_bytes(serialization.Encoding.Raw, serialization.PublicFormat.Raw)


class Repository:
    def __init__(self, store, key: Ed25519PrivateKey | None = None):
        self.store = store
        self.key = key

    # ------------------------------------------------------------------ branches
    def _branch_table(self) -> dict[bytes, tuple[str, bytes | None]]:
        """branch id -> (name, head) — the last record of a branch id wins."""
        table: dict[bytes, tuple[str, bytes | None]] = {}
        for bid, payload in self.store.branch_records():
            ts = TribleSet.from_archive(payload)
            name = r_shortstring(ts.one(bid, A_BRANCH_NAME))
            head = ts.maybe(bid, A_BRANCH_HEAD)
            table[bid] = (name, head)
        return table

    def branches(self) -> dict[str, list[bytes]]:
        out: dict[str, list[bytes]] = {}
        for bid, (name, _h) in self._branch_table().items():
            out.setdefault(name, []).append(bid)
        return out

    def lookup_branch(self, name: str) -> bytes:
        ids = self.branches().get(name, [])
        if len(ids) != 1:
            raise RepoError(f"branch {name!r}: found {len(ids)}, expected exactly 1")
        return ids[0]

    def create_branch(self, name: str) -> bytes:
        if name in self.branches():
            raise RepoError(f"branch {name!r} already exists")
        bid = fresh_id()
        self._write_branch(bid, name, None)
        return bid

    def ensure_branch(self, name: str) -> bytes:
        ids = self.branches().get(name, [])
        if len(ids) > 1:
            raise RepoError(f"branch {name!r} is ambiguous ({len(ids)} ids)")
        return ids[0] if ids else self.create_branch(name)

    def _write_branch(self, bid: bytes, name: str, head: bytes | None) -> None:
        b = TribleBuilder()
        b.add(bid, A_BRANCH_NAME, v_shortstring(name))
        if head is not None:
            b.add(bid, A_BRANCH_HEAD, v_handle(head))
        self.store.put_branch(bid, b.build().archive())

    def head(self, branch: bytes) -> bytes | None:
        t = self._branch_table()
        if branch not in t:
            raise RepoError(f"unknown branch id {branch.hex()}")
        return t[branch][1]

    # ------------------------------------------------------------------ commits
    def commit(self, branch: bytes, content: TribleSet, message: str = "") -> bytes:
        if self.key is None:
            raise RepoError("a signing key is required to commit")
        name, parent = self._branch_table()[branch]
        content_h = self.store.put(content.archive())
        pairs = [(A_CONTENT, v_handle(content_h)), (A_MESSAGE, v_shortstring(message[:32]))]
        if parent is not None:
            pairs.append((A_PARENT, v_handle(parent)))
        signed = content_h + (parent or b"")
        sig = self.key.sign(signed)
        pairs += [(A_SIGNED_BY, public_bytes(self.key)), (A_SIG_R, sig[:32]), (A_SIG_S, sig[32:])]
        b = TribleBuilder()
        b.entity(pairs)
        commit_h = self.store.put(b.build().archive())
        self._write_branch(branch, name, commit_h)
        return commit_h

    def read_commit(self, commit_h: bytes, verify: bool = True) -> dict:
        ts = TribleSet.from_archive(self.store.get(commit_h))
        ents = {e for e, _ in ts.with_attr(A_CONTENT)}
        if len(ents) != 1:
            raise RepoError(f"commit {commit_h.hex()} is malformed")
        e = next(iter(ents))
        content = ts.one(e, A_CONTENT)
        parents = ts.values(e, A_PARENT)
        pub = ts.one(e, A_SIGNED_BY)
        sig = ts.one(e, A_SIG_R) + ts.one(e, A_SIG_S)
        if verify:
            try:
                Ed25519PublicKey.from_public_bytes(pub).verify(sig, content + b"".join(parents))
            except Exception as ex:  # cryptography.exceptions.InvalidSignature
                raise RepoError(f"commit {commit_h.hex()}: bad signature") from ex
        return {"content": content, "parents": parents, "signed_by": pub,
                "message": r_shortstring(ts.one(e, A_MESSAGE))}

    def ancestors(self, head: bytes | None, verify: bool = True) -> list[bytes]:
        seen, order, stack = set(), [], [head] if head else []
        while stack:
            c = stack.pop()
            if c in seen:
                continue
            seen.add(c)
            order.append(c)
            stack.extend(self.read_commit(c, verify)["parents"])
        return order

    def checkout(self, branch: bytes, verify: bool = True) -> TribleSet:
        """Union of the content of every commit reachable from the branch head."""
        sets = []
        for c in self.ancestors(self.head(branch), verify):
            sets.append(TribleSet.from_archive(self.store.get(self.read_commit(c, False)["content"])))
        return TribleSet.union(sets)

    def checkout_name(self, name: str) -> TribleSet:
        return self.checkout(self.lookup_branch(name))

    # ------------------------------------------------------------------ transfer
    def push(self, other_store, branch: bytes, handle_attrs: set[bytes] | None = None) -> int:
        """Copy a branch (commits, content archives and every blob referenced by a value whose attribute
        is in ``handle_attrs``; all 32-byte values that resolve in this store when ``None``) to another store."""
        n = 0
        name, head = self._branch_table()[branch]
        for c in self.ancestors(head):
            info = self.read_commit(c, False)
            for h in (c, info["content"]):
                other_store.put(self.store.get(h)); n += 1
            ts = TribleSet.from_archive(self.store.get(info["content"]))
            for _e, a, v in ts:
                if (handle_attrs is None or a in handle_attrs) and self.store.has(v):
                    other_store.put(self.store.get(v)); n += 1
        b = TribleBuilder()
        b.add(branch, A_BRANCH_NAME, v_shortstring(name))
        if head:
            b.add(branch, A_BRANCH_HEAD, v_handle(head))
        other_store.put_branch(branch, b.build().archive())
        return n


class Collection:
    """Append-only signed union of fragments (src/model_collection.rs:60-76,346-900).

    A collection is kept on a branch named after it; each ``publish`` is one signed commit.  A *ticket*
    is a commit handle: ``snapshot(ticket)`` reads exactly the state at that commit, ``latest()`` the
    local head.  ``teams()`` lists the keys that signed into it; ``sole_team()`` insists on exactly one."""

    def __init__(self, repo: Repository, name: str = MODEL_GRAPH):
        self.repo, self.name = repo, name

    def _branch(self, create: bool) -> bytes | None:
        ids = self.repo.branches().get(self.name, [])
        if len(ids) > 1:
            raise RepoError(f"collection {self.name!r} is ambiguous")
        if ids:
            return ids[0]
        return self.repo.create_branch(self.name) if create else None

    def publish(self, fragment: TribleSet, message: str = "fragment") -> bytes:
        return self.repo.commit(self._branch(True), fragment, message)

    def latest(self) -> TribleSet:
        b = self._branch(False)
        if b is None:
            raise RepoError(f"collection {self.name!r} does not exist in this pile")
        return self.repo.checkout(b)

    def exists(self) -> bool:
        return self._branch(False) is not None

    def ticket(self) -> bytes | None:
        b = self._branch(False)
        return self.repo.head(b) if b else None

    def snapshot(self, ticket: bytes) -> TribleSet:
        sets = []
        for c in self.repo.ancestors(ticket):
            sets.append(TribleSet.from_archive(self.repo.store.get(self.repo.read_commit(c, False)["content"])))
        return TribleSet.union(sets)

    def teams(self) -> set[bytes]:
        b = self._branch(False)
        if b is None:
            return set()
        return {self.repo.read_commit(c)["signed_by"] for c in self.repo.ancestors(self.repo.head(b))}

    def sole_team(self) -> bytes:
        t = self.teams()
        if len(t) != 1:
            raise RepoError(f"collection {self.name!r} has {len(t)} signing teams, expected exactly 1")
        return next(iter(t))
