import os

import numpy as np
import pytest

from mary_b200.pile import (Collection, MemoryBlobStore, Pile, PileError, RepoError, Repository, TribleBuilder,
                            TribleSet, blake3, blake3_py, content_id, id_hex, signing_key_file)
from mary_b200.pile.trible import v_shortstring, v_u256

A = id_hex("4C1CD1611863E7854C59C7DC706DF77A")
B = id_hex("52C4A211D2A08BA25C27FFD79FF24C93")


def test_blake3_vectors_and_twin():
    assert blake3(b"").hex() == "af1349b9f5f9a1a6a0404dea36dcc9499bcb25c9adc112b7cc9a93cae41f3262"
    assert blake3(bytes([0])).hex() == "2d3adedff11b61f14c886e35afa036736dcd87a74d27b5c1510225d0f592e213"
    for n in (1, 63, 64, 65, 1023, 1024, 1025, 2048, 3 * 1024 + 1, 7 * 1024 + 100):
        d = bytes(i % 251 for i in range(n))
        assert blake3(d) == blake3_py(d), n


def test_blake3_parallel_path_matches_sequential():
    # > 8 MiB goes through the threaded tree; hashing it in one piece and via a memoryview must agree,
    # and the result must equal the sequential implementation run on the same bytes (pure Python on a prefix tree
    # would be too slow, so compare against a second native call with a copy that defeats any caching).
    d = np.random.default_rng(0).integers(0, 256, 9 * (1 << 20) + 12345, dtype=np.uint8)
    h1 = blake3(d.tobytes())
    h2 = blake3(memoryview(d))
    assert h1 == h2
    # a one-byte change must change the hash
    d[len(d) // 2] ^= 1
    assert blake3(d.tobytes()) != h1


def test_put_get_dedup_alignment(tmp_path):
    p = Pile.open(str(tmp_path / "a.pile"))
    h1 = p.put(b"hello world")
    h2 = p.put(b"hello world")
    assert h1 == h2 and bytes(p.get(h1)) == b"hello world"
    st = p.stats()
    assert st["bytes_dedup"] == 11 and st["records"] == 1
    big = os.urandom(1000)
    hb = p.put(big)
    for r in p.records():
        assert r.offset % 256 == 0          # payloads sit at 256-byte aligned file offsets
    assert bytes(p.get(hb)) == big
    p.close()
    p = Pile.open(str(tmp_path / "a.pile"), create=False)
    assert bytes(p.get(hb)) == big
    with pytest.raises(PileError):
        p.get(b"\x00" * 32)
    p.close()


def test_torn_tail_is_refused_and_amputate_repairs(tmp_path):
    path = str(tmp_path / "a.pile")
    p = Pile.open(path)
    h = p.put(b"x" * 300)
    size = p.size
    p.close()
    with open(path, "ab") as f:
        f.write(b"garbage" * 10)
    with pytest.raises(PileError, match="torn tail"):
        Pile.open(path)
    assert os.path.getsize(path) == size + 70        # refusing did not truncate
    assert Pile.amputate(path) == 70
    p = Pile.open(path)
    assert bytes(p.get(h)) == b"x" * 300
    p.close()


def test_corrupt_blob_fails_validation(tmp_path):
    path = str(tmp_path / "a.pile")
    p = Pile.open(path)
    h = p.put(b"y" * 1000)
    off = next(iter(p.records())).offset
    p.close()
    with open(path, "r+b") as f:
        f.seek(off + 10)
        f.write(b"Z")
    p = Pile.open(path)
    with pytest.raises(PileError, match="BLAKE3"):
        p.get(h)
    p.close()


def test_tribleset_canonical_and_queries():
    tb = TribleBuilder()
    e1 = tb.entity([(A, v_shortstring("one")), (B, v_u256(1))])
    e2 = tb.entity([(A, v_shortstring("two")), (B, v_u256(2))])
    tb.entity([(A, v_shortstring("one")), (B, v_u256(1))])     # same content -> same id, deduped
    ts = tb.build()
    assert len(ts) == 4 and e1 != e2
    assert e1 == content_id([(B, v_u256(1)), (A, v_shortstring("one"))])   # order-independent
    assert ts.entities_where(A, v_shortstring("two")) == [e2]
    assert TribleSet.from_archive(ts.archive()) == ts
    assert (ts | ts) == ts
    assert ts.find([("e", A, v_shortstring("one")), ("e", B, "n")]) == [{"e": e1, "n": v_u256(1)}]
    with pytest.raises(LookupError):
        ts.one(e1, id_hex("00" * 15 + "01"))


@pytest.mark.parametrize("kind", ["pile", "memory"])
def test_branches_commits_checkout(tmp_path, kind):
    store = Pile.open(str(tmp_path / "r.pile")) if kind == "pile" else MemoryBlobStore()
    key = signing_key_file(str(tmp_path / "k"))
    repo = Repository(store, key)
    b = repo.create_branch("main")
    with pytest.raises(RepoError):
        repo.create_branch("main")
    t1, t2 = TribleBuilder(), TribleBuilder()
    t1.entity([(A, v_shortstring("a"))])
    t2.entity([(A, v_shortstring("b"))])
    c1 = repo.commit(b, t1.build(), "first")
    c2 = repo.commit(b, t2.build(), "second")
    assert repo.head(b) == c2 and repo.ancestors(c2) == [c2, c1]
    assert len(repo.checkout(b)) == 2
    assert repo.lookup_branch("main") == b
    with pytest.raises(RepoError):
        repo.lookup_branch("nope")
    # a reader without a key can check signatures but cannot commit
    with pytest.raises(RepoError):
        Repository(store).commit(b, t1.build())


def test_bad_signature_detected(tmp_path):
    store = MemoryBlobStore()
    key = signing_key_file(str(tmp_path / "k"))
    repo = Repository(store, key)
    b = repo.create_branch("main")
    tb = TribleBuilder()
    tb.entity([(A, v_shortstring("a"))])
    c = repo.commit(b, tb.build(), "x")
    blob = bytearray(store._blobs[c])
    from mary_b200.pile.repo import A_SIG_R
    ts = TribleSet.from_archive(bytes(blob))
    row = [i for i, (_e, a, _v) in enumerate(ts) if a == A_SIG_R][0]
    blob[row * 64 + 40] ^= 0xFF
    store._blobs[c] = bytes(blob)
    with pytest.raises(RepoError, match="signature"):
        repo.read_commit(c)


def test_collection_publish_snapshot_teams(tmp_path):
    store = MemoryBlobStore()
    key = signing_key_file(str(tmp_path / "k"))
    col = Collection(Repository(store, key))
    assert not col.exists()
    t1, t2 = TribleBuilder(), TribleBuilder()
    t1.entity([(A, v_shortstring("a"))])
    t2.entity([(A, v_shortstring("b"))])
    ticket1 = col.publish(t1.build())
    col.publish(t2.build())
    assert len(col.latest()) == 2 and len(col.snapshot(ticket1)) == 1
    assert len(col.sole_team()) == 32
    other = Collection(Repository(store, signing_key_file(str(tmp_path / "k2"))))
    other.publish(t1.build())
    with pytest.raises(RepoError):
        col.sole_team()


def test_push_copies_reachable_blobs(tmp_path):
    src, dst = MemoryBlobStore(), MemoryBlobStore()
    key = signing_key_file(str(tmp_path / "k"))
    repo = Repository(src, key)
    b = repo.create_branch("main")
    payload = src.put(b"tensor-bytes")
    tb = TribleBuilder()
    tb.entity([(A, payload)])
    repo.commit(b, tb.build(), "m")
    repo.push(dst, b)
    r2 = Repository(dst)
    assert len(r2.checkout_name("main")) == 1 and bytes(dst.get(payload)) == b"tensor-bytes"
