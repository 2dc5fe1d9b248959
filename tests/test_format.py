import io
import json
import pickle
import struct
import zipfile

import numpy as np
import pytest

from mary_b200.format import jsonfacts, schema as S
from mary_b200.format.formats import detect_format, iter_gguf, iter_pickle
from mary_b200.format.ingest import f32_to_bf16_bits, ingest_model, ingest_tensors
from mary_b200.format.leaf import (Elem, LeafError, put_array, put_leaf, put_leaf_legacy, resolve, tensor_blob)
from mary_b200.format.model import build_model_root, index_keymap, put_fp4_tensor, put_tensor
from mary_b200.format.persist import (derive_half_root, import_model_to_collection, load_config, read_model_pile)
from mary_b200.format.safetensors import SafeTensors, save_file
from mary_b200.format.selection import ModelSelector, SelectedModelIndex, SelectionError, select_model_root
from mary_b200.format.tiktoken import TikToken
from mary_b200.format.tokenizer import (build_tokenizer, load_tiktoken, load_tokenizer_json, save_tiktoken,
                                        save_tokenizer_json)
from mary_b200.nn.fp4 import quantize_weight_nvfp4
from mary_b200.pile import MemoryBlobStore, Pile, TribleBuilder
from mary_b200.pile.trible import v_handle


@pytest.mark.parametrize("form", ["typed", "legacy"])
def test_leaf_both_forms_roundtrip(form):
    st, tb = MemoryBlobStore(), TribleBuilder()
    a = np.arange(24, dtype=np.float32).reshape(2, 3, 4)
    e = put_array(st, tb, a) if form == "typed" else put_leaf_legacy(st, tb, a)
    leaf = resolve(st, tb.build(), e)
    assert leaf.dims == (2, 3, 4) and np.array_equal(leaf.to_f32(), a)
    assert leaf.view_f32().base is not None          # zero-copy view


def test_leaf_scalar_rank0_and_rank_limits():
    st, tb = MemoryBlobStore(), TribleBuilder()
    e = put_array(st, tb, np.float32(3.5).reshape(()))
    assert resolve(st, tb.build(), e).to_f32().reshape(()) == 3.5
    put_array(st, tb, np.zeros((1,) * 6, dtype=np.float32))
    with pytest.raises(LeafError, match="rank 7"):
        put_array(st, tb, np.zeros((1,) * 7, dtype=np.float32))


def test_leaf_identical_tensors_dedupe_and_two_payloads_refused():
    st, tb = MemoryBlobStore(), TribleBuilder()
    a = np.ones((4, 4), dtype=np.float32)
    e1, e2 = put_array(st, tb, a), put_array(st, tb, a.copy())
    assert e1 == e2 and st.bytes_dedup > 0
    h = st.put(a.tobytes())
    tb.add(e1, S.DATA, v_handle(h))                  # a second payload on the same entity
    with pytest.raises(LeafError, match="payloads"):
        resolve(st, tb.build(), e1)


def test_leaf_header_payload_mismatch_refused():
    with pytest.raises(LeafError):
        tensor_blob(Elem.F32, (2, 2), b"\x00" * 15)


def test_f16_bf16_and_nvfp4_leaves():
    st, tb = MemoryBlobStore(), TribleBuilder()
    a = np.random.default_rng(0).standard_normal((8, 64)).astype(np.float32)
    e16 = put_array(st, tb, a.astype(np.float16))
    eb = put_array(st, tb, f32_to_bf16_bits(a), Elem.BF16)
    codes, scales, s2 = quantize_weight_nvfp4(a)
    m = put_fp4_tensor(st, tb, "experts.0.w13", codes, scales, s2, layer=3, expert=0)
    facts = tb.build()
    assert np.allclose(resolve(st, facts, e16).to_f32(), a, atol=2e-3)
    assert np.allclose(resolve(st, facts, eb).to_f32(), a, atol=2e-2)
    from mary_b200.format.model import load_module_leaf
    leaf = load_module_leaf(st, facts, m)
    assert leaf.elem == Elem.NVFP4 and leaf.dims == (8, 64)
    c2, sc2, g2 = leaf.fp4_parts()
    assert np.array_equal(c2, codes) and np.array_equal(sc2, scales) and g2 == pytest.approx(s2)
    assert np.abs(leaf.to_f32() - a).max() < 0.6


def test_root_id_depends_on_members_only_and_names_unique():
    st, tb = MemoryBlobStore(), TribleBuilder()
    m1 = put_tensor(st, tb, "a.weight", np.ones((2, 2), np.float32))
    m2 = put_tensor(st, tb, "b.weight", np.zeros((2,), np.float32))
    r1 = build_model_root(st, tb, [m1, m2], name="x", source="s1")
    r2 = build_model_root(st, TribleBuilder(), [m2, m1], name="other", source="s2")
    assert r1 == r2
    facts = tb.build()
    assert set(index_keymap(st, facts, r1)) == {"a.weight", "b.weight"}
    dup = put_tensor(st, tb, "a.weight", np.full((2, 2), 2, np.float32))
    r3 = build_model_root(st, tb, [m1, dup])
    with pytest.raises(LookupError, match="twice"):
        index_keymap(st, tb.build(), r3)


def test_selection_is_exact_cardinality_and_shards_merge():
    st, tb = MemoryBlobStore(), TribleBuilder()
    a = put_tensor(st, tb, "l0.w", np.ones((2, 2), np.float32))
    b = put_tensor(st, tb, "l1.w", np.zeros((2, 2), np.float32))
    ra = build_model_root(st, tb, [a], name="m", source="src")
    rb = build_model_root(st, tb, [b], name="m", source="src")
    facts = tb.build()
    with pytest.raises(SelectionError):
        select_model_root(st, facts, ModelSelector.only())
    with pytest.raises(SelectionError):
        select_model_root(st, facts, ModelSelector.by_name("absent"))
    assert select_model_root(st, facts, ModelSelector.by_root(ra)) == ra
    idx = SelectedModelIndex.from_snapshot(st, facts, ModelSelector.by_name("m"), shards=True)
    assert idx.names() == ["l0.w", "l1.w"] and idx.leaf("l1.w").dims == (2, 2)
    c = put_tensor(st, tb, "l0.w", np.full((2, 2), 7, np.float32))
    build_model_root(st, tb, [c], name="m", source="src")
    with pytest.raises(SelectionError, match="overlap"):
        SelectedModelIndex.from_snapshot(st, tb.build(), ModelSelector.by_name("m"), shards=True)


def test_experts_in_layers_is_a_query():
    st, tb = MemoryBlobStore(), TribleBuilder()
    rng = np.random.default_rng(0)
    mem = []
    for layer in range(3):
        for ex in range(2):
            c, s, g = quantize_weight_nvfp4(rng.standard_normal((4, 32)).astype(np.float32))
            mem.append(put_fp4_tensor(st, tb, f"layers.{layer}.experts.{ex}.w13", c, s, g, layer, ex))
    r = build_model_root(st, tb, mem)
    idx = SelectedModelIndex(st, tb.build(), [r])
    q = idx.experts_in_layers(1, 3)
    assert sorted(q) == [(1, 0), (1, 1), (2, 0), (2, 1)] and q[(2, 1)] == ["layers.2.experts.1.w13"]


def test_jsonfacts_roundtrip_exact():
    st, tb = MemoryBlobStore(), TribleBuilder()
    doc = {"hidden_size": 256, "eps": 1e-6, "one": 1.0, "flag": True, "none": None, "name": "gemma",
           "layers": ["a", "b", {"x": [1, 2.5, False]}], "nested": {"k": {"deep": -7}}, "big": 2 ** 62, "twins": [1, 1],
           "same": {"a": 1, "b": 1}}
    jsonfacts.save_document(st, tb, "config.json", doc)
    back = jsonfacts.load_document(st, tb.build(), "config.json")
    assert back == doc and list(back) == sorted(doc)          # canonical key order
    assert json.dumps(back, sort_keys=True) == json.dumps(doc, sort_keys=True)
    assert isinstance(back["one"], float) and isinstance(back["hidden_size"], int)
    with pytest.raises(ValueError):                           # an integer beyond 64 bits is refused, not rounded
        jsonfacts.save_document(st, TribleBuilder(), "x.json", {"big": 2 ** 70})
    # the reference's attribute ids (src/jsonfacts.rs:89-102), so either side reads the other's facts
    from mary_b200.format import schema as S
    assert S.JSON_KEY.hex().upper() == "051B238236962081B98F5D44BD9FA999" and S.JSON_INT.hex().upper() == "8657CA9A8F2864E21FA1793AF47AACA2"
    assert S.LORA_A.hex().upper() == "7CD7F0DC8BDA328735A22DF02B4B8828"
    with pytest.raises(LookupError):
        jsonfacts.load_document(st, tb.build(), "missing.json")


def _tiny_tokenizer_json():
    from tokenizers import Tokenizer, models, pre_tokenizers, decoders
    vocab = {"<unk>": 0, "h": 1, "e": 2, "l": 3, "o": 4, "he": 5, "ll": 6, "hell": 7, "hello": 8, "Ġ": 9, "w": 10}
    merges = [("h", "e"), ("l", "l"), ("he", "ll"), ("hell", "o")]
    tok = Tokenizer(models.BPE(vocab=vocab, merges=merges, unk_token="<unk>"))
    tok.pre_tokenizer = pre_tokenizers.ByteLevel(add_prefix_space=False)
    tok.decoder = decoders.ByteLevel()
    tok.add_special_tokens(["<bos>", "<turn|>"])
    return tok


def test_tokenizer_graph_roundtrip_and_build_without_json():
    tok = _tiny_tokenizer_json()
    st, tb = MemoryBlobStore(), TribleBuilder()
    tid = save_tokenizer_json(st, tb, "tiny", tok.to_str())
    facts = tb.build()
    assert load_tokenizer_json(st, facts, tid) == json.loads(tok.to_str())
    rebuilt = build_tokenizer(st, facts)
    for s in ("hello", "hello hello", "<bos>hello<turn|>"):
        assert rebuilt.encode(s).ids == tok.encode(s).ids
    # mutant 1: the facts of one merge entity vanish -> the strict reader refuses (a missing merge would change encodings silently)
    from mary_b200.format.tokenizer import MERGE, MERGE_RANK
    from mary_b200.pile.trible import r_genid, r_u256
    from mary_b200.pile import TribleSet
    merges = {r_genid(v) for _e, v in facts.with_attr(MERGE)}
    victim = [e for e, v in facts.with_attr(MERGE_RANK) if e in merges and r_u256(v) == 1][0]
    keep = [i for i, (e, _a, _v) in enumerate(facts) if e != victim]
    with pytest.raises((LookupError, ValueError)):
        build_tokenizer(st, TribleSet(facts.data[keep]))
    # mutant 2: the tokenizer no longer points at that merge -> a gap in the ranks, refused as well
    keep = [i for i, (_e, a, v) in enumerate(facts) if not (a == MERGE and r_genid(v) == victim)]
    with pytest.raises(ValueError, match="merge ranks"):
        build_tokenizer(st, TribleSet(facts.data[keep]))


def test_tokenizer_graph_uses_the_typed_node_forms_and_keeps_what_they_cannot_say():
    from mary_b200.format import tokenizer as T
    from mary_b200.pile.trible import r_genid
    doc = {"version": "1.0", "truncation": None, "padding": None,
           "added_tokens": [{"id": 0, "content": "[UNK]", "single_word": False, "lstrip": False, "rstrip": True, "normalized": False,
                             "special": True}],
           "normalizer": {"type": "Sequence", "normalizers": [
               {"type": "NFC"}, {"type": "Replace", "pattern": {"String": "  "}, "content": " "},
               {"type": "BertNormalizer", "clean_text": True, "handle_chinese_chars": True, "strip_accents": None, "lowercase": True},
               {"type": "NFC"}]},
           "pre_tokenizer": {"type": "Sequence", "pretokenizers": [
               {"type": "Split", "pattern": {"Regex": "\\d"}, "behavior": "Isolated", "invert": False},
               {"type": "Metaspace", "replacement": "\u2581", "prepend_scheme": "always", "split": True}]},
           "post_processor": None,
           "decoder": {"type": "WordPiece", "prefix": "##", "cleanup": True},
           "model": {"type": "WordPiece", "unk_token": "[UNK]", "continuing_subword_prefix": "##", "max_input_chars_per_word": 100,
                     "vocab": {"[UNK]": 0, "a": 1, "##b": 2}}}
    st, tb = MemoryBlobStore(), TribleBuilder()
    root = b"\x07" * 16
    tid = T.save_tokenizer_json(st, tb, "wp", doc, owner=root)
    facts = tb.build()
    assert T.load_tokenizer_json(st, facts, tid) == doc
    assert T.find_tokenizers(facts) == [tid]                      # the WordPiece DECODER node shares the tag but has no name
    assert r_genid(facts.one(root, T.TOKENIZER)) == tid
    norm = r_genid(facts.one(tid, T.NORMALIZER))
    kids = T.ordered_members(facts, norm)
    assert [T.ty.NFC in T.node_tags(facts, k) for k in kids] == [True, False, False, True] and len(set(kids)) == 4
    assert T.flag.PATTERN_IS_STRING in T.node_tags(facts, kids[1]) and T.flag.LOWERCASE in T.node_tags(facts, kids[2])
    pre = T.ordered_members(facts, r_genid(facts.one(tid, T.PRE_TOKENIZER)))
    assert T.ty.SPLIT in T.node_tags(facts, pre[0]) and T.ty.OPAQUE in T.node_tags(facts, pre[1])
    assert T.tokenizer_kind(facts, tid) == "WordPiece"
    # unigram pieces written from a SentencePiece table come back typed and build a working tokenizer
    st, tb = MemoryBlobStore(), TribleBuilder()
    pieces = [("<unk>", 0.0), ("\u2581a", -1.0), ("\u2581b", -1.5), ("b", -2.0)]
    uid = T.save_spm_unigram(st, tb, "spm", pieces)
    facts = tb.build()
    assert [(b.decode(), t) for b, _s, t in T.load_spm_pieces(st, facts, uid)] == [("<unk>", 2), ("\u2581a", 1), ("\u2581b", 1), ("b", 1)]
    assert T.has_add_prefix_space(facts, uid)
    assert T.build_tokenizer(st, facts, uid).encode("a b").ids == [1, 2]


def test_tiktoken_bpe_and_pile_roundtrip():
    ranks = {bytes([b]): b for b in range(256)}
    for i, t in enumerate([b"he", b"ll", b"hell", b"hello", b" w", b"or", b" wor"]):
        ranks[t] = 256 + i
    tk = TikToken(ranks, special={"<|im_end|>": 1000})
    ids = tk.encode("hello world<|im_end|>")
    assert ids[0] == ranks[b"hello"] and ids[-1] == 1000 and tk.decode(ids) == "hello world<|im_end|>"
    assert tk.decode(tk.encode("数字 123456 tests")) == "数字 123456 tests"
    st, tb = MemoryBlobStore(), TribleBuilder()
    tid = save_tiktoken(st, tb, "k3", ranks, tk._re.pattern, {"<|im_end|>": 1000})
    tk2 = load_tiktoken(st, tb.build(), tid)
    assert tk2.encode("hello world<|im_end|>") == ids


def test_safetensors_and_import_idempotent(tmp_path):
    rng = np.random.default_rng(0)
    tensors = {"model.a.weight": rng.standard_normal((4, 8)).astype(np.float32),
               "model.b.weight": rng.standard_normal((8,)).astype(np.float16),
               "model.ids": np.arange(4, dtype=np.int64)}
    d = tmp_path / "ckpt"
    d.mkdir()
    save_file(tensors, str(d / "model.safetensors"))
    (d / "config.json").write_text(json.dumps({"hidden_size": 8, "eps": 1e-5}))
    st = SafeTensors(str(d / "model.safetensors"))
    assert np.array_equal(st.array("model.a.weight"), tensors["model.a.weight"]) and st.f32("model.ids") is None
    from mary_b200.pile import signing_key_file
    key = signing_key_file(str(tmp_path / "k"))
    pile = Pile.open(str(tmp_path / "m.pile"))
    r1 = import_model_to_collection(pile, key, d, name="toy")
    size1 = len(read_model_pile(pile))
    r2 = import_model_to_collection(pile, key, d, name="toy")          # idempotent re-import
    facts = read_model_pile(pile)
    assert r1 == r2 and len(facts) == size1
    idx = SelectedModelIndex.from_snapshot(pile, facts)
    assert idx.names() == ["model.a.weight", "model.b.weight"]          # the int tensor was skipped
    assert load_config(pile, facts, r1) == {"hidden_size": 8, "eps": 1e-5}
    h = derive_half_root(pile, key, facts, r1, "bf16")
    facts = read_model_pile(pile)
    idx16 = SelectedModelIndex.from_snapshot(pile, facts, ModelSelector.by_root(h))
    assert idx16.leaf("model.a.weight").elem == Elem.BF16
    assert np.allclose(idx16.leaf("model.a.weight").to_f32(), tensors["model.a.weight"], atol=2e-2)
    pile.close()


def _write_gguf(path, tensors):
    def s(x):
        b = x.encode()
        return struct.pack("<Q", len(b)) + b
    kv = s("general.alignment") + struct.pack("<I", 4) + struct.pack("<I", 32)
    infos, data = b"", b""
    for name, (t, shape, raw) in tensors.items():
        pad = (-len(data)) % 32
        data += b"\x00" * pad
        infos += s(name) + struct.pack("<I", len(shape)) + b"".join(struct.pack("<Q", d) for d in reversed(shape))
        infos += struct.pack("<I", t) + struct.pack("<Q", len(data))
        data += raw
    head = b"GGUF" + struct.pack("<I", 3) + struct.pack("<Q", len(tensors)) + struct.pack("<Q", 1) + kv + infos
    head += b"\x00" * ((-len(head)) % 32)
    path.write_bytes(head + data)


def test_gguf_f32_f16_q8_q4(tmp_path):
    rng = np.random.default_rng(1)
    a = rng.standard_normal((2, 32)).astype(np.float32)
    d = (np.abs(a).max(1) / 127).astype(np.float16)
    q8 = np.rint(a / d.astype(np.float32)[:, None]).astype(np.int8)
    raw8 = b"".join(d[i].tobytes() + q8[i].tobytes() for i in range(2))
    d4 = (np.abs(a).max(1) / 7).astype(np.float16)
    q4 = np.clip(np.rint(a / d4.astype(np.float32)[:, None]) + 8, 0, 15).astype(np.uint8)
    raw4 = b"".join(d4[i].tobytes() + (q4[i, :16] | (q4[i, 16:] << 4)).tobytes() for i in range(2))
    p = tmp_path / "m.gguf"
    _write_gguf(p, {"f32": (0, (2, 32), a.tobytes()), "f16": (1, (2, 32), a.astype(np.float16).tobytes()),
                    "q8": (8, (2, 32), raw8), "q4": (2, (2, 32), raw4)})
    out = dict(iter_gguf(p))
    assert np.array_equal(out["f32"], a) and np.allclose(out["f16"], a, atol=2e-3)
    assert np.allclose(out["q8"], q8 * d.astype(np.float32)[:, None])
    assert np.allclose(out["q4"], (q4.astype(np.float32) - 8) * d4.astype(np.float32)[:, None])
    assert detect_format(p)[0] == "gguf"


def test_torch_pickle_reader_and_refusal(tmp_path):
    import torch
    sd = {"w": torch.arange(12, dtype=torch.float32).reshape(3, 4), "h": torch.ones(5, dtype=torch.float16),
          "t": torch.arange(6, dtype=torch.float32).reshape(2, 3).t(), "ids": torch.arange(3)}
    p = tmp_path / "m.pth"
    torch.save(sd, str(p))
    out = dict(iter_pickle(p))
    assert set(out) == {"w", "h", "t"}
    assert np.array_equal(out["w"], sd["w"].numpy()) and np.array_equal(out["t"], sd["t"].numpy())
    # a pickle that names an arbitrary callable is refused
    evil = tmp_path / "evil.pth"
    with zipfile.ZipFile(evil, "w") as z:
        z.writestr("archive/data.pkl", pickle.dumps(print))
    with pytest.raises(pickle.UnpicklingError):
        list(iter_pickle(evil))


def test_dyntensor_roundtrip_alignment_and_rejections():
    import struct
    import torch
    from mary_b200.format import dyntensor as dt
    rng = np.random.default_rng(0)
    for arr in (rng.standard_normal((3, 5)).astype(np.float32), rng.integers(-5, 5, (2, 3, 4)).astype(np.int64), np.float64(3.5).reshape(()),
                rng.integers(0, 255, (7,)).astype(np.uint8), np.array([True, False, True])):
        blob = dt.encode(arr)
        back, name = dt.decode(blob)
        assert back.dtype == arr.dtype and back.shape == arr.shape and np.array_equal(back, arr)
        n, shape, off = dt.header(blob)
        assert off % arr.dtype.itemsize == 0                         # data starts on the dtype's alignment
    t = torch.randn(4, 6).bfloat16()
    blob = dt.encode(t)
    assert dt.header(blob)[0] == "bf16" and torch.equal(dt.decode_torch(blob), t)
    assert struct.unpack_from("<I", blob)[0] == 0x534E5444 and blob[4] == 1 and blob[5] == 2       # magic, tag bf16 = 1, rank 2
    for bad in (b"abc", b"\\0" * 16, blob[:-2], struct.pack("<IBBH", dt.MAGIC, 99, 0, 0)):
        with pytest.raises(dt.DynTensorError):
            dt.header(bad)


def test_legacy_leaves_migrate_to_typed_tensors_keeping_entity_ids(tmp_path, capsys):
    import numpy as np
    from mary_b200.cli import mary
    from mary_b200.format import schema as S
    from mary_b200.format.leaf import put_array, put_leaf_legacy
    from mary_b200.format.migrate import loader_equiv, migrate_leaves
    from mary_b200.format.model import build_model_root, put_module
    from mary_b200.format.persist import publish_fragment, read_model_pile
    from mary_b200.pile import Pile, signing_key_file
    from mary_b200.pile.trible import TribleBuilder
    key = signing_key_file(str(tmp_path / "k"))
    src = Pile.open(str(tmp_path / "old.pile"))
    rng = np.random.default_rng(0)
    arrs = {"a.weight": rng.standard_normal((4, 6)).astype(np.float32), "b.weight": rng.standard_normal((3,)).astype(np.float16),
            "c.weight": rng.standard_normal((2, 2, 5)).astype(np.float32)}
    tb = TribleBuilder()
    leaves = {"a.weight": put_leaf_legacy(src, tb, arrs["a.weight"]), "b.weight": put_leaf_legacy(src, tb, arrs["b.weight"], f16=True),
              "c.weight": put_array(src, tb, arrs["c.weight"])}                      # one leaf is typed already
    members = [put_module(src, tb, n, leaves[n], arrs[n].ndim) for n in arrs]
    root = build_model_root(src, tb, members, name="old-model")
    publish_fragment(src, key, tb.build(), "legacy")
    dst = Pile.open(str(tmp_path / "new.pile"))
    st = migrate_leaves(src, dst, key)
    assert st["converted"] == 2 and st["passed_through"] == 0 and st["blobs_dropped"] == 4
    facts = read_model_pile(dst)
    for n, e in leaves.items():
        attrs = {a for a, _ in facts.of_entity(e)}                                 # same entity ids, no legacy facts left
        assert attrs and not ({S.DATA, S.DATA_F16, S.SHAPE} & attrs)
    assert loader_equiv(src, dst) == {"tensors": 3, "typed": 3}
    with pytest.raises(AssertionError, match="typed"):
        loader_equiv(dst, src)                                                       # the unconverted side must not pass as converted
    again = Pile.open(str(tmp_path / "again.pile"))
    assert migrate_leaves(dst, again, key)["converted"] == 0                         # idempotent
    src.close(), dst.close(), again.close()
    assert mary.main(["migrate", "--pile", str(tmp_path / "old.pile"), "--out", str(tmp_path / "cli.pile"), "--key", str(tmp_path / "k")]) == 0
    assert "converted=2" in capsys.readouterr().out
    assert mary.main(["equiv", "--pile", str(tmp_path / "old.pile"), "--other", str(tmp_path / "cli.pile")]) == 0
    assert mary.main(["equiv", "--pile", str(tmp_path / "cli.pile"), "--other", str(tmp_path / "old.pile")]) == 1


def test_quantised_leaves_round_trip_and_derive_a_sibling_root(tmp_path):
    import numpy as np
    from mary_b200.format import schema as S
    from mary_b200.format.leaf import LeafError
    from mary_b200.format.model import build_model_root, index_keymap, put_tensor
    from mary_b200.format.persist import publish_fragment, read_model_pile
    from mary_b200.format.qleaf import MARKER, dequantize_leaf_q, derive_q_root, load_leaf_q, module_weight_q, put_leaf_q
    from mary_b200.format.selection import model_roots
    from mary_b200.nn.q4 import QLinear, dequantize_q4, quantize_q4
    from mary_b200.pile import Pile, signing_key_file
    from mary_b200.pile.trible import TribleBuilder, r_shortstring, v_shortstring
    key = signing_key_file(str(tmp_path / "k"))
    pile = Pile.open(str(tmp_path / "m.pile"))
    rng = np.random.default_rng(0)
    w, b = rng.standard_normal((6, 64)).astype(np.float32), rng.standard_normal((6,)).astype(np.float32)
    tb = TribleBuilder()
    root = build_model_root(pile, tb, [put_tensor(pile, tb, "l.weight", w), put_tensor(pile, tb, "l.bias", b)], name="m")
    publish_fragment(pile, key, tb.build(), "f32")
    facts = read_model_pile(pile)
    for kind, tol in (("q4", 0.2), ("q8", 0.02)):
        qroot = derive_q_root(pile, key, facts, root, kind)
        f2 = read_model_pile(pile)
        assert qroot != root and r_shortstring(f2.one(qroot, S.QUANTIZATION)) == kind and len(model_roots(f2)) >= 2
        km = index_keymap(pile, f2, qroot)
        k2, packed, dims = module_weight_q(pile, f2, km["l.weight"])
        assert k2 == kind and dims == (6, 64) and module_weight_q(pile, f2, km["l.bias"]) is None       # vectors stay f32 leaves
        if kind == "q4":
            assert np.array_equal(packed, quantize_q4(w)) and np.array_equal(dequantize_q4(packed), dequantize_q4(quantize_q4(w)))
        from mary_b200.pile.trible import r_genid
        deq = dequantize_leaf_q(pile, f2, r_genid(f2.one(km["l.weight"], S.WEIGHT)))
        assert np.abs(deq - w).max() < tol * np.abs(w).max()
    # a marker this reader does not know is refused
    tb = TribleBuilder()
    e = put_leaf_q(pile, tb, w, "q4")
    bad = TribleBuilder()
    for ent, a, v in tb.build():
        bad.add(ent, a, v_shortstring("q4_0.v9") if a == S.FORMAT_MARKER else v)
    with pytest.raises(LeafError, match="format marker"):
        load_leaf_q(pile, bad.build(), e)
    with pytest.raises(LeafError):
        put_leaf_q(pile, TribleBuilder(), rng.standard_normal((4, 40)).astype(np.float32))
    assert MARKER["q8"] == "q8_0.v1"
    pile.close()


def test_filtered_component_import_and_split_half_single_index(tmp_pile):
    from mary_b200.format.persist import import_file_filtered_to_collection, load_split_index_from_pile, read_model_pile
    import tempfile, os
    pile, key = tmp_pile
    rng = np.random.default_rng(0)
    tensors = {"vision.patch.weight": rng.standard_normal((4, 8)).astype(np.float32), "vision.norm.weight": np.ones(8, np.float32),
               "text.embed.weight": rng.standard_normal((16, 8)).astype(np.float32)}
    d = tempfile.mkdtemp()
    f = os.path.join(d, "model.safetensors")
    save_file(tensors, f)
    r1 = import_file_filtered_to_collection(pile, key, f, "f16", source="hf/x", keep=lambda n: n.startswith("vision.") and n.endswith("patch.weight"),
                                            name="f16/vision")
    r2 = import_file_filtered_to_collection(pile, key, f, "f32", source="hf/x", keep=lambda n: n.endswith("norm.weight"), name="f32/vision")
    assert r1 != r2
    with pytest.raises(ValueError, match="selected no"):
        import_file_filtered_to_collection(pile, key, f, keep=lambda n: False)
    half, single = load_split_index_from_pile(pile, "f16/")
    assert set(half) == {"vision.patch.weight"} and set(single) == {"vision.norm.weight"}
    assert half["vision.patch.weight"].elem == Elem.F16 and single["vision.norm.weight"].elem == Elem.F32
    assert np.allclose(half["vision.patch.weight"].to_f32(), tensors["vision.patch.weight"], atol=2e-3)
    idx = SelectedModelIndex.from_snapshot(pile, read_model_pile(pile), ModelSelector.by_source("hf/x", "f16"))
    assert idx.names() == ["vision.patch.weight"]


def test_legacy_attribute_projection_is_additive_idempotent_and_counted():
    from mary_b200.format import legacy, schema as S
    from mary_b200.format.tokenizer import PIECE, TOKEN_ID
    from mary_b200.pile import TribleSet
    from mary_b200.pile.trible import v_u256
    aliases = legacy.legacy_model_attribute_aliases()
    assert len(aliases) == 45 and {a.label.split(".")[0] for a in aliases} == {"format", "gemma_lora", "tokenizer"}
    by_label = {a.label: a for a in aliases}
    assert by_label["format.index"].historical == S.INDEX and by_label["tokenizer.piece"].historical == PIECE
    tok = _tiny_tokenizer_json()
    st, tb = MemoryBlobStore(), TribleBuilder()
    tid = save_tokenizer_json(st, tb, "tiny", tok.to_str())
    other = b"\x09" * 16
    tb.add(tid, other, v_u256(7))                                   # an attribute outside the table
    facts = tb.build()
    p = legacy.project_legacy_model_attributes(facts)
    assert p.input_facts == len(facts) and p.aliases_added == p.source_facts > 0 and len(p.facts) == len(facts) + p.aliases_added
    assert all(tuple(r) in {tuple(x) for x in p.facts.data.tolist()} for r in facts.data.tolist()[:50])       # nothing dropped
    cnt = {c.alias.label: c for c in p.mappings}
    assert cnt["tokenizer.token_id"].source_facts == len(facts.with_attr(TOKEN_ID)) and cnt["format.data"].source_facts == 0
    assert not p.facts.with_attr(legacy.anchored_id("00" * 16, "U256BE")) and len(p.facts.with_attr(other)) == 1
    again = legacy.project_legacy_model_attributes(p.facts)
    assert again.aliases_added == 0 and again.facts == p.facts and sum(c.aliases_already_present for c in again.mappings) == p.aliases_added
    # a fact set that carries ONLY derived ids becomes readable here through the opposite projection
    canon = {a.historical: a.canonical for a in aliases}
    rows = [e + canon.get(a, a) + v for e, a, v in facts]
    only_new = TribleSet.from_tribles(rows)
    assert not only_new.with_attr(TOKEN_ID)
    back = legacy.project_to_literal(only_new).facts
    assert build_tokenizer(st, back).encode("hello hello").ids == tok.encode("hello hello").ids
