"""Packaged voice prompts (.pt reader that never runs the pickle), the SentencePiece unigram tokenizer and the system-prompt flow."""
import io

import pytest
import torch

from mary_b200.format import torch_pt
from mary_b200.format.spm import BYTE, NORMAL, SpmTokenizer, parse_model
from mary_b200.models.moshi import LmGen, MoshiConfig, Prompt, VoicePrompt, init_random_, wrap_with_system_tags


def _saved(obj) -> bytes:
    buf = io.BytesIO()
    torch.save(obj, buf)
    return buf.getvalue()


def test_pt_reader_equals_torch_load_and_refuses_code():
    g = torch.Generator().manual_seed(0)
    obj = {"embeddings": torch.randn(5, 1, 1, 8, generator=g).bfloat16(), "cache": torch.randint(0, 9, (1, 5, 4), generator=g),
           "nested": [torch.randn(3, 4, generator=g).t(), (torch.arange(6, dtype=torch.int32)[2:], 1.5, "s", None, True)],
           "half": torch.randn(2, 3, generator=g).half(), "empty": torch.zeros(0, 3), "big": 1 << 40}
    got = torch_pt.load_pt(_saved(obj))
    want = torch.load(io.BytesIO(_saved(obj)))

    def same(a, b):
        if isinstance(a, torch.Tensor):
            assert a.dtype == b.dtype and a.shape == b.shape and torch.equal(a, b)
        elif isinstance(a, (list, tuple)):
            assert type(a) is type(b) and len(a) == len(b)
            for x, y in zip(a, b):
                same(x, y)
        else:
            assert a == b
    assert got.keys() == want.keys()
    for k in want:
        same(got[k], want[k])
    # a pickle that names any other callable is refused, not run
    import pickle

    class Evil:
        def __reduce__(self):
            return (print, ("ran",))
    with pytest.raises(ValueError, match="refusing to call|unsupported"):
        torch_pt.unpickle(pickle.dumps({"x": Evil()}, protocol=2))
    # deflated entries and truncated archives are refused
    import zipfile
    z = io.BytesIO()
    with zipfile.ZipFile(z, "w", zipfile.ZIP_DEFLATED) as f:
        f.writestr("a/data.pkl", b"x" * 100)
    with pytest.raises(ValueError, match="STORED"):
        torch_pt.zip_entries(z.getvalue())
    with pytest.raises(ValueError):
        torch_pt.load_pt(_saved(obj)[:200])


def _spm_model(vocab=400) -> bytes:
    import sentencepiece as spm
    corpus = ["the quick brown fox jumps over the lazy dog", "hello world hello there", "a system prompt that is nice",
              "Grüße aus München", "be nice to the user and answer briefly", "numbers 123 456 and punctuation (a) [b] {c} <d>",
              "the system said hello to the world"] * 20
    out = io.BytesIO()
    spm.SentencePieceTrainer.train(sentence_iterator=iter(corpus), model_writer=out, vocab_size=vocab, model_type="unigram", byte_fallback=True,
                                   normalization_rule_name="identity", remove_extra_whitespaces=False, add_dummy_prefix=True, pad_id=3,
                                   character_coverage=1.0, hard_vocab_limit=False, minloglevel=2)
    return out.getvalue()


BATTERY = ["Hello, world!", "The quick brown fox.", "a  b   c", "tab\tand\nnewline", "Grüße aus München", "日本語のテスト", "Привет мир",
           "emoji 😀🎉 test", "<system> be nice <system>", "mixed 混合 text 123", "punctuation: (a) [b] {c} <d>", " leading", "trailing ", "🚀"]


def test_spm_unigram_encodes_like_sentencepiece_and_round_trips():
    import sentencepiece as spm
    data = _spm_model()
    pieces, prefix, fallback = parse_model(data)
    assert prefix and fallback and sum(t == BYTE for _, _, t in pieces) == 256 and any(t == NORMAL for _, _, t in pieces)
    tok = SpmTokenizer(pieces, prefix)
    oracle = spm.SentencePieceProcessor(model_proto=data)
    assert tok.vocab_size() == oracle.get_piece_size()
    for text in BATTERY:
        ids = tok.encode(text)
        assert ids == oracle.encode(text), text
        assert tok.decode(ids) == text == oracle.decode(ids)
    assert tok.encode("") == []
    ids = tok.encode("😀")
    assert all(tok.is_byte[i] for i in ids[1:]) and b"".join(tok.piece_bytes(i) for i in ids[1:]) == "😀".encode()
    # mutant: with one piece's score raised the segmentation changes (the comparison can fail)
    k = next(i for i, (p, _s, t) in enumerate(pieces) if t == NORMAL and len(p) == 1 and p.isalpha())
    worse = list(pieces)
    worse[k] = (worse[k][0], 50.0, NORMAL)
    assert any(SpmTokenizer(worse, prefix).encode(t) != oracle.encode(t) for t in BATTERY)
    # a model this implementation does not restate is refused by name
    with pytest.raises(ValueError, match="USER_DEFINED"):
        SpmTokenizer(pieces + [(b"<x>", 0.0, 4)], prefix)
    # the typed piece table of a pile gives the same tokenizer back
    from mary_b200.format.tokenizer import has_add_prefix_space, load_spm_pieces, save_spm_unigram
    from mary_b200.pile import MemoryBlobStore, TribleBuilder
    st, tb = MemoryBlobStore(), TribleBuilder()
    tid = save_spm_unigram(st, tb, "spm", pieces, add_dummy_prefix=prefix, byte_fallback=fallback)
    facts = tb.build()
    again = SpmTokenizer(load_spm_pieces(st, facts, tid), has_add_prefix_space(facts, tid))
    assert all(again.encode(t) == tok.encode(t) for t in BATTERY)


def test_voice_prompt_package_and_the_prompt_flow_through_the_model(tmp_path):
    c = MoshiConfig.tiny()
    g = torch.Generator().manual_seed(1)
    ring = c.max_delay + 3
    voice = VoicePrompt(torch.randn(4, c.dim, generator=g), torch.randint(0, c.card, (c.num_streams, ring), generator=g))
    for dt in (torch.float32, torch.bfloat16):
        path = tmp_path / f"v_{dt}.pt".replace("torch.", "")
        voice.save(path, dt)
        back = VoicePrompt.load(path, c)
        assert back.n_frames == 4 and torch.equal(back.cache, voice.cache)
        assert torch.equal(back.embeddings, voice.embeddings.to(dt).float())             # bf16 widens exactly
    with pytest.raises(ValueError, match="embeddings"):
        VoicePrompt.load(_saved({"embeddings": torch.zeros(4, c.dim), "cache": voice.cache[None]}), c)
    with pytest.raises(ValueError, match="cache"):
        VoicePrompt.load(_saved({"embeddings": torch.zeros(4, 1, 1, c.dim), "cache": voice.cache[None, :, :2]}), c)
    assert wrap_with_system_tags("  be nice ") == "<system> be nice <system>"
    assert wrap_with_system_tags("<system> x <system>") == "<system> x <system>"

    tok = SpmTokenizer(*parse_model(_spm_model())[:2])
    prompt = Prompt.build(tmp_path / "v_float32.pt", tok, "be nice", c)
    prompt.text_tokens = [t % c.text_card for t in prompt.text_tokens]                  # the tiny model has a 50-entry text table
    prompt.silence_frames = 2
    assert prompt.total_steps() == 4 + 4 + len(prompt.text_tokens)
    sine, silence = [1, 2], [3, 4]

    def run(replay):
        m = LmGen(c)
        init_random_(m, 0)
        m.reset_session()
        replay(m)
        return m, [m.step(user_audio=[5, 6]) for _ in range(3)]
    m1, out1 = run(lambda m: m.run_prompt(prompt, sine, silence))
    assert m1.pos == prompt.total_steps() + 3 and all(o is not None and len(o) == c.num_streams for o in out1)
    _, out2 = run(lambda m: m.run_prompt(prompt, sine, silence))
    assert out1 == out2                                                                 # deterministic
    # the replayed embeddings reach the model: another voice changes what follows
    other = Prompt(VoicePrompt(voice.embeddings * -1.0, voice.cache), prompt.text_tokens, 2)
    _, out3 = run(lambda m: m.run_prompt(other, sine, silence))
    assert out3 != out1
    # the snapshot replaces the ring wholesale and leaves offset and flags alone
    m = LmGen(c)
    init_random_(m, 0)
    m.prompt_voice(voice)
    assert m.stream.cache == voice.cache.tolist() and m.stream.offset == 5 and m.pos == 4
    with pytest.raises(ValueError):
        m.stream.overwrite([[0] * ring] * 2)
    with pytest.raises(ValueError):
        m.prompt_silence(1)                                                             # the 12.5 Hz codec's tokens do not fit a 24-entry table
