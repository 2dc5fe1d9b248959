"""The in-process seams (chat engine, say, speak) on tiny random models."""
import numpy as np
import torch

from mary_b200.api import local
from mary_b200.api.local import LocalChatTurn as Turn, LocalRole as R


def test_chat_template_folds_system_turns_and_splits_channels():
    turns = [Turn(R.SYSTEM, "be brief"), Turn(R.USER, "hi"), Turn(R.ASSISTANT, "hello"), Turn(R.USER, "bye"), Turn(R.SYSTEM, "tail")]
    s = local.build_chat(turns)
    assert s == ("<bos><|turn>user\nbe brief\nhi<turn|>\n<|turn>model\nhello<turn|>\n<|turn>user\nbye<turn|>\n<|turn>user\ntail\n<turn|>\n<|turn>model\n")
    raw = "<|channel>thought<channel|>let me think<|channel>final<channel|>42\nmore<turn|>"
    text, why = local.split_channels(raw)
    assert text == "42\nmore" and why == "let me think"
    assert local.apply_stop(text, ["\n", "zzz"]) == "42" and local.split_channels("plain<turn|>") == ("plain", None)
    assert local.split_channels("<|channel>only one") == ("only one", None)


def test_gemma_engine_generates_through_the_seam():
    from tokenizers import Tokenizer, models, pre_tokenizers
    from mary_b200.models.gemma4 import Gemma4Model, tiny_config
    from mary_b200.models.gemma4.lm import GemmaLM
    from mary_b200.models.gemma4.weights import init_random_
    torch.manual_seed(0)
    cfg = tiny_config()
    m = Gemma4Model(cfg)
    init_random_(m, 0)
    vocab = {f"t{i}": i for i in range(cfg.vocab_size)}
    vocab.update({"<bos>": 2})
    tok = Tokenizer(models.WordLevel({**{k: v for k, v in vocab.items()}, "[UNK]": 3}, unk_token="[UNK]"))
    tok.pre_tokenizer = pre_tokenizers.Whitespace()
    lm = GemmaLM(m, tokenizer=tok)
    g = local.GemmaEngine(lm).generate([Turn(R.USER, "t5 t6 t7")], local.LocalGenParams(max_tokens=5))
    assert g.completion_tokens == 5 and g.prompt_tokens > 0 and isinstance(g.text, str)


def test_say_voice_synthesises_with_weights_loaded_once():
    from mary_b200.api.say import Voice
    from mary_b200.cli.families import _random_init
    from mary_b200.models.f5 import DiT, F5Config, Vocos, VocosConfig
    c = F5Config.tiny()
    dit = _random_init(DiT(c))
    voc = _random_init(Vocos(VocosConfig(n_mels=c.n_mels, dim=16, ffn=32, layers=1, n_fft=64, hop=16)))
    ref = np.sin(np.arange(4000) * 0.05).astype(np.float32)
    v = Voice(dit, voc, ref, 16000, "hello", n_fft=64, hop=16, nfe=2)
    a, b = v.synthesize("good day", seed=1), v.synthesize("good day", seed=1)
    assert a.shape == b.shape and a.shape[0] > 0 and np.array_equal(a, b) and np.isfinite(a).all()
    assert v.synthesize("a much longer sentence than before", seed=1).shape[0] > a.shape[0]


def test_speak_streams_one_chunk_per_frame():
    from mary_b200.api.speak import Speaker
    from mary_b200.models.codec.mimi import MimiCodec, MimiConfig
    from mary_b200.models.codec.mimi import init_random_ as init_codec
    from mary_b200.models.qwen3tts.model import CodePredictor, Qwen3TTSConfig, Talker
    from mary_b200.models.qwen3tts.model import init_random_ as init_tts
    cfg = Qwen3TTSConfig.tiny()
    talker, pred = Talker(cfg), CodePredictor(cfg)
    init_tts(talker, pred, 0)
    codec = MimiCodec(MimiConfig.tiny())
    init_codec(codec, 0)
    sp = Speaker(talker, pred, codec, cfg)
    chunks = list(sp.synthesize_stream([5, 6, 7, 8, 9, 10], max_frames=4, seed=3))
    assert 1 <= len(chunks) <= 4 and all(c.ndim == 1 and c.size > 0 for c in chunks)
    assert np.array_equal(np.concatenate(chunks), sp.synthesize([5, 6, 7, 8, 9, 10], max_frames=4, seed=3))
