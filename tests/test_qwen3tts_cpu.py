"""Qwen3-TTS frame generator on a tiny configuration: the predictor's cached steps equal one uncached pass, the logits
processor follows the reference rules, and the frame loop is deterministic, streams and stops."""
import numpy as np
import torch

from mary_b200 import ops
from mary_b200.models.qwen3tts import (CodePredictor, Qwen3TTSConfig, SamplingParams, Talker, generate_frames, init_random_,
                                       process_talker_logits)
from mary_b200.runtime.batch import BatchMeta
from mary_b200.runtime.kv_cache import PagedKVCache


def _models(seed=0):
    cfg = Qwen3TTSConfig.tiny()
    t, p = Talker(cfg), CodePredictor(cfg)
    init_random_(t, p, seed, std=0.2)
    return cfg, t, p


def test_predictor_cached_steps_equal_full_recompute():
    cfg, t, p = _models()
    torch.manual_seed(1)
    h, e0 = torch.randn(cfg.talker_hidden), torch.randn(cfg.talker_hidden)
    with torch.no_grad():
        codes, esum = p.predict_frame(h, e0, temperature=0.0)
        # uncached: feed the whole prefix again for every codebook
        xs = [p.project(torch.stack([h, e0]))]
        want = []
        for i in range(cfg.num_code_groups - 1):
            x = torch.cat(xs)
            spec = p.stack.kv_spec()
            cache = PagedKVCache(spec["num_layers"], 3, 16, spec["kv_heads"], spec["head_dim"], dtype=torch.float32)
            cache.alloc.extend(0, x.shape[0])
            table, lens = cache.alloc.page_table([0])
            hid = p.stack.hidden_from_embeds(x, BatchMeta.build([x.shape[0]], lens, table, 16), cache)[-1:]
            tok = int(ops.linear(hid, p.heads[i]).argmax())
            want.append(tok)
            xs.append(p.project(ops.embed(torch.tensor([tok], dtype=torch.int32), p.embeddings[i])))
    assert codes.tolist() == want
    assert torch.allclose(esum, p.accumulate_frame(want), atol=1e-5)


def test_logits_processing_rules():
    cfg = Qwen3TTSConfig.tiny()
    lg = torch.linspace(-1, 1, cfg.codec_vocab)
    out = process_talker_logits(lg, [3, 60, 3], 0, 2.0, cfg)
    assert out[3] == lg[3] * 2.0 and out[60] == lg[60] / 2.0          # negative logits are multiplied, positive divided
    assert out[cfg.codec_eos] == float("-inf")                          # no end of speech in the first two frames
    assert torch.isinf(out[cfg.pred_vocab:]).all()
    out2 = process_talker_logits(lg, [], 2, 2.0, cfg)
    assert out2[cfg.codec_eos] == lg[cfg.codec_eos]
    assert torch.isinf(out2[cfg.pred_vocab:cfg.codec_eos]).all() and torch.isinf(out2[cfg.codec_eos + 1:]).all()
    assert torch.equal(out2[:cfg.pred_vocab], lg[:cfg.pred_vocab])


def test_frame_loop_is_deterministic_streams_and_stops():
    cfg, t, p = _models(3)
    text = torch.randint(0, cfg.text_vocab, (9,), dtype=torch.int32)
    with torch.no_grad():
        prefill = t.embed_text(text[:6]) + t.embed_codec(torch.full((6,), cfg.codec_pad, dtype=torch.int32))
        trailing = t.embed_text(text[6:])
        pad = t.embed_text(torch.tensor([0], dtype=torch.int32))[0]
    params = SamplingParams(max_frames=7, seed=5)
    a = generate_frames(t, p, prefill, trailing, pad, params)
    b = generate_frames(t, p, prefill, trailing, pad, params)
    assert a.shape[1] == cfg.num_code_groups and 1 <= a.shape[0] <= 7 and np.array_equal(a, b)
    assert (a[:, 0] < cfg.codec_vocab).all() and (a[:, 1:] < cfg.pred_vocab).all() and (a >= 0).all()
    c = generate_frames(t, p, prefill, trailing, pad, SamplingParams(max_frames=7, seed=6))
    assert a.shape != c.shape or not np.array_equal(a, c)                # another seed, another utterance
    seen = []
    d = generate_frames(t, p, prefill, trailing, pad, params, on_frame=lambda f: (seen.append(f), len(seen) < 3)[1])
    assert len(seen) == min(3, a.shape[0]) and d.shape[0] == min(2, a.shape[0])
    assert np.array_equal(d, a[:d.shape[0]])
