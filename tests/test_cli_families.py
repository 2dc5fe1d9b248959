"""The speech / vision / image entry points end to end on tiny random models, and on a model imported into a pile by name."""
import numpy as np
import torch

from mary_b200.cli import families


def test_say_listen_embed_imagine_act_on_random_tiny_models(tmp_path, capsys):
    sr = 16000
    t = np.arange(sr // 2) / sr
    families.write_wav(str(tmp_path / "ref.wav"), 0.3 * np.sin(2 * np.pi * 220 * t), sr)
    x, got_sr = families.read_wav(str(tmp_path / "ref.wav"))
    assert got_sr == sr and abs(x.max() - 0.3) < 1e-3

    assert families.main(["say", "--random", "--ref-wav", str(tmp_path / "ref.wav"), "--ref-text", "hello", "--text", "hello there", "--out",
                          str(tmp_path / "o.wav"), "--nfe", "2"]) == 0
    y, _ = families.read_wav(str(tmp_path / "o.wav"))
    n_ref = sr // 2 // 16 + 1
    assert len(y) == int(n_ref * 11 / 5) * 16                      # frames scale with the character ratio; 16 samples per frame

    assert families.main(["listen", "--random", "--wav", str(tmp_path / "ref.wav"), "--chunk", "2"]) == 0
    toks = capsys.readouterr().out.strip().splitlines()[-1].split(",")
    assert len(toks) == (sr // 2 // 160) // 8 // 2 * 2 or len(toks) >= 4

    np.save(tmp_path / "img.npy", np.random.default_rng(0).random((3, 40, 48), dtype=np.float32))
    for kind, extra in (("clip", ["--image", str(tmp_path / "img.npy")]), ("siglip", ["--ids", "1,2,3"]), ("nomic", ["--ids", "4,5,6,7"]),
                        ("nomic-vision", ["--image", str(tmp_path / "img.npy")])):
        assert families.main(["embed", "--random", "--kind", kind] + extra) == 0
        v = np.array(capsys.readouterr().out.split(), dtype=np.float64)
        assert abs(np.linalg.norm(v) - 1.0) < 1e-4

    np.save(tmp_path / "feat.npy", np.random.default_rng(1).standard_normal((5, 24)).astype(np.float32))
    assert families.main(["imagine", "--random", "--features", str(tmp_path / "feat.npy"), "--out", str(tmp_path / "im.npy"), "--height", "16",
                          "--width", "24", "--steps", "2"]) == 0
    assert np.load(tmp_path / "im.npy").shape == (3, 16, 24)
    capsys.readouterr()

    np.save(tmp_path / "cam.npy", np.random.default_rng(2).random((3, 32, 32), dtype=np.float32) * 2 - 1)
    np.save(tmp_path / "state.npy", np.zeros(8, dtype=np.float32))
    assert families.main(["act", "--random", "--image", str(tmp_path / "cam.npy"), "--ids", "3,4,5", "--state", str(tmp_path / "state.npy")]) == 0
    rows = capsys.readouterr().out.strip().splitlines()
    assert len(rows) == 6 and len(rows[0].split()) == 3


def test_embedder_loaded_from_a_pile_by_name(tmp_path, capsys):
    from mary_b200.cli import mary
    from mary_b200.format.safetensors import save_file
    from mary_b200.models.embed import NomicConfig, NomicTextEmbedder
    c = NomicConfig.tiny()
    src = families._random_init(NomicTextEmbedder(c), seed=3)
    sd = {"embeddings.word_embeddings.weight": src.tok, "embeddings.token_type_embeddings.weight": src.typ,
          "embeddings.LayerNorm.weight": src.emb_ln_w, "embeddings.LayerNorm.bias": src.emb_ln_b}
    H = c.hidden
    for i, L in enumerate(src.layers):
        p = f"layers.{i}."
        q, k, v = L.w_qkv.split(H, 0)
        g, u = L.w_gu.split(c.ffn, 0)
        sd.update({p + "self_attn.q_proj.weight": q, p + "self_attn.k_proj.weight": k, p + "self_attn.v_proj.weight": v, p + "self_attn.o_proj.weight": L.w_o,
                   p + "mlp.gate_proj.weight": g, p + "mlp.up_proj.weight": u, p + "mlp.down_proj.weight": L.w_down,
                   p + "post_attention_layernorm.weight": L.ln1_w, p + "post_attention_layernorm.bias": L.ln1_b,
                   p + "post_mlp_layernorm.weight": L.ln2_w, p + "post_mlp_layernorm.bias": L.ln2_b})
    save_file({k: v.detach().contiguous().numpy() for k, v in sd.items()}, str(tmp_path / "model.safetensors"))
    assert mary.main(["import", str(tmp_path / "model.safetensors"), "--pile", str(tmp_path / "p.pile"), "--key", str(tmp_path / "k"), "--name", "nomic-tiny"]) == 0
    capsys.readouterr()
    # the tiny geometry has no preset: load through the same helper the CLI uses
    dst = NomicTextEmbedder(c)
    from mary_b200.models.embed import nomic
    nomic.load_into(dst, families._loader(str(tmp_path / "p.pile"), "nomic-tiny"))
    ids = torch.tensor([[4, 5, 6, 7]])
    with torch.no_grad():
        assert torch.allclose(dst.embed_text(ids), src.embed_text(ids), atol=1e-6)


def test_hear_and_speak_on_random_tiny_models(tmp_path, capsys):
    sr = 16000
    t = np.arange(sr // 2) / sr
    families.write_wav(str(tmp_path / "q.wav"), 0.3 * np.sin(2 * np.pi * 330 * t), sr)
    assert families.main(["hear", "--random", "--wav", str(tmp_path / "q.wav"), "--ids", "2,7", "--ids-after", "9", "--max-new", "5"]) == 0
    cap = capsys.readouterr()
    assert len(cap.out.strip().split(",")) == 5 and "audio tokens" in cap.err
    assert families.main(["speak", "--random", "--ids", "5,6,7,8,9,10,11,12", "--out", str(tmp_path / "s.wav"), "--max-frames", "5"]) == 0
    y, rate = families.read_wav(str(tmp_path / "s.wav"))
    n_frames = int(capsys.readouterr().out.split()[0])
    assert rate == 24000 and len(y) == n_frames * 16 and 1 <= n_frames <= 5          # tiny codec: 16 samples per frame


def test_converse_streams_user_audio_through_codec_and_speech_lm(tmp_path, capsys):
    sr = 24000
    t = np.arange(16 * 12) / sr                                   # 12 codec frames of the tiny codec
    families.write_wav(str(tmp_path / "u.wav"), 0.3 * np.sin(2 * np.pi * 440 * t), sr)
    assert families.main(["converse", "--random", "--wav", str(tmp_path / "u.wav"), "--out", str(tmp_path / "a.wav")]) == 0
    toks = capsys.readouterr().out.strip().split(",")
    y, _ = families.read_wav(str(tmp_path / "a.wav"))
    assert 8 <= len(toks) <= 12 and len(y) == len(toks) * 16


def test_say_serve_answers_one_request_per_line_with_warm_weights(tmp_path, capsys, monkeypatch):
    import io
    import sys
    sr = 16000
    t = np.arange(sr // 2) / sr
    families.write_wav(str(tmp_path / "ref.wav"), 0.3 * np.sin(2 * np.pi * 220 * t), sr)
    reqs = f"{tmp_path / 'a.wav'}\thello there\nnot a request\n\n{tmp_path / 'b.wav'}\thi\n"
    monkeypatch.setattr(sys, "stdin", io.StringIO(reqs))
    assert families.main(["say", "--random", "--serve", "--ref-wav", str(tmp_path / "ref.wav"), "--ref-text", "hello", "--nfe", "2"]) == 0
    out = capsys.readouterr().out.splitlines()
    assert out[0] == "ready" and out[1].startswith(str(tmp_path / "a.wav")) and "bad request" in out[2] and out[3].startswith(str(tmp_path / "b.wav"))
    a, _ = families.read_wav(str(tmp_path / "a.wav"))
    b, _ = families.read_wav(str(tmp_path / "b.wav"))
    assert len(a) > len(b) > 0                                      # duration follows the character ratio


def test_rank_orders_documents_by_cosine_and_puts_the_identical_text_first(capsys):
    assert families.main(["rank", "--random", "--kind", "nomic", "--queries", "4,5,6;9,8", "--docs", "1,2,3;4,5,6;9,8"]) == 0
    lines = capsys.readouterr().out.strip().splitlines()
    assert lines[0].startswith("query 0: 1:1.0000") and lines[1].startswith("query 1: 2:1.0000")
    sims = [float(x.split(":")[1]) for x in lines[0].split()[2:]]
    assert sims == sorted(sims, reverse=True)
