"""Entry points of the speech, vision and image families, all loading weights from a pile by model name:

    families say       --pile P --model f5 --vocoder vocos --ref-wav r.wav --ref-text "..." --text "..." --out o.wav   (``say`` / ``say_serve``)
    families listen    --pile P --model voxtral --wav a.wav [--delay 6]                                                  (``voxtral_listen``)
    families embed     --pile P --model clip|siglip|nomic --kind clip|siglip|nomic|nomic-vision [--image i.npy] [--ids 1,2,3]         (``local_demo``, ``embed_persist``)
    families imagine   --pile P --transformer T --vae V --features f.npy --out img.npy [--steps 4] [--seed 0]            (the FLUX.2 pipeline)
    families rank      --pile P --model nomic --kind nomic --queries "1,2;3,4" --docs "5,6;1,2"                             (``nomic_semantic_probe``, ``embed_bakeoff``)
    families act       --pile P --model smolvla --image i.npy --ids 1,2,3 --state s.npy                                  (``smolvla_infer``)
    families hear      --pile P --model gemma-audio --wav a.wav [--ids 2,.. --ids-after ..]                              (``gemma_hear`` / ``gemma_listen``)
    families speak     --pile P --model qwen3tts --codec codec --ids 5,6,7 --out o.wav                                                            (``speak`` / ``qwen3tts_say|stream``)
    families converse  --pile P --model moshi --codec mimi --wav in.wav --out agent.wav                                                       (``personaplex_listen``)

Checkpoints get into a pile with ``mary import`` (the reference's ``*_persist`` importers); ``--random`` instead builds the tiny
configuration with random weights, which is what the tests drive.  Audio is read and written as 16-bit mono WAV with the standard
library; images and feature matrices as ``.npy``."""
from __future__ import annotations

import argparse
import sys
import wave as wavlib

import numpy as np
import torch

from ..format.persist import read_model_pile
from ..format.selection import ModelSelector, SelectedModelIndex
from ..nn.weight_loader import WeightLoader
from ..pile import Pile


def _loader(pile_path: str, name: str):
    pile = Pile.open(pile_path, create=False)
    facts = read_model_pile(pile)
    ld = WeightLoader.from_pile(SelectedModelIndex.from_snapshot(pile, facts, ModelSelector.by_name(name)))
    ld._pile = pile                     # leaf views alias the mapping
    return ld


def read_wav(path: str) -> tuple[np.ndarray, int]:
    with wavlib.open(path, "rb") as f:
        assert f.getsampwidth() == 2, "16-bit PCM expected"
        x = np.frombuffer(f.readframes(f.getnframes()), dtype="<i2").astype(np.float32) / 32768.0
        if f.getnchannels() > 1:
            x = x.reshape(-1, f.getnchannels()).mean(1)
        return x, f.getframerate()


def write_wav(path: str, x, sr: int) -> None:
    pcm = (np.clip(np.asarray(x, dtype=np.float32), -1.0, 1.0) * 32767.0).astype("<i2")
    with wavlib.open(path, "wb") as f:
        f.setnchannels(1), f.setsampwidth(2), f.setframerate(sr)
        f.writeframes(pcm.tobytes())


def _random_init(m, seed=0, std=0.05):
    g = torch.Generator().manual_seed(seed)
    for n, p in m.named_parameters():
        if p.dim() == 1:
            p.data.fill_(0.0 if n.split(".")[-1].endswith(("_b", "bias")) or n.split(".")[-1].startswith("b") else 1.0)
        else:
            p.data.normal_(0.0, std, generator=g)
    return m


def cmd_say(a) -> int:
    from ..models.f5 import CFM, DiT, F5Config, Vocos, VocosConfig, mel_spectrogram
    from ..models.f5 import dit as f5
    if a.random:
        c = F5Config.tiny()
        dit, voc = _random_init(DiT(c)), _random_init(Vocos(VocosConfig(n_mels=c.n_mels, dim=16, ffn=32, layers=1, n_fft=64, hop=16)))
        n_fft, hop = 64, 16
    else:
        dit, voc = DiT(F5Config()), Vocos(VocosConfig())
        f5.load_into(dit, _loader(a.pile, a.model))
        from ..models.f5.vocos import load_into as load_vocos
        load_vocos(voc, _loader(a.pile, a.vocoder))
        n_fft, hop = 1024, 256
    wav, sr = read_wav(a.ref_wav)
    ref = mel_spectrogram(torch.from_numpy(wav), n_mels=dit.c.n_mels, n_fft=n_fft, hop=hop, sr=sr).T.contiguous()
    cfm = CFM(dit, nfe=a.nfe, cfg_strength=a.cfg)

    def synth(text: str, out_path: str, seed: int) -> float:
        chars = [ord(ch) % (dit.c.text_vocab - 1) for ch in a.ref_text + " " + text]          # byte-level ids when the pile holds no vocabulary
        # duration rule of the reference front end: target frames = reference frames * (target characters / reference characters)
        total = ref.shape[0] + max(1, int(ref.shape[0] * len(text) / max(1, len(a.ref_text)) / a.speed))
        mel = cfm.sample(ref, chars, total, generator=torch.Generator().manual_seed(seed))
        out = voc(mel[ref.shape[0]:].T.contiguous())
        write_wav(out_path, out.numpy(), sr)
        return out.shape[0] / sr
    if not a.serve:
        print(f"{synth(a.text, a.out, a.seed):.2f} s of audio -> {a.out}")
        return 0
    # warm server (``say_serve``): weights, vocoder, mel front end and the reference voice are loaded ONCE; every line of standard
    # input is one request ``<out.wav>\t<text>``; the per-request time is printed so that the warm / cold difference is measurable
    import time
    print("ready", flush=True)
    for n, line in enumerate(sys.stdin):
        line = line.rstrip("\n")
        if not line:
            continue
        if "\t" not in line:
            print(f"bad request (want <out.wav>\\t<text>): {line!r}", flush=True)
            continue
        out_path, text = line.split("\t", 1)
        t0 = time.perf_counter()
        secs = synth(text, out_path, a.seed + n)
        dt = time.perf_counter() - t0
        print(f"{out_path}\t{secs:.2f} s of audio in {dt:.2f} s (x{secs / max(dt, 1e-9):.2f} real time)", flush=True)
    return 0


def cmd_listen(a) -> int:
    from ..models.voxtral import VoxtralConfig, VoxtralListener, VoxtralModel, load_into, log_mel
    c = VoxtralConfig.tiny() if a.random else VoxtralConfig()
    m = VoxtralModel(c)
    _random_init(m) if a.random else load_into(m, _loader(a.pile, a.model))
    wav, sr = read_wav(a.wav)
    assert sr == 16000, "16 kHz audio expected"
    mel = log_mel(wav, n_mels=c.n_mels)
    step = 2 * c.downsample
    lis = VoxtralListener(m, a.delay, n_pages=max(64, mel.shape[1] // 16 + 8))
    out = []
    for lo in range(0, mel.shape[1] - step + 1, step * a.chunk):          # a.chunk text positions per call: the streaming granularity
        hi = min(mel.shape[1] // step * step, lo + step * a.chunk)
        out += lis.feed(mel[:, lo:hi])
    print(",".join(map(str, out)))
    return 0


def cmd_embed(a) -> int:
    from ..models import embed as E
    kinds = {"clip": (E.ClipConfig, E.ClipEmbedder, E.clip.load_into), "siglip": (E.SiglipConfig, E.SiglipEmbedder, E.siglip.load_into),
             "nomic": (E.NomicConfig, E.NomicTextEmbedder, E.nomic.load_into),
             "nomic-vision": (E.NomicVisionConfig, E.NomicVisionEmbedder, E.nomic.load_vision_into)}
    Cfg, Model, load = kinds[a.kind]
    m = Model(Cfg.tiny() if a.random else Cfg())
    _random_init(m) if a.random else load(m, _loader(a.pile, a.model))
    with torch.no_grad():
        if a.image:
            img = torch.from_numpy(np.load(a.image)).float()
            v = m.embed_image(m.preprocess(img)[None])[0]
        else:
            v = m.embed_text(torch.tensor([[int(x) for x in a.ids.split(",")]]))[0]
    print(" ".join(f"{x:.6f}" for x in v.tolist()))
    return 0


def cmd_rank(a) -> int:
    """Semantic probe (``nomic_semantic_probe`` / ``embed_bakeoff``): embed queries and documents (token-id lists separated by ``;``,
    or images as ``.npy`` files for the image arm), print for every query the documents by descending cosine similarity."""
    from ..models import embed as E
    kinds = {"clip": (E.ClipConfig, E.ClipEmbedder, E.clip.load_into), "siglip": (E.SiglipConfig, E.SiglipEmbedder, E.siglip.load_into),
             "nomic": (E.NomicConfig, E.NomicTextEmbedder, E.nomic.load_into)}
    Cfg, Model, load = kinds[a.kind]
    m = Model(Cfg.tiny() if a.random else Cfg())
    _random_init(m) if a.random else load(m, _loader(a.pile, a.model))

    def embed(item: str):
        with torch.no_grad():
            if item.endswith(".npy"):
                return m.embed_image(m.preprocess(torch.from_numpy(np.load(item)).float())[None])[0]
            return m.embed_text(torch.tensor([[int(x) for x in item.split(",")]]))[0]
    q = torch.stack([embed(x) for x in a.queries.split(";")])
    d = torch.stack([embed(x) for x in a.docs.split(";")])
    sim = q @ d.T
    for i, row in enumerate(sim):
        order = torch.argsort(row, descending=True)
        print(f"query {i}: " + " ".join(f"{int(j)}:{float(row[j]):.4f}" for j in order))
    return 0


def cmd_imagine(a) -> int:
    from ..models.flux import Flux2Config, Flux2Transformer, Flux2VAE, FluxPipeline, VAEConfig
    from ..models.flux import transformer as T, vae as V
    if a.random:
        vae = _random_init(Flux2VAE(VAEConfig.tiny()))
        c = Flux2Config.tiny()
        c.in_channels = 4 * vae.c.latent_channels
        tr = _random_init(Flux2Transformer(c), std=0.2)
    else:
        tr, vae = Flux2Transformer(Flux2Config()), Flux2VAE(VAEConfig())
        T.load_into(tr, _loader(a.pile, a.transformer))
        V.load_into(vae, _loader(a.pile, a.vae))
    feats = torch.from_numpy(np.load(a.features)).float()
    img = FluxPipeline(tr, vae)(feats, a.height, a.width, steps=a.steps, seed=a.seed)
    np.save(a.out, img.numpy())
    print(f"image {tuple(img.shape)} -> {a.out}")
    return 0


def cmd_act(a) -> int:
    from ..models.smolvla import SmolVLA, SmolVLAConfig, load_into
    if a.random:
        m = _random_init(SmolVLA(SmolVLAConfig.tiny()), std=0.2)
    else:
        m = SmolVLA(SmolVLAConfig())
        load_into(m, _loader(a.pile, a.model))
    img = torch.from_numpy(np.load(a.image)).float()
    state = torch.from_numpy(np.load(a.state)).float()
    chunk = m.act([img], [int(x) for x in a.ids.split(",")], state, generator=torch.Generator().manual_seed(a.seed))
    for row in chunk.tolist():
        print(" ".join(f"{x:.5f}" for x in row))
    return 0


def cmd_hear(a) -> int:
    """Audio question answering with Gemma-4 (``gemma_hear`` / ``gemma_listen``): log-mel -> audio tower -> soft tokens spliced into the
    prompt at the placeholder rows -> greedy completion."""
    from ..models.gemma4.audio import Gemma4AudioConfig, Gemma4AudioTower, usm_log_mel
    from ..models.gemma4.audio import load_into as load_audio
    from ..models.gemma4.lm import GemmaLM
    wav, sr = read_wav(a.wav)
    assert sr == 16000, "16 kHz audio expected"
    if a.random:
        from ..models.gemma4.config import Gemma4TextConfig
        from ..models.gemma4.model import Gemma4Model
        from ..models.gemma4.weights import init_random_
        cfg = Gemma4TextConfig(hidden_size=64, num_hidden_layers=2, num_attention_heads=2, head_dim=32, intermediate_size=96, vocab_size=128)
        model = Gemma4Model(cfg)
        init_random_(model, a.seed, std=0.05)
        lm = GemmaLM(model, max_seq=512, max_batch=2)
        tower = _random_init(Gemma4AudioTower(Gemma4AudioConfig(n_mels=128, hidden=32, layers=1, heads=4, conv_channels=(128, 8), out_dims=24,
                                                                text_hidden=cfg.hidden_size)), a.seed, 0.1)
    else:
        lm = GemmaLM.from_pile(a.pile)
        tower = Gemma4AudioTower(Gemma4AudioConfig(text_hidden=lm.model.cfg.hidden_size))
        load_audio(tower, _loader(a.pile, a.model))
    with torch.no_grad():
        soft = tower(usm_log_mel(wav))
    before = [int(x) for x in a.ids.split(",")] if a.ids else [2]
    after = [int(x) for x in a.ids_after.split(",")] if a.ids_after else []
    ids = before + [a.placeholder] * soft.shape[0] + after
    rows = list(range(len(before), len(before) + soft.shape[0]))
    out = lm.complete_multimodal(ids, rows, soft, a.max_new, stop_on_eos=not a.random)
    print(f"{soft.shape[0]} audio tokens ({len(wav) / sr:.2f} s)", file=sys.stderr)
    print(lm.tokenizer.decode(out) if lm.tokenizer is not None else ",".join(map(str, out)))
    return 0


def cmd_speak(a) -> int:
    """Qwen3-TTS (``speak`` / ``qwen3tts_say`` / ``qwen3tts_stream``): text ids -> talker + code predictor frames (streamed to the codec
    decoder frame by frame) -> waveform."""
    from ..models.codec.mimi import MimiCodec, MimiConfig
    from ..models.codec.mimi import init_random_ as init_codec
    from ..models.qwen3tts.model import CodePredictor, Qwen3TTSConfig, SamplingParams, Talker, generate_frames
    from ..models.qwen3tts.model import init_random_ as init_tts
    from ..models.qwen3tts.model import load_into as load_tts
    if a.random:
        cfg = Qwen3TTSConfig.tiny()
        talker, pred = Talker(cfg), CodePredictor(cfg)
        init_tts(talker, pred, a.seed)
        mc = MimiConfig.tiny()
        codec = MimiCodec(mc)
        init_codec(codec, a.seed)
    else:
        cfg = Qwen3TTSConfig()
        talker, pred = Talker(cfg), CodePredictor(cfg)
        load_tts(talker, pred, _loader(a.pile, a.model))
        from ..models.codec.mimi import load_into as load_codec
        mc = MimiConfig()
        mc.num_codebooks, mc.codebook_size = cfg.num_code_groups, cfg.pred_vocab
        codec = MimiCodec(mc)
        load_codec(codec, _loader(a.pile, a.codec))              # a codec checkpoint in the Mimi layout (``mary import`` it under this name)
    text = torch.tensor([int(x) for x in a.ids.split(",")], dtype=torch.int32)
    n0 = max(1, min(len(text), a.prefill))
    with torch.no_grad():
        prefill = talker.embed_text(text[:n0]) + talker.embed_codec(torch.full((n0,), cfg.codec_pad, dtype=torch.int32))
        trailing = talker.embed_text(text[n0:]) if len(text) > n0 else torch.zeros(0, prefill.shape[1])
        pad = talker.embed_text(torch.tensor([0], dtype=torch.int32))[0]
    chunks, state = [], [None]

    def sink(frame):                                       # streaming: every frame is decoded as soon as it exists
        codes = (torch.tensor(frame[:codec.c.num_codebooks], dtype=torch.long) % codec.c.codebook_size)[None]
        pcm, state[0] = codec.decode_step(codes, state[0])
        chunks.append(pcm.reshape(-1))
        return True
    frames = generate_frames(talker, pred, prefill, trailing, pad, SamplingParams(max_frames=a.max_frames, seed=a.seed), on_frame=sink)
    pcm = torch.cat(chunks) if chunks else torch.zeros(0)
    write_wav(a.out, pcm.numpy(), codec.c.sample_rate)
    print(f"{frames.shape[0]} frames, {pcm.shape[0]} samples -> {a.out}")
    return 0


def cmd_converse(a) -> int:
    """Full-duplex speech LM (``personaplex_listen``): the user's audio is encoded frame by frame with the streaming codec, every frame
    runs one temporal + depformer step (the user's codes are forced into their streams, text and the agent's codes are generated),
    the agent's codes are decoded to audio frame by frame.  Prints the text tokens; writes the agent's waveform."""
    from ..models.codec.mimi import MimiCodec, MimiConfig
    from ..models.codec.mimi import init_random_ as init_codec
    from ..models.moshi import LmGen, MoshiConfig
    from ..models.moshi import init_random_ as init_lm
    from ..models.codec import mimi
    from ..models import moshi
    if a.random:
        c = MoshiConfig.tiny()
        mc = MimiConfig.tiny()
        mc.num_codebooks, mc.codebook_size = c.codebooks_per_stream, c.card
        codec, lm = MimiCodec(mc), LmGen(c)
        init_codec(codec, a.seed), init_lm(lm, a.seed)
    else:
        c, mc = MoshiConfig(), MimiConfig()
        codec, lm = MimiCodec(mc), LmGen(c, dtype=torch.bfloat16 if torch.cuda.is_available() else torch.float32,
                                         device="cuda" if torch.cuda.is_available() else "cpu")
        mimi.load_into(codec, _loader(a.pile, a.codec))
        moshi.load_into(lm, _loader(a.pile, a.model))
    wav, sr = read_wav(a.wav)
    spf = mc.samples_per_frame
    n = len(wav) // spf
    enc_state = dec_state = None
    text, chunks = [], []
    with torch.no_grad():
        for f in range(min(n, c.context - 2)):
            codes, enc_state = codec.encode_step(torch.from_numpy(wav[f * spf:(f + 1) * spf]).float(), enc_state)
            out = lm.step(user_audio=[int(x) for x in codes.reshape(-1)[:c.codebooks_per_stream]])
            if out is None:                              # still inside the delay horizon
                continue
            text.append(out[0])
            agent = torch.tensor(out[1:1 + c.codebooks_per_stream], dtype=torch.long)[None] % mc.codebook_size
            pcm, dec_state = codec.decode_step(agent, dec_state)
            chunks.append(pcm.reshape(-1))
    write_wav(a.out, (torch.cat(chunks) if chunks else torch.zeros(0)).numpy(), mc.sample_rate)
    print(",".join(map(str, text)))
    return 0


def main(argv=None) -> int:
    ap = argparse.ArgumentParser(prog="families")
    sub = ap.add_subparsers(dest="cmd", required=True)

    def common(p):
        p.add_argument("--pile")
        p.add_argument("--model")
        p.add_argument("--random", action="store_true", help="tiny configuration with random weights (no pile)")
        p.add_argument("--seed", type=int, default=0)
        return p
    s = common(sub.add_parser("say"))
    s.add_argument("--vocoder", default="vocos"), s.add_argument("--ref-wav", required=True), s.add_argument("--ref-text", required=True)
    s.add_argument("--text"), s.add_argument("--out"), s.add_argument("--nfe", type=int, default=32)
    s.add_argument("--serve", action="store_true", help="load once, then one request per line of standard input: <out.wav>\\t<text>")
    s.add_argument("--cfg", type=float, default=2.0), s.add_argument("--speed", type=float, default=1.0)
    s.set_defaults(fn=cmd_say)
    li = common(sub.add_parser("listen"))
    li.add_argument("--wav", required=True), li.add_argument("--delay", type=int), li.add_argument("--chunk", type=int, default=4)
    li.set_defaults(fn=cmd_listen)
    e = common(sub.add_parser("embed"))
    e.add_argument("--kind", required=True, choices=["clip", "siglip", "nomic", "nomic-vision"]), e.add_argument("--image"), e.add_argument("--ids")
    e.set_defaults(fn=cmd_embed)
    rk = common(sub.add_parser("rank"))
    rk.add_argument("--kind", required=True, choices=["clip", "siglip", "nomic"]), rk.add_argument("--queries", required=True)
    rk.add_argument("--docs", required=True)
    rk.set_defaults(fn=cmd_rank)
    im = common(sub.add_parser("imagine"))
    im.add_argument("--transformer"), im.add_argument("--vae"), im.add_argument("--features", required=True), im.add_argument("--out", required=True)
    im.add_argument("--height", type=int, default=1024), im.add_argument("--width", type=int, default=1024), im.add_argument("--steps", type=int, default=4)
    im.set_defaults(fn=cmd_imagine)
    ac = common(sub.add_parser("act"))
    ac.add_argument("--image", required=True), ac.add_argument("--ids", required=True), ac.add_argument("--state", required=True)
    ac.set_defaults(fn=cmd_act)
    he = common(sub.add_parser("hear"))
    he.add_argument("--wav", required=True), he.add_argument("--ids"), he.add_argument("--ids-after"), he.add_argument("--placeholder", type=int, default=3)
    he.add_argument("--max-new", type=int, default=32)
    he.set_defaults(fn=cmd_hear)
    sp = common(sub.add_parser("speak"))
    sp.add_argument("--ids", required=True), sp.add_argument("--out", required=True), sp.add_argument("--max-frames", type=int, default=64)
    sp.add_argument("--prefill", type=int, default=6), sp.add_argument("--codec", default="codec")
    sp.set_defaults(fn=cmd_speak)
    cv = common(sub.add_parser("converse"))
    cv.add_argument("--wav", required=True), cv.add_argument("--out", required=True), cv.add_argument("--codec", default="mimi")
    cv.set_defaults(fn=cmd_converse)
    a = ap.parse_args(argv)
    if argv is None:                                  # run as a program: fail loudly on any thread
        from ..utils import fatal
        fatal.arm()
    return a.fn(a)


if __name__ == "__main__":
    sys.exit(main())
