"""The Qwen3-TTS speech codec (decoder and encoder) against plain PyTorch convolutions and its own structural invariants."""
import pytest
import torch
import torch.nn.functional as F

from mary_b200.models.qwen3tts import codec as C


def test_causal_convolutions_as_gemms_equal_the_plain_convolutions():
    g = torch.Generator().manual_seed(0)
    x = torch.randn(37, 6, generator=g)                                              # time-major [T, C]
    for k, dil in ((1, 1), (3, 1), (7, 3), (7, 9)):
        w, b = torch.randn(5, 6, k, generator=g), torch.randn(5, generator=g)
        want = F.conv1d(F.pad(x.t()[None], ((k - 1) * dil, 0)), w, b, dilation=dil)[0].t()
        assert torch.allclose(C.causal_conv(x, C.conv_weight(w), b, k, dil), want, atol=1e-5)
    w, b = torch.randn(6, 1, 7, generator=g), torch.randn(6, generator=g)
    want = F.conv1d(F.pad(x.t()[None], (6, 0)), w, b, groups=6)[0].t()
    assert torch.allclose(C.depthwise_causal_conv(x, w, b), want, atol=1e-5)
    for k, s in ((2, 2), (4, 2), (6, 3), (16, 8)):
        w, b = torch.randn(6, 4, k, generator=g), torch.randn(4, generator=g)
        want = F.conv_transpose1d(x.t()[None], w, b, stride=s)[0].t()[:37 * s]          # causal: the right trim drops k - s samples
        assert torch.allclose(C.causal_transconv(x, C.transconv_weight(w), b, 4, k, s), want, atol=1e-5)
    with pytest.raises(ValueError):
        C.causal_transconv(x, torch.zeros(12, 6), torch.zeros(4), 4, 3, 2)
    # the encoder's strided form: left pad k - s, right pad to whole frames; zeros or edge values
    for k, s, rep, T in ((7, 1, False, 37), (8, 4, False, 37), (4, 2, True, 37), (4, 2, True, 36), (10, 5, False, 3)):
        w, b = torch.randn(5, 6, k, generator=g), torch.randn(5, generator=g)
        xt = x[:T]
        n_frames = -(-T // s)
        pad_r = max((n_frames - 1) * s + k - (k - s) - T, 0)
        xp = F.pad(xt.t()[None], (k - s, pad_r), mode="replicate" if rep else "constant")
        want = F.conv1d(xp, w, b, stride=s)[0].t()
        got = C.strided_causal_conv(xt, w, b, s, rep)
        assert got.shape == want.shape and torch.allclose(got, want, atol=1e-5), (k, s, rep, T)


def test_snake_rope_attention_and_rvq_pieces():
    g = torch.Generator().manual_seed(1)
    x, a, b = torch.randn(9, 4, generator=g), torch.randn(4, generator=g), torch.randn(4, generator=g)
    assert torch.allclose(C.snake_beta(x, a, b), x + torch.sin(x * a.exp()) ** 2 / (b.exp() + 1e-9))
    q, k, v = (torch.randn(12, 2, 8, generator=g) for _ in range(3))
    got = C.windowed_attention(q, k, v, 4)
    for t in (0, 3, 11):
        lo = max(0, t - 3)
        p = torch.softmax(torch.einsum("hd,shd->hs", q[t], k[lo:t + 1]) / 8 ** 0.5, -1)
        assert torch.allclose(got[t], torch.einsum("hs,shd->hd", p, v[lo:t + 1]), atol=1e-5)
    # relative positions only: shifting all positions leaves q.k unchanged
    pos = torch.arange(12)
    s0 = torch.einsum("thd,shd->hts", C.rope_half(q, pos, 1e4), C.rope_half(k, pos, 1e4))
    s1 = torch.einsum("thd,shd->hts", C.rope_half(q, pos + 5, 1e4), C.rope_half(k, pos + 5, 1e4))
    assert torch.allclose(s0, s1, atol=1e-4)
    # residual VQ: a vector that IS a sum of one row per codebook (shrinking scales) comes back as those rows
    books = [torch.randn(16, 8, generator=g) * sc for sc in (4.0, 1.0, 0.25)]
    want = torch.tensor([[3, 7, 1], [15, 0, 9]])
    r = sum(bk[want[:, i]] for i, bk in enumerate(books))
    assert torch.equal(C.rvq_encode(r, books), want)
    tie = [torch.tensor([[1.0, 0.0], [1.0, 0.0], [0.0, 1.0]])]
    assert C.rvq_encode(torch.tensor([[1.0, 0.0]]), tie).tolist() == [[0]]                # first minimum wins


def test_decoder_is_causal_shapes_add_up_and_chunking_matches_the_tail():
    cfg = C.CodecConfig.tiny()
    dec = C.CodecDecoder(cfg).init_random_(0)
    assert not dec.missing() and cfg.samples_per_frame == 12
    g = torch.Generator().manual_seed(2)
    codes = torch.randint(0, cfg.codebook_size, (20, cfg.num_code_groups), generator=g)
    wav = dec.decode(codes)
    assert wav.shape == (20 * 12,) and wav.abs().max() <= 1.0 and wav.std() > 1e-3
    # fully causal: the first n frames decode to the same samples whatever follows
    assert torch.allclose(dec.decode(codes[:9]), wav[:9 * 12], atol=1e-4)
    other = codes.clone()
    other[9:] = (other[9:] + 1) % cfg.codebook_size
    assert torch.allclose(dec.decode(other)[:9 * 12], wav[:9 * 12], atol=1e-4) and not torch.allclose(dec.decode(other), wav, atol=1e-2)
    # every codebook of both banks reaches the output
    for gidx in (0, 1, cfg.num_code_groups - 1):
        alt = codes.clone()
        alt[:, gidx] = (alt[:, gidx] + 1) % cfg.codebook_size
        assert not torch.allclose(dec.decode(alt), wav, atol=1e-4)
    # chunked decode: the first chunk is exact; later chunks see `context` frames only, so they agree once the receptive field is covered
    full = dec.chunked_decode(codes, chunk=50, context=5)
    assert torch.allclose(full, wav, atol=1e-4)
    ch = dec.chunked_decode(codes, chunk=8, context=8)
    assert ch.shape == wav.shape and torch.allclose(ch[:8 * 12], wav[:8 * 12], atol=1e-4)
    with pytest.raises(ValueError):
        dec.decode(torch.full((3, cfg.num_code_groups), cfg.codebook_size))
    with pytest.raises(ValueError):
        dec.set_tensor("decoder.pre_conv.conv.bias", torch.zeros(3))
    with pytest.raises(KeyError):
        dec.set_tensor("decoder.nope", torch.zeros(3))


def test_encoder_frames_causality_and_round_trip_through_its_own_codebooks():
    cfg = C.CodecConfig.tiny()
    enc = C.CodecEncoder(cfg).init_random_(3)
    g = torch.Generator().manual_seed(4)
    wav = torch.randn(12 * 10 + 5, generator=g) * 0.3
    codes = enc.encode(wav)
    assert codes.shape == (11, cfg.num_code_groups) and codes.min() >= 0 and codes.max() < cfg.codebook_size
    assert torch.equal(codes, enc.encode(wav))                                          # deterministic
    # causal up to the frame that holds the change: a different tail leaves the earlier frames' codes alone
    other = wav.clone()
    other[12 * 6:] = torch.randn(wav.numel() - 12 * 6, generator=g)
    c2 = enc.encode(other)
    assert torch.equal(c2[:6], codes[:6]) and not torch.equal(c2, codes)
    assert enc.encode(wav[:12 * 4]).shape[0] == 4 and enc.encode(wav[:12 * 4 + 1]).shape[0] == 5
    # decoder and encoder share the checkpoint's naming scheme but no tensors
    dec = C.CodecDecoder(cfg)
    assert not {n for n, _ in dec.expected()} & {n for n, _ in enc.expected()}
    assert all(n.startswith("encoder.") for n, _ in enc.expected()) and all(n.startswith("decoder.") for n, _ in dec.expected())


def test_full_size_declarations_match_the_checkpoint_dimensions():
    dec, enc = C.CodecDecoder(), C.CodecEncoder()
    s = dict(dec.expected())
    assert dec.cfg.samples_per_frame == 1920
    assert s["decoder.decoder.0.conv.weight"] == (1536, 1024, 7) and s["decoder.decoder.1.block.1.conv.weight"] == (1536, 768, 16)
    assert s["decoder.decoder.4.block.4.conv1.conv.weight"] == (96, 96, 7) and s["decoder.decoder.6.conv.weight"] == (1, 96, 7)
    assert s["decoder.quantizer.rvq_rest.vq.layers.14._codebook.embedding_sum"] == (2048, 256)
    assert s["decoder.pre_transformer.layers.7.self_attn.q_proj.weight"] == (1024, 512)
    e = dict(enc.expected())
    assert e["encoder.encoder.layers.14.conv.weight"] == (512, 1024, 3) and e["encoder.encoder.layers.12.conv.weight"] == (1024, 512, 16)
    assert e["encoder.downsample.conv.weight"] == (512, 512, 4)
    assert e["encoder.quantizer.acoustic_residual_vector_quantizer.layers.30.codebook.embed_sum"] == (2048, 256)


@pytest.mark.gpu
def test_decoder_in_bf16_on_the_gpu_runs_on_the_package_gemm_and_tracks_the_f32_decoder():
    from mary_b200.ops import cuda as K
    cfg = C.CodecConfig(num_code_groups=4, codebook_size=64, code_dim=64, quant_out=128, latent=256, hidden=128, tr_layers=2, tr_heads=2,
                        tr_head_dim=64, tr_inter=256, tr_window=8, decoder_dim=256, upsample_rates=[4, 2], upsampling_ratios=[2])
    cpu = C.CodecDecoder(cfg).init_random_(0)
    tail = "decoder.decoder.4.conv.weight"
    cpu.set_tensor(tail, cpu.P[tail] * 0.02)                                             # keep the waveform inside (-1, 1): no clamping hides or blows up errors
    gpu = C.CodecDecoder(cfg, dtype=torch.bfloat16, device="cuda")
    for n, v in cpu.P.items():
        gpu.set_tensor(n, v)
    codes = torch.randint(0, 64, (40, 4), generator=torch.Generator().manual_seed(5))
    want = cpu.decode(codes)
    before = K.LAUNCHES
    got = gpu.decode(codes).cpu()
    assert K.LAUNCHES > before + 20 and K.last_status() == 0                             # the convolutions ran as this package's GEMMs
    err = (got - want).abs()
    assert got.shape == want.shape and want.abs().max() < 1.0 and want.abs().max() > 0.1
    assert err.max() < 0.25 * want.abs().max() and err.median() < 0.04 * want.abs().max()    # bf16 through ~20 stacked layers
