"""Mimi-style streaming codec: streaming in frames equals one offline pass (encoder and decoder), the residual quantiser
picks exact nearest codewords level by level, causality holds, shapes follow the frame rate."""
import pytest
import torch

from mary_b200.models.codec import MimiCodec, MimiConfig, init_random_


def _codec(seed=0):
    c = MimiConfig.tiny()
    m = MimiCodec(c)
    init_random_(m, seed)
    return c, m


def test_streaming_encoder_and_decoder_equal_offline():
    c, m = _codec()
    spf = c.samples_per_frame
    assert spf == 4 * 2 * 2
    torch.manual_seed(1)
    pcm = torch.randn(spf * 9)
    with torch.no_grad():
        codes = m.encode(pcm)
        assert codes.shape == (9, c.num_codebooks) and int(codes.max()) < c.codebook_size
        st, parts = None, []
        for n in (1, 3, 2, 3):                              # uneven chunking, whole frames
            a = sum(x.shape[0] for x in parts) * spf
            cs, st = m.encode_step(pcm[a:a + n * spf], st)
            parts.append(cs)
        assert torch.equal(torch.cat(parts), codes)
        wav = m.decode(codes)
        assert wav.shape == (9 * spf,)
        st, outs = None, []
        for a, b in ((0, 2), (2, 3), (3, 9)):
            w, st = m.decode_step(codes[a:b], st)
            outs.append(w)
        assert torch.allclose(torch.cat(outs), wav, atol=1e-5)


def test_codec_is_causal():
    c, m = _codec(1)
    spf = c.samples_per_frame
    torch.manual_seed(2)
    a = torch.randn(spf * 6)
    b = a.clone()
    b[spf * 4:] = torch.randn(spf * 2)                      # change only the last two frames
    with torch.no_grad():
        ca, cb = m.encode(a), m.encode(b)
        assert torch.equal(ca[:4], cb[:4])
        codes2 = ca.clone()
        codes2[5] = (codes2[5] + 1) % c.codebook_size
        wa, wb = m.decode(ca), m.decode(codes2)
        assert torch.allclose(wa[:5 * spf], wb[:5 * spf], atol=1e-6) and not torch.allclose(wa[5 * spf:], wb[5 * spf:])


def test_residual_quantiser_is_greedy_nearest_and_lowers_the_error():
    c, m = _codec(2)
    torch.manual_seed(3)
    x = torch.randn(20, c.hidden)
    rvq = m.rvq_rest
    with torch.no_grad():
        codes = rvq.encode(x)
        r = x @ rvq.input_proj.T
        errs = [float(r.norm())]
        for j, b in enumerate(rvq.books):
            cw = b.codewords()
            d = ((r[:, None, :] - cw[None]) ** 2).sum(-1)
            assert torch.equal(codes[:, j], d.argmin(-1))
            r = r - cw[codes[:, j]]
            errs.append(float(r.norm()))
        assert all(b <= a + 1e-6 for a, b in zip(errs, errs[1:]))
        q = sum(b.codewords()[codes[:, j]] for j, b in enumerate(rvq.books)) @ rvq.output_proj.T
        assert torch.allclose(rvq.decode(codes), q, atol=1e-6)


def test_codec_matches_the_huggingface_mimi_implementation():
    """Same weights by name: the codes of the streaming encoder and the waveform of the streaming decoder equal the library's offline
    encode / decode (which also proves the streaming state handling: the library processes the whole signal at once)."""
    transformers = pytest.importorskip("transformers")
    from transformers.models.mimi import MimiConfig as HC, MimiModel
    from mary_b200.models.codec.mimi import MimiCodec, MimiConfig, load_into
    torch.manual_seed(0)
    hc = HC(hidden_size=32, num_filters=4, upsampling_ratios=[4, 2], num_hidden_layers=2, intermediate_size=64, num_attention_heads=2,
            num_key_value_heads=2, codebook_size=32, codebook_dim=16, vector_quantization_hidden_dimension=16, num_quantizers=3,
            sliding_window=6, upsample_groups=32, head_dim=16)
    hc._attn_implementation = "eager"
    hf = MimiModel(hc).eval()
    with torch.no_grad():
        for n, p in hf.named_parameters():
            if n.endswith("layer_scale.scale"):
                p.fill_(0.5)
        for n, b in hf.named_buffers():
            if n.endswith("embed_sum"):
                b.copy_(torch.randn_like(b))
            if n.endswith("cluster_usage"):
                b.copy_(torch.rand_like(b) + 0.5)
    sd = {k: v.detach().clone() for k, v in hf.state_dict().items()}

    class L:
        def load_tensor(self, n, dtype):
            return sd[n].to(dtype)
    c = MimiConfig(hidden=32, n_filters=4, ratios=(4, 2), kernel=7, tr_layers=2, tr_heads=2, tr_ffn=64, tr_window=6, code_dim=16,
                   codebook_size=32, num_codebooks=3)
    m = MimiCodec(c)
    load_into(m, L())
    pcm = torch.randn(c.samples_per_frame * 20) * 0.3
    with torch.no_grad():
        want = hf.encode(pcm[None, None]).audio_codes[0].T                      # [T, n_q]
        st, got = None, []
        for lo in range(0, 20, 5):                                              # four chunks of five frames through the streaming encoder
            codes, st = m.encode_step(pcm[lo * c.samples_per_frame:(lo + 5) * c.samples_per_frame], st)
            got.append(codes)
        got = torch.cat(got)
        assert got.shape == want.shape == (20, 3)
        assert (got == want).float().mean() >= 0.95, (got != want).nonzero()    # a near-tie of two codewords may resolve differently
        audio = hf.decode(want.T[None]).audio_values[0, 0]
        st, out = None, []
        for lo in range(0, 20, 4):
            y, st = m.decode_step(want[lo:lo + 4], st)
            out.append(y)
        out = torch.cat(out)
    n = min(len(out), len(audio))
    assert abs(len(out) - len(audio)) <= c.samples_per_frame
    assert torch.allclose(out[:n], audio[:n], atol=1e-4), float((out[:n] - audio[:n]).abs().max())
