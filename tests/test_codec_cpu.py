"""Mimi-style streaming codec: streaming in frames equals one offline pass (encoder and decoder), the residual quantiser
picks exact nearest codewords level by level, causality holds, shapes follow the frame rate."""
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
