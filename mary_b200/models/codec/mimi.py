"""Streaming neural audio codec of the Mimi family: SEANet convolutional encoder / decoder, an 8-layer transformer
bottleneck on either side, and a split residual vector quantiser (1 semantic + N acoustic codebooks).

Reference (dimensions measured from the Moshi checkpoint): src/models/personaplex/mimi/config.rs:1-48; encoder
src/models/personaplex/mimi/encoder.rs:1-30 (stem conv k7, per ratio {residual unit, ELU, strided conv k = 2r}, ELU + conv k3,
transformer with LayerNorm / RoPE / sliding window 250 / GELU / LayerScale, downsampling conv k4 s2 with replicate padding,
nearest-codeword search); decoder src/models/personaplex/mimi/decoder.rs:1-26 (codebook sums, output projections, depthwise
transposed conv k4 s2, transformer, conv k7, per ratio {ELU, transposed conv k = 2r with causal right trim, residual unit},
ELU + conv k3).  Everything is causal: a convolution with kernel k and stride s sees ``k - s`` samples of left context, a
transposed convolution carries the ``k - s`` samples that overlap the next chunk.

Two execution arms over the same weights.  ``device="cpu"`` uses ``torch.nn.functional`` convolutions and is the oracle.  On
CUDA every convolution is an im2col gather (activation applied on the way, left context read from the streaming state) followed
by the tensor-core GEMM, every transposed convolution the GEMM followed by an overlap-add that carries the tail, the codebook
search a GEMM with the ``-|c|^2 / 2`` bias and the device arg-max (``csrc/kernels/codec.cu``).  Streaming: ``encode_step`` /
``decode_step`` process whole frames and keep conv contexts, overlap tails and transformer KV caches between calls; feeding a
clip frame by frame gives the codes / samples of one offline pass."""
from __future__ import annotations

import math
from dataclasses import dataclass, field

import torch
import torch.nn.functional as F
from torch import nn


@dataclass
class MimiConfig:
    hidden: int = 512
    n_filters: int = 64
    ratios: tuple = (8, 6, 5, 4)              # decoder order; the encoder applies them reversed
    kernel: int = 7
    last_kernel: int = 3
    residual_kernel: int = 3
    compress: int = 2
    tr_layers: int = 8
    tr_heads: int = 8
    tr_ffn: int = 2048
    tr_window: int = 250
    tr_eps: float = 1e-5
    rope_theta: float = 10000.0
    code_dim: int = 256
    codebook_size: int = 2048
    num_codebooks: int = 8                    # 1 semantic + 7 acoustic
    sample_rate: int = 24000

    @property
    def samples_per_frame(self) -> int:
        return math.prod(self.ratios) * 2

    @staticmethod
    def tiny():
        return MimiConfig(hidden=32, n_filters=4, ratios=(4, 2), kernel=7, tr_layers=2, tr_heads=2, tr_ffn=64, tr_window=6,
                          code_dim=16, codebook_size=32, num_codebooks=3)


def _P(*shape):
    return nn.Parameter(torch.empty(*shape), requires_grad=False)


class CausalConv1d(nn.Module):
    """``x [C_in, L] -> [C_out, L / stride]`` with ``k - stride`` samples of left context (zeros, or the first sample repeated)."""

    def __init__(self, cin, cout, k, stride=1, bias=True, replicate=False):
        super().__init__()
        self.k, self.stride, self.replicate = k, stride, replicate
        self.weight = _P(cout, cin, k)
        self.bias = _P(cout) if bias else None

    def new_state(self, dev):
        return None

    def forward(self, x, state=None):
        ctx = self.k - self.stride
        if state is None:
            left = x[:, :1].expand(-1, ctx) if self.replicate else x.new_zeros(x.shape[0], ctx)
        else:
            left = state
        xx = torch.cat([left, x], 1)
        y = F.conv1d(xx[None], self.weight.to(x.dtype), None if self.bias is None else self.bias.to(x.dtype), stride=self.stride)[0]
        used = y.shape[1] * self.stride                      # input samples consumed by whole output frames
        return y, xx[:, used:used + ctx] if ctx else xx[:, :0]


class CausalConvTranspose1d(nn.Module):
    """``x [C_in, L] -> [C_out, L * stride]``; the ``k - stride`` tail that overlaps the next chunk is carried in the state."""

    def __init__(self, cin, cout, k, stride, depthwise=False):
        super().__init__()
        self.k, self.stride, self.groups = k, stride, (cin if depthwise else 1)
        self.weight = _P(cin, cout // self.groups, k)
        self.bias = None if depthwise else _P(cout)

    def forward(self, x, state=None):
        y = F.conv_transpose1d(x[None], self.weight.to(x.dtype), None, stride=self.stride, groups=self.groups)[0]
        tail = self.k - self.stride
        if state is not None:
            y = torch.cat([y[:, :tail] + state, y[:, tail:]], 1)
        out, new_state = y[:, :y.shape[1] - tail], y[:, y.shape[1] - tail:]
        if self.bias is not None:
            out = out + self.bias.to(x.dtype)[:, None]
        return out, new_state


class ResUnit(nn.Module):
    def __init__(self, dim, compress, k):
        super().__init__()
        self.c1 = CausalConv1d(dim, dim // compress, k)
        self.c2 = CausalConv1d(dim // compress, dim, 1)

    def forward(self, x, state=None):
        s = state or [None, None]
        h, s0 = self.c1(F.elu(x), s[0])
        h, s1 = self.c2(F.elu(h), s[1])
        return x + h, [s0, s1]


class TransformerLayer(nn.Module):
    def __init__(self, c: MimiConfig):
        super().__init__()
        H = c.hidden
        self.c = c
        self.ln1_w, self.ln1_b, self.ln2_w, self.ln2_b = _P(H), _P(H), _P(H), _P(H)
        self.w_qkv, self.w_o = _P(3 * H, H), _P(H, H)
        self.w_fc1, self.w_fc2 = _P(c.tr_ffn, H), _P(H, c.tr_ffn)
        self.scale1, self.scale2 = _P(H), _P(H)

    def forward(self, x, pos0: int, kv):
        """``x [T, H]`` rows at positions ``pos0 ..``; ``kv`` = (k, v) of the previous ``<= window`` positions or None."""
        c = self.c
        T, H = x.shape
        nh, hd = c.tr_heads, H // c.tr_heads
        h = F.layer_norm(x, (H,), self.ln1_w.to(x.dtype), self.ln1_b.to(x.dtype), c.tr_eps)
        q, k, v = (h @ self.w_qkv.to(x.dtype).T).view(T, 3, nh, hd).unbind(1)
        pos = torch.arange(pos0, pos0 + T, device=x.device)
        inv = c.rope_theta ** (-torch.arange(0, hd, 2, device=x.device, dtype=torch.float32) / hd)
        ang = pos[:, None].float() * inv[None]
        cos, sin = ang.cos()[:, None, :].to(x.dtype), ang.sin()[:, None, :].to(x.dtype)

        def rot(t):                                           # interleaved pairs (x0, x1), (x2, x3) ...
            a, b = t[..., 0::2], t[..., 1::2]
            return torch.stack([a * cos - b * sin, a * sin + b * cos], -1).reshape(t.shape)
        q, k = rot(q), rot(k)
        if kv is not None:
            k, v = torch.cat([kv[0], k]), torch.cat([kv[1], v])
        L = k.shape[0]
        kpos = torch.arange(pos0 + T - L, pos0 + T, device=x.device)
        mask = (kpos[None, :] <= pos[:, None]) & (pos[:, None] - kpos[None, :] < c.tr_window)
        s = torch.einsum("thd,lhd->htl", q, k) * hd ** -0.5
        p = torch.softmax(s.masked_fill(~mask[None], float("-inf")).float(), -1).to(x.dtype)
        a = torch.einsum("htl,lhd->thd", p, v).reshape(T, H) @ self.w_o.to(x.dtype).T
        x = x + self.scale1.to(x.dtype) * a
        h = F.layer_norm(x, (H,), self.ln2_w.to(x.dtype), self.ln2_b.to(x.dtype), c.tr_eps)
        m = F.gelu(h @ self.w_fc1.to(x.dtype).T) @ self.w_fc2.to(x.dtype).T
        keep = c.tr_window - 1
        return x + self.scale2.to(x.dtype) * m, (k[-keep:], v[-keep:]) if keep > 0 else None


class Transformer(nn.Module):
    def __init__(self, c: MimiConfig):
        super().__init__()
        self.layers = nn.ModuleList([TransformerLayer(c) for _ in range(c.tr_layers)])

    def forward(self, x, state=None):
        """``x [H, T]`` (channels first, as the convolutions use) -> same shape."""
        st = state or {"pos": 0, "kv": [None] * len(self.layers)}
        h = x.T
        kvs = []
        for L, kv in zip(self.layers, st["kv"]):
            h, kv2 = L(h, st["pos"], kv)
            kvs.append(kv2)
        return h.T, {"pos": st["pos"] + x.shape[1], "kv": kvs}


class Codebook(nn.Module):
    """Euclidean codebook stored as running sums: the codewords are ``embedding_sum / clamp(cluster_usage, 1e-5)``."""

    def __init__(self, size, dim):
        super().__init__()
        self.embedding_sum, self.cluster_usage = _P(size, dim), _P(size)

    def codewords(self):
        return self.embedding_sum / self.cluster_usage.clamp_min(1e-5)[:, None]

    def nearest(self, x):
        """``x [T, dim]`` -> index of the closest codeword (first one on ties): argmax of ``x . c - |c|^2 / 2``."""
        c = self.codewords().to(x.dtype)
        return (x @ c.T - 0.5 * (c * c).sum(-1)[None]).argmax(-1)


class ResidualVQ(nn.Module):
    def __init__(self, n, c: MimiConfig):
        super().__init__()
        self.input_proj, self.output_proj = _P(c.code_dim, c.hidden), _P(c.hidden, c.code_dim)
        self.books = nn.ModuleList([Codebook(c.codebook_size, c.code_dim) for _ in range(n)])

    def encode(self, x):
        """``x [T, hidden]`` -> codes ``[T, n]``: every level quantises what the previous levels left over."""
        r = x @ self.input_proj.to(x.dtype).T
        codes = []
        for b in self.books:
            i = b.nearest(r)
            r = r - b.codewords().to(x.dtype)[i]
            codes.append(i)
        return torch.stack(codes, -1)

    def decode(self, codes, dtype=torch.float32):
        q = sum(b.codewords().to(dtype)[codes[:, j]] for j, b in enumerate(self.books))
        return q @ self.output_proj.to(dtype).T


class MimiCodec(nn.Module):
    def __init__(self, c: MimiConfig):
        super().__init__()
        self.c = c
        nf, enc_r = c.n_filters, tuple(reversed(c.ratios))
        # encoder: stem, per ratio {res unit, ELU, strided conv}, ELU + final conv
        self.enc_stem = CausalConv1d(1, nf, c.kernel)
        self.enc_res, self.enc_down = nn.ModuleList(), nn.ModuleList()
        d = nf
        for r in enc_r:
            self.enc_res.append(ResUnit(d, c.compress, c.residual_kernel))
            self.enc_down.append(CausalConv1d(d, 2 * d, 2 * r, r))
            d *= 2
        self.enc_last = CausalConv1d(d, c.hidden, c.last_kernel)
        self.enc_tr = Transformer(c)
        self.downsample = CausalConv1d(c.hidden, c.hidden, 4, 2, bias=False, replicate=True)
        self.rvq_first, self.rvq_rest = ResidualVQ(1, c), ResidualVQ(c.num_codebooks - 1, c)
        # decoder
        self.upsample = CausalConvTranspose1d(c.hidden, c.hidden, 4, 2, depthwise=True)
        self.dec_tr = Transformer(c)
        self.dec_stem = CausalConv1d(c.hidden, d, c.kernel)
        self.dec_up, self.dec_res = nn.ModuleList(), nn.ModuleList()
        for r in c.ratios:
            self.dec_up.append(CausalConvTranspose1d(d, d // 2, 2 * r, r))
            d //= 2
            self.dec_res.append(ResUnit(d, c.compress, c.residual_kernel))
        self.dec_last = CausalConv1d(d, 1, c.last_kernel)

    # ------------------------------------------------------------------ encoder
    def new_encoder_state(self):
        return {}

    def encode_step(self, pcm, state=None):
        """``pcm [L]`` with ``L`` a multiple of ``samples_per_frame`` -> ``(codes [L / samples_per_frame, num_codebooks], state)``."""
        assert pcm.shape[0] % self.c.samples_per_frame == 0, "feed whole frames"
        st = dict(state or {})
        x = pcm[None].to(self.enc_stem.weight.dtype if self.enc_stem.weight.is_floating_point() else torch.float32)
        x, st["stem"] = self.enc_stem(x, st.get("stem"))
        for i, (res, down) in enumerate(zip(self.enc_res, self.enc_down)):
            x, st[f"res{i}"] = res(x, st.get(f"res{i}"))
            x, st[f"down{i}"] = down(F.elu(x), st.get(f"down{i}"))
        x, st["last"] = self.enc_last(F.elu(x), st.get("last"))
        x, st["tr"] = self.enc_tr(x, st.get("tr"))
        x, st["ds"] = self.downsample(x, st.get("ds"))
        lat = x.T
        return torch.cat([self.rvq_first.encode(lat), self.rvq_rest.encode(lat)], -1), st

    def encode(self, pcm):
        """Offline: right-pad to whole frames, one pass."""
        spf = self.c.samples_per_frame
        pad = (-pcm.shape[0]) % spf
        return self.encode_step(F.pad(pcm, (0, pad)))[0]

    # ------------------------------------------------------------------ decoder
    def decode_step(self, codes, state=None):
        """``codes [T, num_codebooks]`` -> ``(pcm [T * samples_per_frame], state)``."""
        st = dict(state or {})
        dt = self.dec_stem.weight.dtype
        x = (self.rvq_first.decode(codes[:, :1], dt) + self.rvq_rest.decode(codes[:, 1:], dt)).T
        x, st["up"] = self.upsample(x, st.get("up"))
        x, st["tr"] = self.dec_tr(x, st.get("tr"))
        x, st["stem"] = self.dec_stem(x, st.get("stem"))
        for i, (up, res) in enumerate(zip(self.dec_up, self.dec_res)):
            x, st[f"up{i}"] = up(F.elu(x), st.get(f"up{i}"))
            x, st[f"res{i}"] = res(x, st.get(f"res{i}"))
        x, st["last"] = self.dec_last(F.elu(x), st.get("last"))
        return x[0], st

    def decode(self, codes):
        return self.decode_step(codes)[0]


def init_random_(m: MimiCodec, seed: int = 0):
    g = torch.Generator().manual_seed(seed)
    for n, p in m.named_parameters():
        if n.endswith("cluster_usage"):
            p.data.uniform_(0.5, 2.0, generator=g)
        elif n.endswith(("ln1_w", "ln2_w")):
            p.data.fill_(1.0)
        elif n.endswith(("ln1_b", "ln2_b")):
            p.data.zero_()
        elif n.endswith(("scale1", "scale2")):
            p.data.fill_(0.3)
        elif p.dim() == 1:
            p.data.normal_(0.0, 0.02, generator=g)
        else:
            fan_in = p[0].numel() if p.dim() > 1 else 1
            p.data.normal_(0.0, 1.0 / math.sqrt(max(fan_in, 1)), generator=g)


def load_into(m: MimiCodec, loader) -> None:
    """Names of the Hugging Face ``MimiModel`` layout (``kyutai/mimi``).  That layout stores q / k projections for a split-half
    rotation; the rows are re-ordered into consecutive pairs, which is what this implementation (and the original codec) rotates."""
    c = m.c
    n = len(c.ratios)

    def get(name):
        return loader.load_tensor(name, torch.float32)

    def conv(mod, name):
        mod.weight.data.copy_(get(name + ".conv.weight").reshape(mod.weight.shape))
        if mod.bias is not None:
            mod.bias.data.copy_(get(name + ".conv.bias"))

    def res(mod, name):
        conv(mod.c1, name + ".block.1"), conv(mod.c2, name + ".block.3")
    conv(m.enc_stem, "encoder.layers.0")
    for i in range(n):
        res(m.enc_res[i], f"encoder.layers.{1 + 3 * i}")
        conv(m.enc_down[i], f"encoder.layers.{3 + 3 * i}")
    conv(m.enc_last, f"encoder.layers.{3 * n + 2}")
    conv(m.dec_stem, "decoder.layers.0")
    for i in range(n):
        conv(m.dec_up[i], f"decoder.layers.{2 + 3 * i}")
        res(m.dec_res[i], f"decoder.layers.{3 + 3 * i}")
    conv(m.dec_last, f"decoder.layers.{3 * n + 2}")
    conv(m.downsample, "downsample")
    conv(m.upsample, "upsample")
    hd = c.hidden // c.tr_heads
    pair = torch.stack([torch.arange(hd // 2), torch.arange(hd // 2) + hd // 2], -1).reshape(-1)       # split-half row -> pair order
    perm = (torch.arange(c.tr_heads)[:, None] * hd + pair[None, :]).reshape(-1)
    for tr, name in ((m.enc_tr, "encoder_transformer"), (m.dec_tr, "decoder_transformer")):
        for i, L in enumerate(tr.layers):
            p = f"{name}.layers.{i}."
            q, k, v = (get(p + f"self_attn.{x}_proj.weight") for x in "qkv")
            L.w_qkv.data.copy_(torch.cat([q[perm], k[perm], v], 0))
            for ours, theirs in (("w_o", "self_attn.o_proj.weight"), ("w_fc1", "mlp.fc1.weight"), ("w_fc2", "mlp.fc2.weight"),
                                 ("ln1_w", "input_layernorm.weight"), ("ln1_b", "input_layernorm.bias"),
                                 ("ln2_w", "post_attention_layernorm.weight"), ("ln2_b", "post_attention_layernorm.bias"),
                                 ("scale1", "self_attn_layer_scale.scale"), ("scale2", "mlp_layer_scale.scale")):
                getattr(L, ours).data.copy_(get(p + theirs))
    for rvq, name in ((m.rvq_first, "quantizer.semantic_residual_vector_quantizer"), (m.rvq_rest, "quantizer.acoustic_residual_vector_quantizer")):
        rvq.input_proj.data.copy_(get(name + ".input_proj.weight")[:, :, 0])
        rvq.output_proj.data.copy_(get(name + ".output_proj.weight")[:, :, 0])
        for j, b in enumerate(rvq.books):
            b.embedding_sum.data.copy_(get(f"{name}.layers.{j}.codebook.embed_sum"))
            b.cluster_usage.data.copy_(get(f"{name}.layers.{j}.codebook.cluster_usage"))
