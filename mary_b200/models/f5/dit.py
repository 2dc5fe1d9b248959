"""F5-TTS: a flow-matching diffusion transformer that in-fills mel frames given a reference recording and the text of both
(src/models/f5/*, docs/F5_ARCH.md; ``say`` / ``say_serve``).

Inputs per frame: the noised mel ``x`` (100), the reference mel ``cond`` (100, zero where speech is to be generated) and a text
feature (512): characters are embedded (id + 1; 0 is the filler that pads the text to the frame count), given a sinusoidal
position code and refined by ConvNeXt-V2 blocks (depthwise kernel-7 convolution, LayerNorm, 512 -> 1024 GELU MLP with global
response normalisation, residual).  ``proj(cat(x, cond, text))`` plus a convolutional position embedding (two grouped kernel-31
convolutions with Mish) feeds ``depth`` AdaLN-zero DiT blocks: the flow time (sinusoid of 256 scaled by 1000 -> SiLU MLP)
produces shift / scale / gate for the attention and the MLP branch of every block; attention is plain multi-head with rotary
positions (interleaved pairs) and no q / k norm; the MLP is Linear-GELU(tanh)-Linear.  A final AdaLN and a projection give the
velocity in mel space.

Sampling (``CFM.sample``): Euler steps from noise at ``t = 0`` to data at ``t = 1`` on a sway-warped time grid
``t + s (cos(pi t / 2) - 1 + t)`` with classifier-free guidance ``v = v_cond + w (v_cond - v_uncond)`` where the unconditional
pass drops both the reference mel and the text; the reference frames are pasted back at the end."""
from __future__ import annotations

import math
from dataclasses import dataclass

import torch
import torch.nn.functional as F
from torch import nn

from ... import ops


@dataclass
class F5Config:
    dim: int = 1024
    depth: int = 22
    heads: int = 16
    ff_mult: int = 2
    n_mels: int = 100
    text_vocab: int = 2546
    text_dim: int = 512
    conv_layers: int = 4
    conv_mult: int = 2
    pos_kernel: int = 31
    pos_groups: int = 16
    time_freq: int = 256
    pe_attn_head: int | None = None        # rotate only the first n heads (an early checkpoint family); None = all heads

    @staticmethod
    def tiny():
        return F5Config(dim=32, depth=2, heads=4, n_mels=12, text_vocab=30, text_dim=16, conv_layers=2, pos_kernel=7, pos_groups=4, time_freq=16)


def _P(*s):
    return nn.Parameter(torch.empty(*s), requires_grad=False)


def _ln(x):
    return F.layer_norm(x, (x.shape[-1],), None, None, 1e-6)


def rope_interleaved(x, pos, inv_freq):
    """Rotate consecutive channel pairs ``(2i, 2i + 1)`` of ``x [T, heads, D]`` by ``pos * inv_freq[i]``."""
    ang = pos.float()[:, None] * inv_freq
    cos, sin = ang.cos()[:, None, :].to(x.dtype), ang.sin()[:, None, :].to(x.dtype)
    a, b = x[..., 0::2], x[..., 1::2]
    return torch.stack([a * cos - b * sin, b * cos + a * sin], -1).flatten(-2)


class ConvNeXtV2Block(nn.Module):
    def __init__(self, dim, inter):
        super().__init__()
        self.dw_w, self.dw_b, self.ln_w, self.ln_b = _P(dim, 1, 7), _P(dim), _P(dim), _P(dim)
        self.w1, self.b1, self.w2, self.b2 = _P(inter, dim), _P(inter), _P(dim, inter), _P(dim)
        self.grn_gamma, self.grn_beta = _P(inter), _P(inter)

    def forward(self, x):
        """``x [T, dim]``.  GRN: per channel, the L2 norm over time divided by its mean over channels rescales the activations."""
        h = F.conv1d(x.T[None], self.dw_w, self.dw_b, padding=3, groups=x.shape[1])[0].T
        h = F.layer_norm(h, (x.shape[1],), self.ln_w, self.ln_b, 1e-6)
        h = F.gelu(ops.linear(h.contiguous(), self.w1, self.b1))
        g = h.float().norm(p=2, dim=0, keepdim=True)
        n = g / (g.mean(dim=-1, keepdim=True) + 1e-6)
        h = (self.grn_gamma * (h * n) + self.grn_beta + h).to(x.dtype)
        return x + ops.linear(h, self.w2, self.b2)


class DiTBlock(nn.Module):
    def __init__(self, c: F5Config):
        super().__init__()
        D, Fd = c.dim, c.dim * c.ff_mult
        self.mod_w, self.mod_b = _P(6 * D, D), _P(6 * D)
        self.w_qkv, self.b_qkv, self.w_o, self.b_o = _P(3 * D, D), _P(3 * D), _P(D, D), _P(D)
        self.ff1_w, self.ff1_b, self.ff2_w, self.ff2_b = _P(Fd, D), _P(Fd), _P(D, Fd), _P(D)


class DiT(nn.Module):
    def __init__(self, c: F5Config):
        super().__init__()
        self.c = c
        D = c.dim
        self.text_embed = _P(c.text_vocab, c.text_dim)
        self.text_blocks = nn.ModuleList([ConvNeXtV2Block(c.text_dim, c.text_dim * c.conv_mult) for _ in range(c.conv_layers)])
        self.in_w, self.in_b = _P(D, 2 * c.n_mels + c.text_dim), _P(D)
        self.pos1_w, self.pos1_b = _P(D, D // c.pos_groups, c.pos_kernel), _P(D)
        self.pos2_w, self.pos2_b = _P(D, D // c.pos_groups, c.pos_kernel), _P(D)
        self.t1_w, self.t1_b, self.t2_w, self.t2_b = _P(D, c.time_freq), _P(D), _P(D, D), _P(D)
        self.blocks = nn.ModuleList([DiTBlock(c) for _ in range(c.depth)])
        self.out_mod_w, self.out_mod_b, self.out_w, self.out_b = _P(2 * D, D), _P(2 * D), _P(c.n_mels, D), _P(c.n_mels)
        hd = D // c.heads
        self.register_buffer("inv_freq", 1.0 / (10000.0 ** (torch.arange(0, hd, 2, dtype=torch.float32) / hd)), persistent=False)

    def time_code(self, t):
        """Scalar flow time -> ``[dim]``: sinusoid(1000 t) of ``time_freq`` -> Linear, SiLU, Linear."""
        half = self.c.time_freq // 2
        f = torch.exp(torch.arange(half, dtype=torch.float32, device=self.t1_w.device) * (-math.log(10000.0) / (half - 1)))
        e = 1000.0 * t.float() * f if (torch.is_tensor(t) and t.is_cuda) else 1000.0 * float(t) * f      # a device scalar stays on the device
        e = torch.cat([e.sin(), e.cos()])[None].to(self.t1_w.dtype)
        return ops.linear(F.silu(ops.linear(e, self.t1_w, self.t1_b)), self.t2_w, self.t2_b)[0]

    def text_features(self, text_ids, T: int, drop: bool = False):
        """``[T, text_dim]``: ids shifted by one, padded with the filler 0 to ``T`` frames (all filler when ``drop``)."""
        c = self.c
        ids = torch.zeros(T, dtype=torch.long, device=self.text_embed.device)
        if not drop:
            t = torch.as_tensor(text_ids, device=ids.device).long()[:T] + 1
            ids[:t.shape[0]] = t
        x = self.text_embed[ids]
        half = c.text_dim // 2
        f = 1.0 / (10000.0 ** (torch.arange(half, dtype=torch.float32, device=x.device) / half))
        ang = torch.arange(T, device=x.device).float()[:, None] * f
        x = x + torch.cat([ang.cos(), ang.sin()], -1).to(x.dtype)
        for b in self.text_blocks:
            x = b(x)
        return x

    def forward(self, x, cond, text_ids, t, drop_cond: bool = False, drop_text: bool = False, text=None):
        """Velocity ``[T, n_mels]`` at flow time ``t`` for the noised mel ``x [T, n_mels]`` and reference mel ``cond [T, n_mels]``.
        ``text``: the result of :meth:`text_features` when the caller holds it (it depends on neither ``x`` nor ``t``)."""
        c = self.c
        T, D, nh = x.shape[0], c.dim, c.heads
        te = self.time_code(t)
        cond = torch.zeros_like(cond) if drop_cond else cond
        tf = self.text_features(text_ids, T, drop_text) if text is None else text
        h = ops.linear(torch.cat([x, cond, tf], -1).to(self.in_w.dtype), self.in_w, self.in_b)
        p = F.mish(F.conv1d(h.T[None], self.pos1_w, self.pos1_b, padding=c.pos_kernel // 2, groups=c.pos_groups))
        p = F.mish(F.conv1d(p, self.pos2_w, self.pos2_b, padding=c.pos_kernel // 2, groups=c.pos_groups))[0].T
        h = h + p
        pos = torch.arange(T, device=h.device)
        st = F.silu(te)[None]
        n_rot = nh if c.pe_attn_head is None else c.pe_attn_head
        for b in self.blocks:
            sh_a, sc_a, g_a, sh_m, sc_m, g_m = ops.linear(st, b.mod_w, b.mod_b)[0].chunk(6)
            y = _ln(h) * (1 + sc_a) + sh_a
            qkv = ops.linear(y.contiguous(), b.w_qkv, b.b_qkv).view(T, 3, nh, D // nh)
            q, k, v = qkv[:, 0], qkv[:, 1], qkv[:, 2]
            q = torch.cat([rope_interleaved(q[:, :n_rot], pos, self.inv_freq), q[:, n_rot:]], 1)
            k = torch.cat([rope_interleaved(k[:, :n_rot], pos, self.inv_freq), k[:, n_rot:]], 1)
            a = F.scaled_dot_product_attention(q.transpose(0, 1)[None], k.transpose(0, 1)[None], v.transpose(0, 1)[None])[0].transpose(0, 1).reshape(T, D)
            h = h + g_a * ops.linear(a, b.w_o, b.b_o)
            y = _ln(h) * (1 + sc_m) + sh_m
            h = h + g_m * ops.linear(F.gelu(ops.linear(y.contiguous(), b.ff1_w, b.ff1_b), approximate="tanh"), b.ff2_w, b.ff2_b)
        sc, sh = ops.linear(st, self.out_mod_w, self.out_mod_b)[0].chunk(2)
        return ops.linear((_ln(h) * (1 + sc) + sh).contiguous(), self.out_w, self.out_b)


def sway_times(nfe: int, sway: float | None = -1.0):
    """``nfe + 1`` flow times from 0 to 1, warped towards 0 by ``t + s (cos(pi t / 2) - 1 + t)`` (more steps where the flow bends)."""
    t = torch.linspace(0.0, 1.0, nfe + 1)
    return t if sway is None else t + sway * (torch.cos(math.pi / 2 * t) - 1 + t)


class CFM:
    """Conditional flow matching sampler around a ``DiT``."""

    def __init__(self, model: DiT, nfe: int = 32, cfg_strength: float = 2.0, sway: float | None = -1.0):
        self.model, self.nfe, self.cfg, self.sway = model, nfe, cfg_strength, sway

    def velocity(self, x, cond, text_ids, t, feats=None):
        tf, tf_drop = feats if feats is not None else (None, None)
        v = self.model(x, cond, text_ids, t, text=tf)
        if self.cfg < 1e-5:
            return v
        return v + (v - self.model(x, cond, text_ids, t, drop_cond=True, drop_text=True, text=tf_drop)) * self.cfg

    use_graph = True

    @torch.no_grad()
    def sample(self, ref_mel, text_ids, total_frames: int, noise=None, generator=None):
        """``ref_mel [T_ref, n_mels]`` + the characters of reference and target -> mel ``[total_frames, n_mels]`` whose first ``T_ref``
        frames are the reference and the rest the generated speech.  The text features (conditioned and dropped) are computed once
        per utterance.  On the GPU ONE Euler step (both guidance passes through all blocks, a few hundred small kernels) is
        captured as a CUDA graph whose flow time comes from a device-resident table and counter, and replayed ``nfe`` times."""
        n_mels = self.model.c.n_mels
        T_ref = ref_mel.shape[0]
        cond = torch.zeros(total_frames, n_mels, dtype=ref_mel.dtype, device=ref_mel.device)
        cond[:T_ref] = ref_mel
        x = torch.randn(total_frames, n_mels, generator=generator).to(ref_mel) if noise is None else noise.clone()
        ts = sway_times(self.nfe, self.sway)
        feats = (self.model.text_features(text_ids, total_frames), self.model.text_features(text_ids, total_frames, True))
        if x.is_cuda and self.use_graph:
            tdev, i = ts.to(x.device), torch.zeros(1, dtype=torch.long, device=x.device)

            def step():
                t0, t1 = tdev.index_select(0, i)[0], tdev.index_select(0, i + 1)[0]
                x.add_(((t1 - t0) * self.velocity(x, cond, text_ids, t0, feats)).to(x.dtype))
                i.add_(1)
            keep = x.clone()
            side = torch.cuda.Stream(device=x.device)
            side.wait_stream(torch.cuda.current_stream(x.device))
            with torch.cuda.stream(side):
                step()                                              # warm-up outside the graph; undone below
            torch.cuda.current_stream(x.device).wait_stream(side)
            g = torch.cuda.CUDAGraph()
            with torch.cuda.graph(g):
                step()
            x.copy_(keep), i.zero_()
            for _ in range(self.nfe):
                g.replay()
        else:
            for i in range(self.nfe):
                x = x + (ts[i + 1] - ts[i]) * self.velocity(x, cond, text_ids, ts[i], feats)
        x[:T_ref] = ref_mel
        return x


def load_into(m: DiT, loader, prefix: str = "ema_model.transformer.") -> None:
    """Names of the ``F5TTS_v1_Base`` checkpoint (docs/F5_ARCH.md of the reference lists them)."""
    dt = m.in_w.dtype

    def get(n):
        return loader.load_tensor(prefix + n, dt)

    def put(p, n):
        p.data.copy_(get(n).reshape(p.shape))
    put(m.text_embed, "text_embed.text_embed.weight")
    for i, b in enumerate(m.text_blocks):
        t = f"text_embed.text_blocks.{i}."
        for p, n in ((b.dw_w, "dwconv.weight"), (b.dw_b, "dwconv.bias"), (b.ln_w, "norm.weight"), (b.ln_b, "norm.bias"), (b.w1, "pwconv1.weight"),
                     (b.b1, "pwconv1.bias"), (b.w2, "pwconv2.weight"), (b.b2, "pwconv2.bias"), (b.grn_gamma, "grn.gamma"), (b.grn_beta, "grn.beta")):
            put(p, t + n)
    for p, n in ((m.in_w, "input_embed.proj.weight"), (m.in_b, "input_embed.proj.bias"), (m.pos1_w, "input_embed.conv_pos_embed.conv1d.0.weight"),
                 (m.pos1_b, "input_embed.conv_pos_embed.conv1d.0.bias"), (m.pos2_w, "input_embed.conv_pos_embed.conv1d.2.weight"),
                 (m.pos2_b, "input_embed.conv_pos_embed.conv1d.2.bias"), (m.t1_w, "time_embed.time_mlp.0.weight"), (m.t1_b, "time_embed.time_mlp.0.bias"),
                 (m.t2_w, "time_embed.time_mlp.2.weight"), (m.t2_b, "time_embed.time_mlp.2.bias"), (m.out_mod_w, "norm_out.linear.weight"),
                 (m.out_mod_b, "norm_out.linear.bias"), (m.out_w, "proj_out.weight"), (m.out_b, "proj_out.bias")):
        put(p, n)
    for i, b in enumerate(m.blocks):
        t = f"transformer_blocks.{i}."
        b.w_qkv.data.copy_(torch.cat([get(t + f"attn.to_{n}.weight") for n in "qkv"], 0))
        b.b_qkv.data.copy_(torch.cat([get(t + f"attn.to_{n}.bias") for n in "qkv"], 0))
        for p, n in ((b.w_o, "attn.to_out.0.weight"), (b.b_o, "attn.to_out.0.bias"), (b.mod_w, "attn_norm.linear.weight"), (b.mod_b, "attn_norm.linear.bias"),
                     (b.ff1_w, "ff.ff.0.0.weight"), (b.ff1_b, "ff.ff.0.0.bias"), (b.ff2_w, "ff.ff.2.weight"), (b.ff2_b, "ff.ff.2.bias")):
            put(p, t + n)


def init_random_(m: nn.Module, seed: int = 0, std: float = 0.1) -> None:
    g = torch.Generator().manual_seed(seed)
    for n, p in m.named_parameters():
        if p.dim() == 1:
            p.data.fill_(1.0 if n.endswith(("ln_w", "ln0_w", "lnf_w", "gamma")) else 0.0)
        else:
            p.data.normal_(0.0, std, generator=g)
