"""FLUX.2 autoencoder (src/models/flux/vae/*): convolutional encoder / decoder with ResNet blocks (GroupNorm 32, SiLU), one
single-head attention block in the middle, nearest-neighbour upsampling + convolution, 8x spatial factor, ``latent_channels``
channels; the diffusion model works on 2 x 2-patchified latents normalised by stored per-channel (BatchNorm) statistics."""
from __future__ import annotations

from dataclasses import dataclass

import torch
import torch.nn.functional as F
from torch import nn


@dataclass
class VAEConfig:
    channels: tuple = (128, 256, 512, 512)
    layers_per_block: int = 2
    latent_channels: int = 32
    groups: int = 32
    bn_eps: float = 1e-4

    @staticmethod
    def tiny():
        return VAEConfig(channels=(8, 16), layers_per_block=1, latent_channels=2, groups=4)


class ResBlock(nn.Module):
    def __init__(self, cin, cout, groups):
        super().__init__()
        self.n1, self.c1 = nn.GroupNorm(groups, cin, eps=1e-6), nn.Conv2d(cin, cout, 3, padding=1)
        self.n2, self.c2 = nn.GroupNorm(groups, cout, eps=1e-6), nn.Conv2d(cout, cout, 3, padding=1)
        self.skip = nn.Conv2d(cin, cout, 1) if cin != cout else None

    def forward(self, x):
        h = self.c2(F.silu(self.n2(self.c1(F.silu(self.n1(x))))))
        return (x if self.skip is None else self.skip(x)) + h


class AttnBlock(nn.Module):
    def __init__(self, ch, groups):
        super().__init__()
        self.norm = nn.GroupNorm(groups, ch, eps=1e-6)
        self.q, self.k, self.v, self.o = (nn.Linear(ch, ch) for _ in range(4))

    def forward(self, x):
        B, C, H, W = x.shape
        h = self.norm(x).flatten(2).transpose(1, 2)
        a = F.scaled_dot_product_attention(self.q(h)[:, None], self.k(h)[:, None], self.v(h)[:, None])[:, 0]
        return x + self.o(a).transpose(1, 2).view(B, C, H, W)


class Flux2VAE(nn.Module):
    def __init__(self, c: VAEConfig):
        super().__init__()
        self.c = c
        ch, g, L = c.channels, c.groups, c.latent_channels
        # encoder
        enc = [nn.Conv2d(3, ch[0], 3, padding=1)]
        cin = ch[0]
        for i, co in enumerate(ch):
            enc += [ResBlock(cin if j == 0 else co, co, g) for j in range(c.layers_per_block)]
            cin = co
            if i + 1 < len(ch):
                enc.append(nn.Conv2d(co, co, 3, stride=2, padding=0))            # fed an input padded by (0, 1, 0, 1)
        self.enc = nn.ModuleList(enc)
        self.enc_mid = nn.ModuleList([ResBlock(cin, cin, g), AttnBlock(cin, g), ResBlock(cin, cin, g)])
        self.enc_norm, self.enc_out = nn.GroupNorm(g, cin, eps=1e-6), nn.Conv2d(cin, 2 * L, 3, padding=1)
        self.quant_conv, self.post_quant_conv = nn.Conv2d(2 * L, 2 * L, 1), nn.Conv2d(L, L, 1)
        # decoder
        self.dec_in = nn.Conv2d(L, ch[-1], 3, padding=1)
        self.dec_mid = nn.ModuleList([ResBlock(ch[-1], ch[-1], g), AttnBlock(ch[-1], g), ResBlock(ch[-1], ch[-1], g)])
        dec, cin = [], ch[-1]
        for i, co in enumerate(reversed(ch)):
            dec += [ResBlock(cin if j == 0 else co, co, g) for j in range(c.layers_per_block + 1)]
            cin = co
            if i + 1 < len(ch):
                dec.append(nn.Conv2d(co, co, 3, padding=1))                      # after a 2x nearest upsample
        self.dec = nn.ModuleList(dec)
        self.dec_norm, self.dec_out = nn.GroupNorm(g, cin, eps=1e-6), nn.Conv2d(cin, 3, 3, padding=1)
        self.register_buffer("bn_mean", torch.zeros(4 * L))
        self.register_buffer("bn_var", torch.ones(4 * L))
        for p in self.parameters():
            p.requires_grad_(False)

    @property
    def scale_factor(self) -> int:
        return 2 ** (len(self.c.channels) - 1)

    def encode(self, image):
        """``image [B, 3, H, W]`` in [-1, 1] -> latent mean ``[B, L, H / f, W / f]``."""
        x = image
        for m in self.enc:
            if isinstance(m, nn.Conv2d) and m.stride == (2, 2):
                x = F.pad(x, (0, 1, 0, 1))
            x = m(x)
        for m in self.enc_mid:
            x = m(x)
        return self.quant_conv(self.enc_out(F.silu(self.enc_norm(x))))[:, :self.c.latent_channels]

    def decode(self, z):
        """``z [B, L, h, w]`` -> image ``[B, 3, h f, w f]`` in about [-1, 1]."""
        x = self.dec_in(self.post_quant_conv(z))
        for m in self.dec_mid:
            x = m(x)
        for m in self.dec:
            if isinstance(m, nn.Conv2d):
                x = F.interpolate(x, scale_factor=2.0, mode="nearest")
            x = m(x)
        return self.dec_out(F.silu(self.dec_norm(x)))

    # the diffusion model's view of the latent: 2 x 2 patches in the channel dim, standardised by the stored statistics
    def patchify(self, z):
        B, C, H, W = z.shape
        return z.view(B, C, H // 2, 2, W // 2, 2).permute(0, 1, 3, 5, 2, 4).reshape(B, 4 * C, H // 2, W // 2)

    def unpatchify(self, p):
        B, C4, h, w = p.shape
        return p.view(B, C4 // 4, 2, 2, h, w).permute(0, 1, 4, 2, 5, 3).reshape(B, C4 // 4, 2 * h, 2 * w)

    def normalize(self, p):
        return (p - self.bn_mean[None, :, None, None]) / torch.sqrt(self.bn_var[None, :, None, None] + self.c.bn_eps)

    def denormalize(self, p):
        return p * torch.sqrt(self.bn_var[None, :, None, None] + self.c.bn_eps) + self.bn_mean[None, :, None, None]


def load_into(m: Flux2VAE, loader) -> None:
    """Names of the ``AutoencoderKLFlux2`` checkpoint layout (``encoder.*``, ``decoder.*``, ``quant_conv``, ``post_quant_conv``, ``bn.*``)."""
    def put(mod, name):
        mod.weight.data.copy_(loader.load_tensor(name + ".weight", mod.weight.dtype))
        if mod.bias is not None:
            mod.bias.data.copy_(loader.load_tensor(name + ".bias", mod.bias.dtype))

    def res(r: ResBlock, p):
        put(r.n1, p + ".norm1"), put(r.c1, p + ".conv1"), put(r.n2, p + ".norm2"), put(r.c2, p + ".conv2")
        if r.skip is not None:
            put(r.skip, p + ".conv_shortcut")

    def mid(mods, p):
        res(mods[0], p + ".resnets.0"), res(mods[2], p + ".resnets.1")
        a = mods[1]
        put(a.norm, p + ".attentions.0.group_norm")
        for lin, n in ((a.q, "to_q"), (a.k, "to_k"), (a.v, "to_v"), (a.o, "to_out.0")):
            put(lin, p + ".attentions.0." + n)
    c = m.c
    put(m.enc[0], "encoder.conv_in")
    it = iter(m.enc[1:])
    for i in range(len(c.channels)):
        for j in range(c.layers_per_block):
            res(next(it), f"encoder.down_blocks.{i}.resnets.{j}")
        if i + 1 < len(c.channels):
            put(next(it), f"encoder.down_blocks.{i}.downsamplers.0.conv")
    mid(m.enc_mid, "encoder.mid_block")
    put(m.enc_norm, "encoder.conv_norm_out"), put(m.enc_out, "encoder.conv_out")
    put(m.quant_conv, "quant_conv"), put(m.post_quant_conv, "post_quant_conv")
    put(m.dec_in, "decoder.conv_in")
    mid(m.dec_mid, "decoder.mid_block")
    it = iter(m.dec)
    for i in range(len(c.channels)):
        for j in range(c.layers_per_block + 1):
            res(next(it), f"decoder.up_blocks.{i}.resnets.{j}")
        if i + 1 < len(c.channels):
            put(next(it), f"decoder.up_blocks.{i}.upsamplers.0.conv")
    put(m.dec_norm, "decoder.conv_norm_out"), put(m.dec_out, "decoder.conv_out")
    m.bn_mean.copy_(loader.load_tensor("bn.running_mean", torch.float32))
    m.bn_var.copy_(loader.load_tensor("bn.running_var", torch.float32))
