"""Checkpoint-name loaders of the families without an installed oracle: every parameter is covered by exactly the names of the
published layouts (a parameter left untouched stays NaN and fails), and fused projections are concatenated in q, k, v order."""
import torch

from mary_b200.models.f5 import DiT, F5Config
from mary_b200.models.f5 import dit as f5_dit
from mary_b200.models.flux import Flux2Config, Flux2Transformer, Flux2VAE, VAEConfig
from mary_b200.models.flux import transformer as flux_tr
from mary_b200.models.flux import vae as flux_vae


class _Recorder:
    """Hands out random tensors of whatever shape is asked for by recording names first (shape unknown), so the test drives the
    loader twice: once to learn the names, once with tensors of the shapes the published checkpoints have."""

    def __init__(self, shapes):
        g = torch.Generator().manual_seed(0)
        self.sd = {n: torch.randn(*s, generator=g) for n, s in shapes.items()}
        self.asked = []

    def load_tensor(self, n, dtype):
        self.asked.append(n)
        return self.sd[n].to(dtype)


def _nan(m):
    for p in m.parameters():
        p.data.fill_(float("nan"))
    return m


def test_flux_transformer_names():
    c = Flux2Config.tiny(guidance=True)
    D, M, hd = c.dim, c.mlp, c.head_dim
    shapes = {"time_guidance_embed.timestep_embedder.linear_1.weight": (D, c.time_channels), "time_guidance_embed.timestep_embedder.linear_2.weight": (D, D),
              "time_guidance_embed.guidance_embedder.linear_1.weight": (D, c.time_channels), "time_guidance_embed.guidance_embedder.linear_2.weight": (D, D),
              "double_stream_modulation_img.linear.weight": (6 * D, D), "double_stream_modulation_txt.linear.weight": (6 * D, D),
              "single_stream_modulation.linear.weight": (3 * D, D), "x_embedder.weight": (D, c.in_channels), "context_embedder.weight": (D, c.joint_dim),
              "norm_out.linear.weight": (2 * D, D), "proj_out.weight": (c.in_channels, D)}
    for i in range(c.layers):
        a = f"transformer_blocks.{i}."
        for n in ("to_q", "to_k", "to_v", "add_q_proj", "add_k_proj", "add_v_proj", "to_out.0", "to_add_out"):
            shapes[a + f"attn.{n}.weight"] = (D, D)
        for n in ("norm_q", "norm_k", "norm_added_q", "norm_added_k"):
            shapes[a + f"attn.{n}.weight"] = (hd,)
        for ff in ("ff", "ff_context"):
            shapes[a + ff + ".linear_in.weight"], shapes[a + ff + ".linear_out.weight"] = (2 * M, D), (D, M)
    for i in range(c.single_layers):
        a = f"single_transformer_blocks.{i}.attn."
        shapes[a + "to_qkv_mlp_proj.weight"], shapes[a + "to_out.weight"] = (3 * D + 2 * M, D), (D, D + M)
        shapes[a + "norm_q.weight"], shapes[a + "norm_k.weight"] = (hd,), (hd,)
    rec = _Recorder(shapes)
    m = _nan(Flux2Transformer(c))
    flux_tr.load_into(m, rec)
    assert sorted(rec.asked) == sorted(shapes) and not any(torch.isnan(p).any() for p in m.parameters())
    b = m.double_blocks[1]
    assert torch.equal(b.txt_qkv[D:2 * D], rec.sd["transformer_blocks.1.attn.add_k_proj.weight"])


def test_flux_vae_names():
    c = VAEConfig.tiny()
    # the published layout, spelled out for the tiny geometry (2 levels, 1 layer per block)
    names = ["encoder.conv_in", "encoder.down_blocks.0.resnets.0.norm1", "encoder.down_blocks.0.resnets.0.conv1", "encoder.down_blocks.0.resnets.0.norm2",
             "encoder.down_blocks.0.resnets.0.conv2", "encoder.down_blocks.0.downsamplers.0.conv", "encoder.down_blocks.1.resnets.0.norm1",
             "encoder.down_blocks.1.resnets.0.conv1", "encoder.down_blocks.1.resnets.0.norm2", "encoder.down_blocks.1.resnets.0.conv2",
             "encoder.down_blocks.1.resnets.0.conv_shortcut", "encoder.conv_norm_out", "encoder.conv_out", "quant_conv", "post_quant_conv",
             "decoder.conv_in", "decoder.conv_norm_out", "decoder.conv_out", "decoder.up_blocks.0.upsamplers.0.conv"]
    for side in ("encoder", "decoder"):
        for r in ("resnets.0", "resnets.1"):
            names += [f"{side}.mid_block.{r}.{n}" for n in ("norm1", "conv1", "norm2", "conv2")]
        names += [f"{side}.mid_block.attentions.0.{n}" for n in ("group_norm", "to_q", "to_k", "to_v", "to_out.0")]
    for i, shortcut in ((0, ()), (1, (0,))):
        for j in range(2):
            names += [f"decoder.up_blocks.{i}.resnets.{j}.{n}" for n in ("norm1", "conv1", "norm2", "conv2")]
            if j in shortcut:
                names.append(f"decoder.up_blocks.{i}.resnets.{j}.conv_shortcut")
    want = {n + s for n in names for s in (".weight", ".bias")} | {"bn.running_mean", "bn.running_var"}

    class Scalars:
        """Answers every name with a 0-dim tensor (``copy_`` broadcasts it), so the test needs no table of shapes."""
        asked = []

        def load_tensor(self, n, dtype):
            self.asked.append(n)
            return torch.tensor(float(len(self.asked)), dtype=dtype)
    probe = _nan(Flux2VAE(c))
    ld = Scalars()
    flux_vae.load_into(probe, ld)
    assert set(ld.asked) == want and len(ld.asked) == len(want)
    assert not any(torch.isnan(p).any() for p in probe.parameters())
    assert float(probe.bn_var[0]) == float(len(ld.asked))


def test_f5_names():
    c = F5Config.tiny()
    m = _nan(DiT(c))
    D, Fd, T, I = c.dim, c.dim * c.ff_mult, c.text_dim, c.text_dim * c.conv_mult
    pre = "ema_model.transformer."
    shapes = {"text_embed.text_embed.weight": (c.text_vocab, T), "input_embed.proj.weight": (D, 2 * c.n_mels + T), "input_embed.proj.bias": (D,),
              "input_embed.conv_pos_embed.conv1d.0.weight": (D, D // c.pos_groups, c.pos_kernel), "input_embed.conv_pos_embed.conv1d.0.bias": (D,),
              "input_embed.conv_pos_embed.conv1d.2.weight": (D, D // c.pos_groups, c.pos_kernel), "input_embed.conv_pos_embed.conv1d.2.bias": (D,),
              "time_embed.time_mlp.0.weight": (D, c.time_freq), "time_embed.time_mlp.0.bias": (D,), "time_embed.time_mlp.2.weight": (D, D),
              "time_embed.time_mlp.2.bias": (D,), "norm_out.linear.weight": (2 * D, D), "norm_out.linear.bias": (2 * D,),
              "proj_out.weight": (c.n_mels, D), "proj_out.bias": (c.n_mels,)}
    for i in range(c.conv_layers):
        t = f"text_embed.text_blocks.{i}."
        shapes.update({t + "dwconv.weight": (T, 1, 7), t + "dwconv.bias": (T,), t + "norm.weight": (T,), t + "norm.bias": (T,),
                       t + "pwconv1.weight": (I, T), t + "pwconv1.bias": (I,), t + "pwconv2.weight": (T, I), t + "pwconv2.bias": (T,),
                       t + "grn.gamma": (1, 1, I), t + "grn.beta": (1, 1, I)})
    for i in range(c.depth):
        t = f"transformer_blocks.{i}."
        for n in ("to_q", "to_k", "to_v", "to_out.0"):
            shapes[t + f"attn.{n}.weight"], shapes[t + f"attn.{n}.bias"] = (D, D), (D,)
        shapes.update({t + "attn_norm.linear.weight": (6 * D, D), t + "attn_norm.linear.bias": (6 * D,), t + "ff.ff.0.0.weight": (Fd, D),
                       t + "ff.ff.0.0.bias": (Fd,), t + "ff.ff.2.weight": (D, Fd), t + "ff.ff.2.bias": (D,)})
    rec = _Recorder({pre + k: v for k, v in shapes.items()})
    f5_dit.load_into(m, rec)
    assert sorted(rec.asked) == sorted(pre + k for k in shapes) and not any(torch.isnan(p).any() for p in m.parameters())
    assert torch.equal(m.blocks[0].w_qkv[2 * D:], rec.sd[pre + "transformer_blocks.0.attn.to_v.weight"])
