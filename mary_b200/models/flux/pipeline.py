"""FLUX.2 text-to-image pipeline (src/models/flux/pipeline.rs): encode the prompt, denoise packed latents with the flow
scheduler, un-normalise, un-patchify and decode.  The three components are used one after the other, so a caller that is short
of memory can build, use and drop each in turn; ``Flux2Transformer.forward(blocks=...)`` additionally streams block weights.

Text features are the concatenated hidden states of three intermediate decoder layers of the language model (Qwen3 layers
9 / 18 / 27 for the step-distilled 4B variant, Mistral layers 10 / 20 / 30 for the guidance-distilled one), which is why
``joint_dim`` is three times the encoder's width."""
from __future__ import annotations

import torch

from .scheduler import FlowMatchEuler
from .transformer import Flux2Transformer
from .vae import Flux2VAE


def pack_latents(z):
    """``[C, h, w] -> [h w, C]`` (one token per latent position, row-major)."""
    return z.flatten(1).T.contiguous()


def unpack_latents(tokens, h: int, w: int):
    return tokens.T.reshape(-1, h, w)


def position_ids(h: int = 0, w: int = 0, n_text: int = 0):
    """``(t, h, w, l)`` ids: image tokens carry their row and column, text tokens their index in the last axis."""
    if n_text:
        ids = torch.zeros(n_text, 4, dtype=torch.long)
        ids[:, 3] = torch.arange(n_text)
        return ids
    ids = torch.zeros(h, w, 4, dtype=torch.long)
    ids[..., 1] = torch.arange(h)[:, None]
    ids[..., 2] = torch.arange(w)[None, :]
    return ids.reshape(h * w, 4)


def encode_prompt(model, ids, layers):
    """Concatenate the hidden states after decoder layers ``layers`` (1-based, like the checkpoints' hidden-state indices) of a
    ``MistralModel``-shaped encoder run once over ``ids`` -> ``[T, len(layers) * hidden]``."""
    from ...runtime.batch import BatchMeta
    from ...runtime.kv_cache import PagedKVCache
    spec = model.kv_spec()
    n = len(ids)
    cache = PagedKVCache(spec["num_layers"], n // 16 + 2, 16, spec["kv_heads"], spec["head_dim"], dtype=model.dtype, device=model.embed.device)
    cache.alloc.extend(0, n)
    table, lens = cache.alloc.page_table([0])
    meta = BatchMeta.build([n], lens, table, 16, device=model.embed.device)
    with torch.no_grad():
        states = model.layer_states(torch.as_tensor(ids, dtype=torch.int32, device=model.embed.device), meta, cache, set(layers))
    return torch.cat([states[i] for i in layers], -1)


class FluxPipeline:
    def __init__(self, transformer: Flux2Transformer, vae: Flux2VAE, guidance_scale: float = 4.0):
        self.tr, self.vae, self.guidance_scale = transformer, vae, guidance_scale

    @torch.no_grad()
    def __call__(self, text_features, height: int, width: int, steps: int = 4, seed: int = 0, noise=None):
        """``text_features [S_txt, joint_dim]`` -> image ``[3, height, width]`` in [0, 1]."""
        f = self.vae.scale_factor * 2                                    # pixels per packed latent position
        height, width = height // f * f, width // f * f                 # align to whole packed positions
        h, w = height // f, width // f
        C = self.tr.c.in_channels
        if noise is None:
            noise = torch.randn(C, h, w, generator=torch.Generator().manual_seed(seed))
        x = pack_latents(noise.to(self.tr.x_embed.device, self.tr.x_embed.dtype))
        img_ids, txt_ids = position_ids(h, w), position_ids(n_text=text_features.shape[0])
        sched = FlowMatchEuler(steps, h * w)
        g = torch.tensor([self.guidance_scale], device=x.device) if self.tr.c.guidance_embeds else None
        for _ in range(steps):
            v = self.tr(x, text_features, sched.t, img_ids, txt_ids, guidance=g)
            x = sched.step(v, x)
        p = self.vae.denormalize(unpack_latents(x.float(), h, w)[None])
        img = self.vae.decode(self.vae.unpatchify(p))[0]
        return (img / 2 + 0.5).clamp(0, 1)
