"""MoE decoders in a pile: NVFP4 expert matrices as ONE blob ``[codes][scales][scale2]`` each with ``layer`` /
``expert_index`` placement facts (src/models/inkling/pile.rs:343-466), everything else as BF16 leaves, the configuration as
``config.json`` facts — so ``open(pile) -> model`` needs no side files (src/bin/inkling_forward.rs:2841-2854).  Which experts a
rank loads is a QUERY over the placement facts (pile.rs:514-549), not a file layout."""
from __future__ import annotations

import numpy as np
import torch

from ...format import jsonfacts
from ...format.ingest import f32_to_bf16_bits
from ...format.leaf import Elem
from ...format.model import build_model_root, put_fp4_tensor, put_tensor
from ...format.persist import load_config, publish_fragment, read_model_pile
from ...format.selection import SelectedModelIndex
from ...ops.moe import NVFP4Experts, swizzle_scales, unswizzle_scales
from ...pile.trible import TribleBuilder
from .config import MoEConfig
from .model import MoEDecoder, MoEFFN


def _moe_modules(model):
    return [(n, m) for n, m in model.named_modules() if isinstance(m, MoEFFN)]


def save_to_pile(pile, key, model: MoEDecoder, name: str = "moe") -> bytes:
    """Single-rank model -> pile.  Returns the model root id."""
    tb = TribleBuilder()
    members = []
    for n, p in model.named_parameters():
        a = p.detach().float().cpu().numpy()
        members.append(put_tensor(pile, tb, n, f32_to_bf16_bits(a) if p.dtype == torch.bfloat16 else a,
                                  Elem.BF16 if p.dtype == torch.bfloat16 else None))
    for li, (n, m) in enumerate(_moe_modules(model)):
        ex = m.experts
        for which, q, sf, s2, rows, K in (("w13", ex.w13_q, ex.w13_sf, ex.w13_s2, 2 * ex.F, ex.H), ("w2", ex.w2_q, ex.w2_sf, ex.w2_s2, ex.H, ex.F)):
            for e in range(ex.E):
                codes = q[e * rows:(e + 1) * rows].cpu().numpy()
                sc = unswizzle_scales(sf[e * rows // 128:(e + 1) * rows // 128].cpu(), rows, K // 16).numpy()
                members.append(put_fp4_tensor(pile, tb, f"{n}.experts.{e}.{which}", codes, np.ascontiguousarray(sc), float(s2[e]),
                                              layer=li, expert=e))
    root = build_model_root(pile, tb, members, name=name, source="mary_b200", quantization="nvfp4")
    jsonfacts.save_document(pile, tb, "config.json", model.cfg.to_json(), owner=root)
    publish_fragment(pile, key, tb.build(), f"moe {name}"[:32])
    return root


def load_from_pile(pile, par=None, device="cpu", dtype=torch.bfloat16) -> MoEDecoder:
    """Config-free load; an expert-parallel rank reads only the experts its placement query returns."""
    facts = read_model_pile(pile)
    index = SelectedModelIndex.from_snapshot(pile, facts)
    cfg = MoEConfig.from_json(load_config(pile, facts, index.roots[0]))
    full_par = par
    model = MoEDecoder(cfg, par=full_par, dtype=dtype, device=device)
    from .shard import cut_parameter
    mods = dict(model.named_modules())
    tp_r, tp_n = model.par.tp_rank, model.par.tp_size
    with torch.no_grad():
        for n, p in model.named_parameters():
            # one full tensor at a time on the host; a tensor-parallel rank keeps its slice only (the same rule that cuts a model
            # in memory), so no rank ever holds the whole model
            leaf = index.leaf(n)
            t = leaf.torch() if leaf.elem in (Elem.BF16, Elem.F32, Elem.F16) else torch.from_numpy(leaf.to_f32())
            t = cut_parameter(cfg, mods.get(n.rpartition(".")[0]), n, t, tp_r, tp_n, getattr(model, "vocab_parallel", False))
            if tuple(t.shape) != tuple(p.shape):
                raise ValueError(f"{n}: the pile holds {tuple(t.shape)} after cutting for rank {tp_r} of {tp_n}, the model wants {tuple(p.shape)}")
            p.copy_(t.to(dtype if p.dtype == dtype else p.dtype))
    moes = _moe_modules(model)
    placement = index.experts_in_layers(0, len(moes))
    for li, (n, m) in enumerate(moes):
        n_tail = 1 if m.shared_in_experts else 0
        wanted = list(range(m.e0, m.e0 + m.e_local)) + ([cfg.n_routed_experts] if n_tail else [])
        parts = {"w13": [], "w2": []}
        for e in wanted:
            names = placement[(li, e)]
            for which in ("w13", "w2"):
                leaf = index.leaf([x for x in names if x.endswith("." + which)][0])
                codes, sc, s2 = leaf.fp4_parts()
                parts[which].append((torch.from_numpy(np.array(codes)), swizzle_scales(torch.from_numpy(np.array(sc))), s2))
        cat = lambda w, i: torch.cat([p[i] for p in parts[w]], 0).to(device)  # noqa: E731
        s2 = lambda w: torch.tensor([p[2] for p in parts[w]], dtype=torch.float32, device=device)  # noqa: E731
        m.experts = NVFP4Experts(len(wanted), cfg.hidden_size, cfg.moe_intermediate_size, cat("w13", 0), cat("w13", 1), s2("w13"),
                                 cat("w2", 0), cat("w2", 1), s2("w2"), cfg.act)
    return model
