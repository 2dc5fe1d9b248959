"""Inkling in a pile: every tensor under its checkpoint name (``models.inkling.layout``), NVFP4 expert matrices as one blob per
(layer, expert, matrix) with ``layer`` / ``expert_index`` placement facts (src/models/inkling/pile.rs:343-466), ``config.json`` as
facts, so ``open(pile) -> decoder`` needs no side file (src/bin/inkling_forward.rs:2841-2854).  Loading goes through the
``Weights`` facade (admission before the first copy, one registration of the mapping, counters)."""
from __future__ import annotations

import numpy as np
import torch

from ...format import jsonfacts
from ...format.ingest import f32_to_bf16_bits
from ...format.leaf import Elem
from ...format.model import build_model_root, put_fp4_tensor, put_tensor
from ...format.persist import publish_fragment
from ...ops.moe import NVFP4Experts, swizzle_scales, unswizzle_scales
from ...pile.trible import TribleBuilder
from .config import InklingConfig
from .decoder import InklingDecoder
from .source import Weights


def save_to_pile(pile, key, dec: InklingDecoder, name: str = "inkling") -> bytes:
    tb = TribleBuilder()
    members = []
    for n, p in dec.P.items():
        a = p.detach().float().cpu().numpy()
        bf = p.dtype in (torch.bfloat16, torch.float32) and not n.endswith(("gate.bias", "gate.global_scale"))
        members.append(put_tensor(pile, tb, n, f32_to_bf16_bits(a) if bf else a, Elem.BF16 if bf else None))
    t = dec.t
    for layer in range(dec.n_llm):
        if t.is_dense(layer):
            continue
        ex = dec._experts(layer)
        if isinstance(ex, NVFP4Experts):
            for which, q, sf, s2, rows, K in (("w13", ex.w13_q, ex.w13_sf, ex.w13_s2, 2 * ex.F, ex.H), ("w2", ex.w2_q, ex.w2_sf, ex.w2_s2, ex.H, ex.F)):
                for e in range(ex.E):
                    codes = q[e * rows:(e + 1) * rows].cpu().numpy()
                    sc = unswizzle_scales(sf[e * rows // 128:(e + 1) * rows // 128].cpu(), rows, K // 16).numpy()
                    members.append(put_fp4_tensor(pile, tb, f"model.llm.layers.{layer}.mlp.experts.{e}.{which}_weight", codes,
                                                  np.ascontiguousarray(sc), float(s2[e]), layer=layer, expert=e))
        else:
            for which, w in (("w13", ex[0]), ("w2", ex[1])):
                members.append(put_tensor(pile, tb, f"model.llm.layers.{layer}.mlp.experts.{which}_weight.bf16",
                                          f32_to_bf16_bits(w.detach().float().cpu().numpy()), Elem.BF16))
    root = build_model_root(pile, tb, members, name=name, source="mary_b200", quantization="nvfp4")
    doc = dec.cfg.to_json()
    doc["quantized_moe_layers"] = sorted(dec.quantized)
    jsonfacts.save_document(pile, tb, "config.json", doc, owner=root)
    publish_fragment(pile, key, tb.build(), f"inkling {name}"[:32])
    return root


def load_from_pile(pile, device="cpu", dtype=torch.bfloat16, max_slots: int = 8, other_bytes: int = 0, weights: Weights | None = None):
    """Config-free load.  Returns ``(decoder, weights facade)``.  On a CUDA device the share is admitted against the free memory
    before the first copy and the mapping is registered once for direct copies."""
    w = weights or Weights.open(pile)
    doc = w.document("config.json")
    cfg = InklingConfig.from_json(doc)
    quantized = set(doc.get("quantized_moe_layers", []))
    dec = InklingDecoder(cfg, quantized=quantized, dtype=dtype, device=device, max_slots=max_slots)
    dev = torch.device(device)
    if dev.type == "cuda":
        free, _ = torch.cuda.mem_get_info(dev)
        w.admit(w.names(), other_bytes, free)
        w.register()
    t = cfg.text_config
    expert_names = {}
    for n in w.names():
        if ".mlp.experts." in n:
            expert_names[n] = True
            continue
        dec.set_tensor(n, w.tensor(n, device))
    placement = w.index.experts_in_layers(0, t.num_hidden_layers)
    for layer in range(t.num_hidden_layers):
        if t.is_dense(layer):
            continue
        if layer in quantized:
            parts = {"w13": [], "w2": []}
            for e in range(t.n_routed_experts):
                names = placement[(layer, e)]
                for which in ("w13", "w2"):
                    c, s, s2 = w.expert_packed([x for x in names if x.endswith(f".{which}_weight")][0], "cpu")
                    parts[which].append((c, swizzle_scales(s), s2))
            cat = lambda m, i: torch.cat([p[i] for p in parts[m]], 0).to(device)  # noqa: E731
            s2v = lambda m: torch.tensor([p[2] for p in parts[m]], dtype=torch.float32, device=device)  # noqa: E731
            dec.set_experts_nvfp4(layer, NVFP4Experts(t.n_routed_experts, t.hidden_size, t.intermediate_size, cat("w13", 0), cat("w13", 1),
                                                      s2v("w13"), cat("w2", 0), cat("w2", 1), s2v("w2"), "swiglu"))
        else:
            d = dec._derived.setdefault(("expert_dense", layer), {})
            for which in ("w13", "w2"):
                d[which] = w.tensor(f"model.llm.layers.{layer}.mlp.experts.{which}_weight.bf16", device, dtype)
    return dec, w
