"""The Inkling checkpoint layout: every tensor name of the four towers and the slot it fills (src/models/inkling/layout.rs).

Names, shapes and dtypes only.  As for the K3 layout the mapping exists twice, in opposite directions and without shared code:
:func:`slots` walks a configuration and formats the name every slot expects; :func:`parse` recovers the slot from a name with
anchored regular expressions.  Four towers share one namespace (``model.llm``, ``model.mtp``, ``model.visual``, ``model.audio``)
and all use ``layers.`` in their names, so every pattern is anchored to its tower (layout.rs:8-13).

Whether a MoE layer's experts are NVFP4 or bf16 is NOT in ``config.json`` (the released small checkpoint leaves layer 2 in
bf16): the caller supplies the set of quantised layers, and :func:`check_headers` asserts the structural invariant instead —
a layer carries all four quantisation sidecars of a matrix or none (layout.rs:15-21).

A slot is a tuple: ``("embed",)``, ``("embed_norm",)``, ``("final_norm",)``, ``("unembed",)``, ``("llm", i, part...)``,
``("mtp", i, part...)``, ``("vision", part, [i])``, ``("audio", part)``; a block part is ``("attn_norm",)``, ``("attn", "wq")``,
``("mlp", "dense", "w13")``, ``("mlp", "moe", "expert", "w13", "scale")`` and so on.  Shapes are in checkpoint order."""
from __future__ import annotations

import re

from .config import GLOBAL, InklingConfig

BF16, F32, U8, F8E4M3, I64 = "BF16", "F32", "U8", "F8_E4M3", "I64"
NVFP4_GROUP = 16

ATTN_NAMES = {"wq": "wq_du.weight", "wk": "wk_dv.weight", "wv": "wv_dv.weight", "wo": "wo_ud.weight", "wr": "wr_du.weight",
              "rel_proj": "rel_logits_proj.proj", "q_norm": "q_norm.weight", "k_norm": "k_norm.weight", "k_sconv": "k_sconv.weight",
              "v_sconv": "v_sconv.weight"}
QUANT_SUFFIX = {"weight": "", "scale": ".scale", "scale2": ".scale2", "input_amax": ".input_amax", "original_shape": ".original_shape"}
SIDECARS = ("scale", "scale2", "input_amax", "original_shape")


# ------------------------------------------------------------------------------------------------ slot -> name (formatting)
def _block_name(part: tuple) -> str:
    if part[0] in ("attn_norm", "attn_sconv", "mlp_norm", "mlp_sconv"):
        return part[0] + ".weight"
    if part[0] == "attn":
        return "attn." + ATTN_NAMES[part[1]]
    if part[:2] == ("mlp", "dense"):
        return {"w13": "mlp.w13_dn.weight", "w2": "mlp.w2_md.weight", "global_scale": "mlp.global_scale"}[part[2]]
    if part[:2] == ("mlp", "moe"):
        if part[2] == "expert":
            return f"mlp.experts.{part[3]}_weight{QUANT_SUFFIX[part[4]]}"
        return {"gate_weight": "mlp.gate.weight", "gate_bias": "mlp.gate.bias", "gate_global_scale": "mlp.gate.global_scale",
                "shared_w13": "mlp.shared_experts.shared_w13_weight", "shared_w2": "mlp.shared_experts.shared_w2_weight"}[part[2]]
    raise KeyError(part)


def tensor_name(slot: tuple) -> str:
    head = slot[0]
    if head in ("embed", "embed_norm", "unembed"):
        return f"model.llm.{head}.weight"
    if head == "final_norm":
        return "model.llm.norm.weight"
    if head == "llm":
        return f"model.llm.layers.{slot[1]}.{_block_name(slot[2:])}"
    if head == "mtp":
        if slot[2] in ("embed_norm", "hidden_norm", "input_proj"):
            return f"model.mtp.layers.{slot[1]}.{slot[2]}.weight"
        return f"model.mtp.layers.{slot[1]}.transformer_block.{_block_name(slot[3:])}"
    if head == "vision":
        return "model.visual.final_norm.weight" if slot[1] == "final_norm" else f"model.visual.layers.{slot[1]}_{slot[2]}.weight"
    if head == "audio":
        return f"model.audio.{slot[1]}.weight"
    raise KeyError(slot)


# ------------------------------------------------------------------------------------------------ name -> slot (regular expressions)
_RE_TOP = re.compile(r"^model\.llm\.(embed|embed_norm|norm|unembed)\.weight$")
_RE_LLM = re.compile(r"^model\.llm\.layers\.(\d+)\.(.+)$")
_RE_MTP = re.compile(r"^model\.mtp\.layers\.(\d+)\.(?:(embed_norm|hidden_norm|input_proj)\.weight|transformer_block\.(.+))$")
_RE_VIS = re.compile(r"^model\.visual\.(?:final_norm\.weight|layers\.(linear|norm)_(\d+)\.weight)$")
_RE_AUD = re.compile(r"^model\.audio\.(encoder|final_norm)\.weight$")
_RE_BLOCK_PLAIN = re.compile(r"^(attn_norm|attn_sconv|mlp_norm|mlp_sconv)\.weight$")
_RE_ATTN = re.compile(r"^attn\.(wq_du|wk_dv|wv_dv|wo_ud|wr_du|q_norm|k_norm|k_sconv|v_sconv)\.weight$|^attn\.(rel_logits_proj)\.proj$")
_RE_EXPERT = re.compile(r"^mlp\.experts\.(w13|w2)_weight(?:\.(scale2|scale|input_amax|original_shape))?$")
_ATTN_BACK = {"wq_du": "wq", "wk_dv": "wk", "wv_dv": "wv", "wo_ud": "wo", "wr_du": "wr", "q_norm": "q_norm", "k_norm": "k_norm",
              "k_sconv": "k_sconv", "v_sconv": "v_sconv", "rel_logits_proj": "rel_proj"}
_MLP_BACK = {"mlp.w13_dn.weight": ("mlp", "dense", "w13"), "mlp.w2_md.weight": ("mlp", "dense", "w2"), "mlp.global_scale": ("mlp", "dense", "global_scale"),
             "mlp.gate.weight": ("mlp", "moe", "gate_weight"), "mlp.gate.bias": ("mlp", "moe", "gate_bias"),
             "mlp.gate.global_scale": ("mlp", "moe", "gate_global_scale"), "mlp.shared_experts.shared_w13_weight": ("mlp", "moe", "shared_w13"),
             "mlp.shared_experts.shared_w2_weight": ("mlp", "moe", "shared_w2")}


def _parse_block(tail: str):
    m = _RE_BLOCK_PLAIN.match(tail)
    if m:
        return (m.group(1),)
    m = _RE_ATTN.match(tail)
    if m:
        return ("attn", _ATTN_BACK[m.group(1) or m.group(2)])
    if tail in _MLP_BACK:
        return _MLP_BACK[tail]
    m = _RE_EXPERT.match(tail)
    if m:
        return ("mlp", "moe", "expert", m.group(1), m.group(2) or "weight")
    return None


def parse(name: str):
    """The slot a checkpoint name fills, or ``None`` for a name this layout does not know."""
    m = _RE_TOP.match(name)
    if m:
        return ("final_norm",) if m.group(1) == "norm" else (m.group(1),)
    m = _RE_LLM.match(name)
    if m:
        b = _parse_block(m.group(2))
        return None if b is None else ("llm", int(m.group(1))) + b
    m = _RE_MTP.match(name)
    if m:
        if m.group(2):
            return ("mtp", int(m.group(1)), m.group(2))
        b = _parse_block(m.group(3))
        return None if b is None else ("mtp", int(m.group(1)), "block") + b
    m = _RE_VIS.match(name)
    if m:
        return ("vision", "final_norm") if m.group(1) is None else ("vision", m.group(1), int(m.group(2)))
    m = _RE_AUD.match(name)
    if m:
        return ("audio", m.group(1))
    return None


# ------------------------------------------------------------------------------------------------ shapes and dtypes from the config
def _grouping_factor(vc, i: int):
    """How many previous-stage vectors stage ``i`` folds into one: the sub-patches of a frame are folded in equal geometric steps
    (64 = 4 x 16 on the released models, layout.rs:560-573)."""
    per_frame = (vc.patch_size // vc.subpatch_size) ** 2
    stages = vc.n_layers - 1
    if (per_frame, stages) == (64, 3):
        return [4, 16][i - 1] if 1 <= i <= 2 else None
    return None


def _describe_block(cfg: InklingConfig, quantized: set, layer: int, dense: bool, kind: str, part: tuple):
    t = cfg.text_config
    k, H = t.sconv_kernel_size, t.hidden_size
    if part[0] in ("attn_norm", "mlp_norm"):
        return (H,), BF16
    if part[0] in ("attn_sconv", "mlp_sconv"):
        return (H, 1, k), BF16
    if part[0] == "attn":
        a = part[1]
        return {"wq": ((t.q_dim(kind), H), BF16), "wk": ((t.kv_dim(kind), H), BF16), "wv": ((t.kv_dim(kind), H), BF16),
                "wo": ((H, t.q_dim(kind)), BF16), "wr": ((t.rel_dim(kind), H), BF16), "rel_proj": ((t.d_rel, t.rel_span(kind)), BF16),
                "q_norm": ((t.norm_dim(kind),), BF16), "k_norm": ((t.norm_dim(kind),), BF16), "k_sconv": ((t.kv_dim(kind), 1, k), BF16),
                "v_sconv": ((t.kv_dim(kind), 1, k), BF16)}[a]
    if part[:2] == ("mlp", "dense"):
        if not dense:
            return None
        return {"w13": ((2 * t.dense_intermediate_size, H), BF16), "w2": ((H, t.dense_intermediate_size), BF16), "global_scale": ((1,), BF16)}[part[2]]
    if part[:2] == ("mlp", "moe"):
        if dense:
            return None
        E, F = t.n_routed_experts, t.intermediate_size
        m = part[2]
        if m == "gate_weight":
            return (t.gate_rows(), H), BF16
        if m == "gate_bias":
            return (E,), F32
        if m == "gate_global_scale":
            return (1,), F32
        if m == "shared_w13":
            return (t.n_shared_experts, H, 2 * F), BF16
        if m == "shared_w2":
            return (t.n_shared_experts, H, F), BF16
        mat, q = part[3], part[4]
        logical = 2 * F if mat == "w13" else F
        if layer not in quantized:
            return ((E, H, logical), BF16) if q == "weight" else None          # a bf16 layer carries no sidecars
        return {"weight": ((E, H, logical // 2), U8), "scale": ((E, H, logical // NVFP4_GROUP), F8E4M3), "scale2": ((E,), F32),
                "input_amax": ((1,), BF16), "original_shape": ((3,), I64)}[q]
    return None


def describe(cfg: InklingConfig, quantized: set, slot: tuple):
    """``(shape, dtype)`` the configuration prescribes for ``slot``, or ``None`` when the model has no such slot."""
    t = cfg.text_config
    head = slot[0]
    if head in ("embed", "unembed"):
        return (t.vocab_size, t.hidden_size), BF16
    if head in ("embed_norm", "final_norm"):
        return (t.hidden_size,), BF16
    if head == "vision":
        vc = cfg.vision_config
        if slot[1] == "final_norm":
            return (vc.decoder_dmodel,), BF16
        i = slot[2]
        if slot[1] == "norm":
            return ((vc.hidden_dims[i],), BF16) if i < len(vc.hidden_dims) else None
        if i >= vc.n_layers:
            return None
        out = vc.decoder_dmodel if i + 1 == vc.n_layers else (vc.hidden_dims[i] if i < len(vc.hidden_dims) else None)
        if i == 0:
            inp = vc.subpatch_elems()
        elif i + 1 == vc.n_layers:
            inp = vc.patch_elems()
        else:
            g = _grouping_factor(vc, i)
            inp = None if g is None else vc.hidden_dims[i - 1] * g
        return None if out is None or inp is None else ((out, inp), BF16)
    if head == "audio":
        ac = cfg.audio_config
        return ((ac.encoder_rows(), ac.decoder_dmodel), BF16) if slot[1] == "encoder" else ((ac.decoder_dmodel,), BF16)
    if head == "llm":
        i = slot[1]
        return None if i >= t.num_hidden_layers else _describe_block(cfg, quantized, i, t.is_dense(i), t.attn_kind(i), slot[2:])
    if head == "mtp":
        i = slot[1]
        if i >= cfg.mtp_config.num_nextn_predict_layers:
            return None
        if slot[2] in ("embed_norm", "hidden_norm"):
            return (t.hidden_size,), BF16
        if slot[2] == "input_proj":
            return (t.hidden_size, 2 * t.hidden_size), BF16
        return _describe_block(cfg, quantized, i, True, cfg.mtp_config.attn_kind(i), slot[3:])       # every MTP block is dense
    return None


def _block_parts(dense: bool, quantized_layer: bool):
    yield ("attn_norm",)
    yield ("attn_sconv",)
    yield ("mlp_norm",)
    yield ("mlp_sconv",)
    for a in ATTN_NAMES:
        yield ("attn", a)
    if dense:
        for d in ("w13", "w2", "global_scale"):
            yield ("mlp", "dense", d)
    else:
        for m in ("gate_weight", "gate_bias", "gate_global_scale", "shared_w13", "shared_w2"):
            yield ("mlp", "moe", m)
        for mat in ("w13", "w2"):
            yield ("mlp", "moe", "expert", mat, "weight")
            if quantized_layer:
                for q in SIDECARS:
                    yield ("mlp", "moe", "expert", mat, q)


def slots(cfg: InklingConfig, quantized: set | None = None):
    """Every slot of the four towers with ``(slot, name, shape, dtype)`` (layout.rs:654 ``for_each_slot``).  ``quantized``: the
    MoE layers whose experts are NVFP4 (default: all of them)."""
    t = cfg.text_config
    if quantized is None:
        quantized = {i for i in range(t.num_hidden_layers) if not t.is_dense(i)}
    out = []

    def emit(slot):
        d = describe(cfg, quantized, slot)
        if d is not None:
            out.append((slot, tensor_name(slot), d[0], d[1]))
    emit(("embed",))
    if t.use_embed_norm:
        emit(("embed_norm",))
    emit(("final_norm",))
    emit(("unembed",))
    for i in range(t.num_hidden_layers):
        for part in _block_parts(t.is_dense(i), i in quantized):
            emit(("llm", i) + part)
    for i in range(cfg.mtp_config.num_nextn_predict_layers):
        for w in ("embed_norm", "hidden_norm", "input_proj"):
            emit(("mtp", i, w))
        for part in _block_parts(True, False):
            emit(("mtp", i, "block") + part)
    vc = cfg.vision_config
    for i in range(vc.n_layers):
        emit(("vision", "linear", i))
        if i + 1 < vc.n_layers:
            emit(("vision", "norm", i))
    if vc.n_layers:
        emit(("vision", "final_norm"))
    if cfg.audio_config.decoder_dmodel:
        emit(("audio", "encoder"))
        emit(("audio", "final_norm"))
    return out


def check_headers(cfg: InklingConfig, headers: dict, quantized: set | None = None) -> list[str]:
    """The layout gate over a checkpoint's headers ``{name: (shape, dtype)}``: every expected slot present with the described
    shape and dtype, every tensor mapped to a slot (name -> slot -> name is the identity), nothing twice, and each expert
    matrix of a layer with all four quantisation sidecars or none.  Returns the list of violations (empty = pass)."""
    t = cfg.text_config
    if quantized is None:                      # read it off the headers: a layer is quantised when its w13 carries a block scale
        quantized = {i for i in range(t.num_hidden_layers) if f"model.llm.layers.{i}.mlp.experts.w13_weight.scale" in headers}
    bad, seen = [], {}
    for name in headers:
        s = parse(name)
        if s is None:
            bad.append(f"unmapped tensor {name}")
            continue
        if tensor_name(s) != name:
            bad.append(f"{name} parses to {s}, which formats to {tensor_name(s)}")
        if s in seen:
            bad.append(f"slot {s} filled twice: {seen[s]} and {name}")
        seen[s] = name
        if describe(cfg, quantized, s) is None:
            bad.append(f"{name}: the configuration has no such slot")
    for slot, name, shape, dtype in slots(cfg, quantized):
        if name not in headers:
            bad.append(f"missing {name}")
            continue
        got_shape, got_dtype = headers[name]
        if tuple(got_shape) != tuple(shape) or got_dtype != dtype:
            bad.append(f"{name}: expected {shape} {dtype}, found {tuple(got_shape)} {got_dtype}")
    for i in range(t.num_hidden_layers):
        if t.is_dense(i):
            continue
        for mat in ("w13", "w2"):
            have = [q for q in SIDECARS if tensor_name(("llm", i, "mlp", "moe", "expert", mat, q)) in headers]
            if have and len(have) != len(SIDECARS):
                bad.append(f"layer {i} {mat}: quantisation sidecars {have} without the others")
    return bad
