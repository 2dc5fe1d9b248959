"""The K3 checkpoint layout: every safetensors tensor name and the module slot it fills (src/models/k3/layout.rs).

Names, shapes and dtypes only; no tensor bytes are read here.  The mapping exists TWICE, in opposite directions and without
shared code, so that comparing them on a checkpoint's headers is a real cross-check:

* :func:`slots` walks a config and yields every slot the model needs with the name it expects (module tree -> checkpoint), built
  by string formatting from per-part tables;
* :func:`parse` takes a tensor name and recovers the slot (checkpoint -> module tree) with one anchored regular expression per
  family and no access to those tables' formatting.

A slot is a plain tuple: ``("embed",)``, ``("final_norm",)``, ``("out_res_norm",)``, ``("out_res_proj",)``, ``("lm_head",)``,
``("layer", i, part...)``, ``("vision", part...)``, ``("mm", part)``.  Shapes are in CHECKPOINT order (``[out, in]`` of a
``torch.nn.Linear``); transposing is the loader's business.

:func:`check_headers` is the gate (tests/k3_layout_gate): every expected slot present with the described shape and dtype, every
tensor in the headers mapped to a slot, nothing twice."""
from __future__ import annotations

import dataclasses
import math
import re

BF16, F32, U8 = "BF16", "F32", "U8"
MXFP4_BLOCK = 32                # elements sharing one E8M0 exponent, along the INPUT axis


@dataclasses.dataclass
class K3Linear:
    kda_layers: list
    full_attn_layers: list
    head_dim: int
    num_heads: int
    short_conv_kernel_size: int = 4

    @property
    def proj_dim(self) -> int:
        return self.num_heads * self.head_dim


@dataclasses.dataclass
class K3Vision:
    patch_size: int
    vt_hidden_size: int
    vt_intermediate_size: int
    vt_num_hidden_layers: int
    qkv_hidden_size: int
    mm_hidden_size: int
    text_hidden_size: int
    init_pos_emb_height: int
    init_pos_emb_width: int
    merge_kernel_size: tuple = (2, 2)

    @property
    def projector_input_dim(self) -> int:
        return self.mm_hidden_size * math.prod(self.merge_kernel_size)


@dataclasses.dataclass
class K3Dims:
    """The fields of ``config.json`` that decide a tensor's existence, shape or dtype (config.rs:84-340)."""
    hidden_size: int
    intermediate_size: int
    num_hidden_layers: int
    num_attention_heads: int
    num_key_value_heads: int
    vocab_size: int
    first_k_dense_replace: int
    num_experts: int
    moe_intermediate_size: int
    kv_lora_rank: int
    qk_nope_head_dim: int
    qk_rope_head_dim: int
    v_head_dim: int
    linear: K3Linear
    vision: K3Vision | None = None
    q_lora_rank: int | None = None
    num_shared_experts: int | None = None
    routed_expert_hidden_size: int | None = None
    latent_moe_use_norm: bool = True
    moe_layer_freq: int = 1

    @classmethod
    def from_json(cls, cfg: dict) -> "K3Dims":
        t = dict(cfg["text_config"])
        la = t.pop("linear_attn_config")
        names = {f.name for f in dataclasses.fields(cls)} - {"linear", "vision"}
        lin = K3Linear(**{f.name: la[f.name] for f in dataclasses.fields(K3Linear) if f.name in la})
        vis = None
        if cfg.get("vision_config"):
            v = cfg["vision_config"]
            vis = K3Vision(**{f.name: (tuple(v[f.name]) if f.name == "merge_kernel_size" else v[f.name])
                              for f in dataclasses.fields(K3Vision) if f.name in v})
        d = cls(linear=lin, vision=vis, **{k: t[k] for k in names if k in t})
        d.validate()
        return d

    def validate(self) -> None:
        """The attention lists are ONE-based and must partition ``1..n``: a zero-based reading leaves the last layer unclaimed and
        names one past the end, and both show up here (config.rs:250-300).  MLA's value width must equal KDA's head width because the
        two layer kinds share ``o_proj`` / ``g_proj`` shapes."""
        n = self.num_hidden_layers
        both = list(self.linear.kda_layers) + list(self.linear.full_attn_layers)
        if sorted(both) != list(range(1, n + 1)):
            raise ValueError(f"attention lists must partition layers 1..{n}: missing {sorted(set(range(1, n + 1)) - set(both))}, "
                             f"out of range {sorted(x for x in both if not 1 <= x <= n)}, "
                             f"duplicated {sorted({x for x in both if both.count(x) > 1})}")
        if self.num_attention_heads * self.v_head_dim != self.linear.proj_dim:
            raise ValueError("MLA value width and KDA head width differ: o_proj / g_proj cannot be shared")

    def attn_kind(self, layer: int) -> str:
        return "mla" if layer + 1 in self.linear.full_attn_layers else "kda"

    def is_moe_layer(self, layer: int) -> bool:
        return layer >= self.first_k_dense_replace and layer % self.moe_layer_freq == 0

    @property
    def moe_hidden_size(self) -> int:
        return self.routed_expert_hidden_size or self.hidden_size

    @property
    def shared_width(self) -> int:
        return self.moe_intermediate_size * (self.num_shared_experts or 0)


# ---- forward half: slot -> name ---------------------------------------------------------------------------------------------------

_TOP = {("embed",): "language_model.model.embed_tokens.weight", ("final_norm",): "language_model.model.norm.weight",
        ("out_res_norm",): "language_model.model.output_attn_res_norm.weight",
        ("out_res_proj",): "language_model.model.output_attn_res_proj.weight", ("lm_head",): "language_model.lm_head.weight"}
_LAYER_NORMS = {"input_ln": "input_layernorm", "post_attn_ln": "post_attention_layernorm", "attn_res_norm": "self_attention_res_norm",
                "attn_res_proj": "self_attention_res_proj", "mlp_res_norm": "mlp_res_norm", "mlp_res_proj": "mlp_res_proj"}
_BOTH = ("g_proj", "o_proj")
_KDA_W = ("q_proj", "k_proj", "v_proj", "q_conv1d", "k_conv1d", "v_conv1d", "f_a_proj", "f_b_proj", "b_proj", "o_norm")
_KDA_BARE = ("A_log", "dt_bias")                                   # parameters, not modules: no ".weight"
_MLA = ("q_a_proj", "q_a_layernorm", "q_b_proj", "kv_a_proj_with_mqa", "kv_a_layernorm", "kv_b_proj")
_MLP = ("gate_proj", "up_proj", "down_proj")
_VBLOCK = {"norm0": "norm0", "wqkv": "wqkv", "wo": "wo", "norm1": "norm1", "fc0": "mlp.fc0", "fc1": "mlp.fc1"}


def tensor_name(slot: tuple) -> str:
    if slot in _TOP:
        return _TOP[slot]
    if slot[0] == "layer":
        head = f"language_model.model.layers.{slot[1]}"
        part = slot[2:]
        if part[0] in _LAYER_NORMS:
            return f"{head}.{_LAYER_NORMS[part[0]]}.weight"
        if part[0] == "attn":
            return f"{head}.self_attn.{part[1]}" + ("" if part[1] in _KDA_BARE else ".weight")
        if part[0] == "mlp":
            return f"{head}.mlp.{part[1]}.weight"
        if part[0] == "moe":
            moe = f"{head}.block_sparse_moe"
            if part[1] == "gate":
                return f"{moe}.gate.weight"
            if part[1] == "gate_bias":
                return f"{moe}.gate.e_score_correction_bias"
            if part[1] in ("down_in", "up_out", "latent_norm"):
                return moe + {"down_in": ".routed_expert_down_proj", "up_out": ".routed_expert_up_proj",
                              "latent_norm": ".routed_expert_norm"}[part[1]] + ".weight"
            if part[1] == "shared":
                return f"{moe}.shared_experts.{part[2]}.weight"
            if part[1] == "expert":
                return f"{moe}.experts.{part[2]}.{part[3]}.weight_{part[4]}"
    if slot[0] == "vision":
        if slot[1] == "patch":
            return "vision_tower.patch_embed.proj.weight"
        if slot[1] == "pos":
            return "vision_tower.patch_embed.pos_emb.weight"
        if slot[1] == "final_ln":
            return "vision_tower.encoder.final_layernorm.weight"
        if slot[1] == "block":
            return f"vision_tower.encoder.blocks.{slot[2]}.{_VBLOCK[slot[3]]}.weight"
    if slot[0] == "mm":
        return {"proj0": "mm_projector.proj.0.weight", "proj2": "mm_projector.proj.2.weight",
                "post_norm": "mm_projector.post_norm.weight"}[slot[1]]
    raise KeyError(f"no tensor name for slot {slot}")


# ---- reverse half: name -> slot (regular expressions only; shares nothing with tensor_name) -----------------------------------

_RE_LAYER = re.compile(r"^language_model\.model\.layers\.(0|[1-9]\d*)\.(.+)$")
_RE_EXPERT = re.compile(r"^block_sparse_moe\.experts\.(0|[1-9]\d*)\.(w[123])\.weight_(packed|scale)$")
_RE_VBLOCK = re.compile(r"^vision_tower\.encoder\.blocks\.(0|[1-9]\d*)\.(norm0|wqkv|wo|norm1|mlp\.fc0|mlp\.fc1)\.weight$")
_RE_ATTN = re.compile(r"^self_attn\.([A-Za-z_0-9]+?)(\.weight)?$")


def parse(name: str) -> tuple | None:
    """The slot a checkpoint name fills, or ``None`` for a name no slot claims.  Strict on purpose: an unknown suffix is ``None``,
    never a fall-through.  Whether the slot is legal for a CONFIG (layer in range, MLA tensor on an MLA layer) is :func:`describe`'s
    decision, not this one's."""
    if name == "language_model.model.embed_tokens.weight":
        return ("embed",)
    if name == "language_model.model.norm.weight":
        return ("final_norm",)
    if name == "language_model.model.output_attn_res_norm.weight":
        return ("out_res_norm",)
    if name == "language_model.model.output_attn_res_proj.weight":
        return ("out_res_proj",)
    if name == "language_model.lm_head.weight":
        return ("lm_head",)
    m = _RE_LAYER.match(name)
    if m:
        i, rest = int(m.group(1)), m.group(2)
        simple = {"input_layernorm.weight": "input_ln", "post_attention_layernorm.weight": "post_attn_ln",
                  "self_attention_res_norm.weight": "attn_res_norm", "self_attention_res_proj.weight": "attn_res_proj",
                  "mlp_res_norm.weight": "mlp_res_norm", "mlp_res_proj.weight": "mlp_res_proj",
                  "block_sparse_moe.gate.weight": ("moe", "gate"),
                  "block_sparse_moe.gate.e_score_correction_bias": ("moe", "gate_bias"),
                  "block_sparse_moe.routed_expert_down_proj.weight": ("moe", "down_in"),
                  "block_sparse_moe.routed_expert_up_proj.weight": ("moe", "up_out"),
                  "block_sparse_moe.routed_expert_norm.weight": ("moe", "latent_norm")}
        if rest in simple:
            s = simple[rest]
            return ("layer", i) + (s if isinstance(s, tuple) else (s,))
        e = _RE_EXPERT.match(rest)
        if e:
            return ("layer", i, "moe", "expert", int(e.group(1)), e.group(2), e.group(3))
        for branch, tag in (("mlp.", ("mlp",)), ("block_sparse_moe.shared_experts.", ("moe", "shared"))):
            if rest.startswith(branch) and rest.endswith(".weight"):
                leaf = rest[len(branch):-len(".weight")]
                if leaf in ("gate_proj", "up_proj", "down_proj"):
                    return ("layer", i) + tag + (leaf,)
        a = _RE_ATTN.match(rest)
        if a:
            leaf, has_w = a.group(1), a.group(2) is not None
            bare = leaf in ("A_log", "dt_bias")
            known = {"g_proj", "o_proj", "q_proj", "k_proj", "v_proj", "q_conv1d", "k_conv1d", "v_conv1d", "f_a_proj", "f_b_proj",
                     "b_proj", "o_norm", "q_a_proj", "q_a_layernorm", "q_b_proj", "kv_a_proj_with_mqa", "kv_a_layernorm", "kv_b_proj"}
            if (bare and not has_w) or (leaf in known and has_w):
                return ("layer", i, "attn", leaf)
        return None
    if name == "vision_tower.patch_embed.proj.weight":
        return ("vision", "patch")
    if name == "vision_tower.patch_embed.pos_emb.weight":
        return ("vision", "pos")
    if name == "vision_tower.encoder.final_layernorm.weight":
        return ("vision", "final_ln")
    v = _RE_VBLOCK.match(name)
    if v:
        return ("vision", "block", int(v.group(1)), {"mlp.fc0": "fc0", "mlp.fc1": "fc1"}.get(v.group(2), v.group(2)))
    mm = {"mm_projector.proj.0.weight": "proj0", "mm_projector.proj.2.weight": "proj2", "mm_projector.post_norm.weight": "post_norm"}
    if name in mm:
        return ("mm", mm[name])
    return None


# ---- shapes and dtypes ------------------------------------------------------------------------------------------------------------

def describe(d: K3Dims, slot: tuple):
    """``(shape, dtype)`` of a slot under config ``d``, or ``None`` when the slot is not legal there: layer out of range, an MLA
    tensor on a KDA layer or the reverse, a dense MLP on a sparse layer, an expert index past the count, a vision slot without a
    vision config.  ``A_log`` is described as the checkpoint ships it, ``[head_dim]``: the first ``num_heads`` entries are the
    per-head decay logs and the rest is zero padding that a loader must DROP (``exp(0) = 1`` is "no decay", not a no-op).  The
    convolution taps, ``A_log``, ``dt_bias``, ``o_norm`` and the router's correction bias are f32; experts are u8 (two E2M1 codes
    per byte, one E8M0 exponent per 32 inputs); everything else is bf16."""
    h = d.hidden_size
    if slot in (("embed",), ("lm_head",)):
        return (d.vocab_size, h), BF16
    if slot in (("final_norm",), ("out_res_norm",)):
        return (h,), BF16
    if slot == ("out_res_proj",):
        return (1, h), BF16
    if slot[0] == "layer":
        i, part = slot[1], slot[2:]
        if not 0 <= i < d.num_hidden_layers:
            return None
        if part[0] in ("input_ln", "post_attn_ln", "attn_res_norm", "mlp_res_norm"):
            return (h,), BF16
        if part[0] in ("attn_res_proj", "mlp_res_proj"):
            return (1, h), BF16
        if part[0] == "attn":
            return _describe_attn(d, i, part[1])
        if part[0] == "mlp":
            if d.is_moe_layer(i):
                return None
            f = d.intermediate_size
            return ((h, f) if part[1] == "down_proj" else (f, h)), BF16
        if part[0] == "moe":
            if not d.is_moe_layer(i):
                return None
            return _describe_moe(d, part[1:])
        return None
    if slot[0] == "vision":
        v = d.vision
        if v is None:
            return None
        vh = v.vt_hidden_size
        if slot[1] == "patch":
            return (vh, 3, v.patch_size, v.patch_size), BF16
        if slot[1] == "pos":
            return (v.init_pos_emb_height, v.init_pos_emb_width, vh), BF16
        if slot[1] == "final_ln":
            return (vh,), BF16
        if slot[1] == "block":
            if not 0 <= slot[2] < v.vt_num_hidden_layers:
                return None
            return {"norm0": (vh,), "norm1": (vh,), "wqkv": (3 * v.qkv_hidden_size, vh), "wo": (vh, v.qkv_hidden_size),
                    "fc0": (v.vt_intermediate_size, vh), "fc1": (vh, v.vt_intermediate_size)}[slot[3]], BF16
        return None
    if slot[0] == "mm":
        v = d.vision
        if v is None:
            return None
        din = v.projector_input_dim
        return {"proj0": (din, din), "proj2": (v.text_hidden_size, din), "post_norm": (v.text_hidden_size,)}[slot[1]], BF16
    return None


def _describe_attn(d: K3Dims, layer: int, leaf: str):
    la, h = d.linear, d.hidden_size
    kind = "kda" if leaf in _KDA_W + _KDA_BARE else "mla" if leaf in _MLA else None
    if kind is not None and d.attn_kind(layer) != kind:
        return None
    P = la.proj_dim
    if leaf == "g_proj":
        return (P, h), BF16
    if leaf == "o_proj":
        return (h, P), BF16
    if leaf in ("q_proj", "k_proj", "v_proj"):
        return (P, h), BF16
    if leaf in ("q_conv1d", "k_conv1d", "v_conv1d"):
        return (P, 1, la.short_conv_kernel_size), F32               # depthwise: one kernel per channel
    if leaf in ("A_log", "o_norm"):
        return (la.head_dim,), F32
    if leaf == "dt_bias":
        return (P,), F32
    if leaf == "f_a_proj":
        return (la.head_dim, h), BF16
    if leaf == "f_b_proj":
        return (P, la.head_dim), BF16
    if leaf == "b_proj":
        return (la.num_heads, h), BF16
    if leaf in ("q_a_proj", "q_a_layernorm", "q_b_proj") and d.q_lora_rank is None:
        return None
    if leaf == "q_a_proj":
        return (d.q_lora_rank, h), BF16
    if leaf == "q_a_layernorm":
        return (d.q_lora_rank,), BF16
    if leaf == "q_b_proj":
        return (d.num_attention_heads * (d.qk_nope_head_dim + d.qk_rope_head_dim), d.q_lora_rank), BF16
    if leaf == "kv_a_proj_with_mqa":
        return (d.kv_lora_rank + d.qk_rope_head_dim, h), BF16
    if leaf == "kv_a_layernorm":
        return (d.kv_lora_rank,), BF16
    if leaf == "kv_b_proj":
        return (d.num_key_value_heads * (d.qk_nope_head_dim + d.v_head_dim), d.kv_lora_rank), BF16
    return None


def _describe_moe(d: K3Dims, part: tuple):
    h, lat, f = d.hidden_size, d.moe_hidden_size, d.moe_intermediate_size
    if part[0] == "gate":
        return (d.num_experts, h), BF16
    if part[0] == "gate_bias":
        return (d.num_experts,), F32
    if part[0] == "down_in":
        return (lat, h), BF16
    if part[0] == "up_out":
        return (h, lat), BF16
    if part[0] == "latent_norm":
        if not d.latent_moe_use_norm or d.routed_expert_hidden_size is None:
            return None
        return (lat,), BF16
    if part[0] == "shared":
        if not d.num_shared_experts:
            return None
        s = d.shared_width
        return ((h, s) if part[1] == "down_proj" else (s, h)), BF16
    if part[0] == "expert":
        e, mat, half = part[1], part[2], part[3]
        if not 0 <= e < d.num_experts:
            return None
        out, inp = (lat, f) if mat == "w2" else (f, lat)           # w1 gate, w3 up: latent -> ffn; w2 down: ffn -> latent
        return (out, inp // 2 if half == "packed" else inp // MXFP4_BLOCK), U8
    return None


# ---- enumeration ------------------------------------------------------------------------------------------------------------------

def slots(d: K3Dims, experts: bool = True):
    """Every slot the model needs, in load order, as ``(slot, name, shape, dtype)``.  A generator: the full model has close to half a
    million expert tensors and a loader streams them against the checkpoint.  ``experts=False`` leaves the routed experts out (the
    rest is a few thousand tensors).  A slot this walk produces that :func:`describe` rejects is a bug in this file, so it raises."""
    def emit(slot):
        spec = describe(d, slot)
        if spec is None:
            raise AssertionError(f"enumerated a slot that describe() rejects: {slot}")
        return slot, tensor_name(slot), spec[0], spec[1]
    yield emit(("embed",))
    for i in range(d.num_hidden_layers):
        L = ("layer", i)
        for p in ("input_ln", "post_attn_ln", "attn_res_norm", "attn_res_proj", "mlp_res_norm", "mlp_res_proj"):
            yield emit(L + (p,))
        leaves = _BOTH + ((_KDA_W + _KDA_BARE) if d.attn_kind(i) == "kda" else _MLA)
        for leaf in leaves:
            yield emit(L + ("attn", leaf))
        if not d.is_moe_layer(i):
            for m in _MLP:
                yield emit(L + ("mlp", m))
            continue
        for p in ("gate", "gate_bias", "down_in", "up_out"):
            yield emit(L + ("moe", p))
        if d.latent_moe_use_norm and d.routed_expert_hidden_size is not None:
            yield emit(L + ("moe", "latent_norm"))
        if d.num_shared_experts:
            for m in _MLP:
                yield emit(L + ("moe", "shared", m))
        if experts:
            for e in range(d.num_experts):
                for mat in ("w1", "w2", "w3"):
                    for half in ("packed", "scale"):
                        yield emit(L + ("moe", "expert", e, mat, half))
    for s in (("final_norm",), ("out_res_norm",), ("out_res_proj",), ("lm_head",)):
        yield emit(s)
    if d.vision is not None:
        yield emit(("vision", "patch"))
        yield emit(("vision", "pos"))
        for b in range(d.vision.vt_num_hidden_layers):
            for p in _VBLOCK:
                yield emit(("vision", "block", b, p))
        yield emit(("vision", "final_ln"))
        for p in ("proj0", "proj2", "post_norm"):
            yield emit(("mm", p))


def check_headers(d: K3Dims, headers: dict) -> dict:
    """Compare the layout with a checkpoint's headers ``{name: (dtype, shape)}``.  Returns the findings; all four lists empty means
    the two directions agree with the file: ``unfilled`` (expected, absent), ``unmapped`` (present, no slot or a slot illegal under
    the config), ``mismatched`` (present with another shape or dtype), ``not_inverse`` (``parse(tensor_name(slot)) != slot``)."""
    out = {"unfilled": [], "unmapped": [], "mismatched": [], "not_inverse": []}
    expected = set()
    for slot, name, shape, dtype in slots(d):
        expected.add(name)
        if parse(name) != slot:
            out["not_inverse"].append(name)
        got = headers.get(name)
        if got is None:
            out["unfilled"].append(name)
        elif (got[0], tuple(got[1])) != (dtype, tuple(shape)):
            out["mismatched"].append((name, got, (dtype, tuple(shape))))
    for name in headers:
        if name in expected:
            continue
        out["unmapped"].append(name)
    return out
