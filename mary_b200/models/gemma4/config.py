"""``Gemma4TextConfig`` (src/models/gemma/gemma4/config.rs:36-101,215-270): parsed from the ``config.json``
document stored as facts in the pile, with the reference's defaults."""
from __future__ import annotations

from dataclasses import dataclass, field


@dataclass
class Gemma4TextConfig:
    hidden_size: int = 256
    num_hidden_layers: int = 4
    num_attention_heads: int = 4
    num_key_value_heads: int = 1
    head_dim: int = 64
    intermediate_size: int = 1024
    vocab_size: int = 4096
    layer_types: list = field(default_factory=list)          # "sliding_attention" | "full_attention"
    sliding_window: int = 128
    rope_theta_local: float = 1e4
    rope_theta_global: float = 1e6
    partial_rotary_factor_global: float = 1.0
    rms_norm_eps: float = 1e-6
    final_logit_softcapping: float = 30.0
    tie_word_embeddings: bool = True
    global_head_dim: int | None = None
    num_global_key_value_heads: int | None = None
    attention_k_eq_v: bool = False      # full-attention layers have no v_proj: k and v come from one projection
    num_kv_shared_layers: int = 0       # the last layers compute no K/V and read the cache of an earlier layer
    apply_sliding_window: bool = True   # the reference's text path never applies the window (layers.rs:210-234
    #                                     has no caller); it is applied here and can be switched off for parity
    max_position_embeddings: int = 131072
    hidden_size_per_layer_input: int = 0    # per-layer embeddings (PLE): width of the per-layer token signal, 0 = off
    vocab_size_per_layer_input: int = 0     # rows of the per-layer embedding table (0 = vocab_size)
    enable_moe_block: bool = False          # 26B-A4B: a routed expert sum runs beside the dense MLP in every layer
    num_experts: int = 0
    top_k_experts: int = 0
    moe_intermediate_size: int = 0
    use_double_wide_mlp: bool = False       # KV-shared layers carry an MLP twice as wide

    def __post_init__(self):
        if not self.layer_types:
            self.layer_types = ["sliding_attention" if i % 2 == 0 else "full_attention"
                                for i in range(self.num_hidden_layers)]
        if len(self.layer_types) != self.num_hidden_layers:
            raise ValueError("layer_types must have one entry per layer")

    @property
    def first_shared_kv_layer(self) -> int:
        return self.num_hidden_layers - self.num_kv_shared_layers

    def kv_source(self, i: int) -> int | None:
        """The layer whose cache layer ``i`` reads, or ``None`` when it keeps its own: the last layer of the same attention
        type before sharing starts — ``first_shared - 2`` for sliding and ``first_shared - 1`` for full attention in the shipped
        layer patterns (src/models/gemma/gemma4/decoder.rs:230-261)."""
        fs = self.first_shared_kv_layer
        if i < fs or self.num_kv_shared_layers == 0:
            return None
        same = [j for j in range(fs) if self.layer_types[j] == self.layer_types[i]]
        if not same:
            raise ValueError(f"KV-shared layer {i} has no earlier layer of type {self.layer_types[i]} to read from")
        return same[-1]

    def layer_intermediate(self, i: int) -> int:
        wide = self.use_double_wide_mlp and self.kv_source(i) is not None
        return self.intermediate_size * (2 if wide else 1)

    @property
    def ple_vocab(self) -> int:
        return self.vocab_size_per_layer_input or self.vocab_size

    def k_eq_v(self, i: int) -> bool:
        return self.attention_k_eq_v and not self.is_sliding(i)

    def is_sliding(self, i: int) -> bool:
        return self.layer_types[i] == "sliding_attention"

    def layer_head_dim(self, i: int) -> int:
        return self.head_dim if self.is_sliding(i) or not self.global_head_dim else self.global_head_dim

    def layer_kv_heads(self, i: int) -> int:
        if self.is_sliding(i) or not self.num_global_key_value_heads:
            return self.num_key_value_heads
        return self.num_global_key_value_heads

    @staticmethod
    def from_json(d: dict) -> "Gemma4TextConfig":
        d = d.get("text_config", d)
        rp = d.get("rope_parameters") or {}
        loc = rp.get("sliding_attention", {})
        glo = rp.get("full_attention", {})
        return Gemma4TextConfig(
            hidden_size=d["hidden_size"], num_hidden_layers=d["num_hidden_layers"],
            num_attention_heads=d["num_attention_heads"], num_key_value_heads=d.get("num_key_value_heads", 1),
            head_dim=d.get("head_dim", d["hidden_size"] // d["num_attention_heads"]),
            intermediate_size=d["intermediate_size"], vocab_size=d["vocab_size"],
            layer_types=list(d.get("layer_types") or []), sliding_window=d.get("sliding_window", 1024),
            rope_theta_local=float(loc.get("rope_theta", d.get("rope_local_base_freq", 1e4))),
            rope_theta_global=float(glo.get("rope_theta", d.get("rope_theta", 1e6))),
            partial_rotary_factor_global=float(glo.get("partial_rotary_factor", 1.0)),
            rms_norm_eps=d.get("rms_norm_eps", 1e-6),
            final_logit_softcapping=float(d.get("final_logit_softcapping") or 30.0),
            tie_word_embeddings=bool(d.get("tie_word_embeddings", True)),
            global_head_dim=d.get("global_head_dim"), num_global_key_value_heads=d.get("num_global_key_value_heads"),
            attention_k_eq_v=bool(d.get("attention_k_eq_v", False)), num_kv_shared_layers=int(d.get("num_kv_shared_layers", 0)),
            apply_sliding_window=bool(d.get("apply_sliding_window", True)),
            max_position_embeddings=d.get("max_position_embeddings", 131072),
            hidden_size_per_layer_input=int(d.get("hidden_size_per_layer_input") or 0),
            vocab_size_per_layer_input=int(d.get("vocab_size_per_layer_input") or 0),
            enable_moe_block=bool(d.get("enable_moe_block", False)), num_experts=int(d.get("num_experts") or 0),
            top_k_experts=int(d.get("top_k_experts") or 0), moe_intermediate_size=int(d.get("moe_intermediate_size") or 0),
            use_double_wide_mlp=bool(d.get("use_double_wide_mlp", False)))

    def to_json(self) -> dict:
        return {
            "model_type": "gemma4_text", "hidden_size": self.hidden_size, "num_hidden_layers": self.num_hidden_layers,
            "num_attention_heads": self.num_attention_heads, "num_key_value_heads": self.num_key_value_heads,
            "head_dim": self.head_dim, "intermediate_size": self.intermediate_size, "vocab_size": self.vocab_size,
            "layer_types": list(self.layer_types), "sliding_window": self.sliding_window,
            "rope_parameters": {"sliding_attention": {"rope_theta": self.rope_theta_local},
                                "full_attention": {"rope_theta": self.rope_theta_global,
                                                   "partial_rotary_factor": self.partial_rotary_factor_global}},
            "rms_norm_eps": self.rms_norm_eps, "final_logit_softcapping": self.final_logit_softcapping,
            "tie_word_embeddings": self.tie_word_embeddings, "apply_sliding_window": self.apply_sliding_window,
            "attention_k_eq_v": self.attention_k_eq_v, "num_kv_shared_layers": self.num_kv_shared_layers,
            "global_head_dim": self.global_head_dim, "num_global_key_value_heads": self.num_global_key_value_heads,
            "max_position_embeddings": self.max_position_embeddings,
            "hidden_size_per_layer_input": self.hidden_size_per_layer_input,
            "vocab_size_per_layer_input": self.vocab_size_per_layer_input, "enable_moe_block": self.enable_moe_block,
            "num_experts": self.num_experts, "top_k_experts": self.top_k_experts,
            "moe_intermediate_size": self.moe_intermediate_size, "use_double_wide_mlp": self.use_double_wide_mlp}


def tiny_config() -> Gemma4TextConfig:
    """4 layers, hidden 256, 4 query heads / 1 KV head x 64, sliding-128 / global alternating, GeGLU 1024,
    vocab 4096, tied head, softcap 30."""
    return Gemma4TextConfig()


def gemma_12b_config() -> Gemma4TextConfig:
    """48 layers, hidden 3840, 16 query / 8 KV heads x 256, 5:1 sliding(1024):global, GeGLU 15360, vocab 262144."""
    lt = ["full_attention" if i % 6 == 5 else "sliding_attention" for i in range(48)]
    return Gemma4TextConfig(hidden_size=3840, num_hidden_layers=48, num_attention_heads=16, num_key_value_heads=8,
                            head_dim=256, intermediate_size=15360, vocab_size=262144, layer_types=lt, sliding_window=1024)
