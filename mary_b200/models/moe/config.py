"""Configuration of the sparse-MoE decoders: the Inkling-style GQA model and the Kimi-K3-class MLA model.

The two workload configurations are abstractions of the reference's real models (src/models/inkling/config.rs:36-306,
src/models/k3/config.rs:153-370): softmax or sigmoid routing, optional group-limited top-k (which the reference
refuses, src/models/k3/router.rs:136-143), shared experts, leading dense layers, NVFP4 experts, MTP draft layers."""
from __future__ import annotations

from dataclasses import asdict, dataclass


@dataclass
class MoEConfig:
    name: str = "moe"
    hidden_size: int = 512
    num_hidden_layers: int = 4
    num_attention_heads: int = 8
    attention: str = "gqa"               # "gqa" | "mla"
    # GQA
    num_key_value_heads: int = 2
    head_dim: int = 64
    # MLA
    q_lora_rank: int = 1536
    kv_lora_rank: int = 512
    qk_nope_head_dim: int = 128
    qk_rope_head_dim: int = 64
    v_head_dim: int = 128
    use_nope: bool = False               # the reference's K3 runs NoPE MLA (src/models/k3/mla.rs)
    rope_theta: float = 1e6
    # FFN
    first_k_dense: int = 0
    dense_intermediate_size: int = 2048
    n_routed_experts: int = 8
    num_experts_per_tok: int = 2
    n_shared_experts: int = 1
    moe_intermediate_size: int = 256
    router: str = "softmax"              # "softmax" | "sigmoid"
    n_group: int = 1
    topk_group: int = 1
    routed_scaling_factor: float = 1.0
    norm_topk_prob: bool = True
    act: str = "swiglu"
    vocab_size: int = 4096
    rms_norm_eps: float = 1e-6
    num_mtp_layers: int = 0
    tie_word_embeddings: bool = False
    shared_expert_nvfp4: bool = False    # run the shared expert through the NVFP4 grouped GEMM as one more expert

    def to_json(self) -> dict:
        d = asdict(self)
        d["model_type"] = "mary_moe"
        return d

    @staticmethod
    def from_json(d: dict) -> "MoEConfig":
        keys = MoEConfig.__dataclass_fields__.keys()
        return MoEConfig(**{k: v for k, v in d.items() if k in keys})

    def is_dense(self, i: int) -> bool:
        return i < self.first_k_dense

    @property
    def attn_scale(self) -> float:
        if self.attention == "mla":
            return (self.qk_nope_head_dim + self.qk_rope_head_dim) ** -0.5
        return self.head_dim ** -0.5


def inkling_style_config() -> MoEConfig:
    """32 layers, hidden 4096, GQA 32/8 x 128, 128 routed experts top-8 (softmax), 1 shared, expert FFN 1536, vocab 151936."""
    return MoEConfig(name="inkling-style", hidden_size=4096, num_hidden_layers=32, num_attention_heads=32, attention="gqa",
                     num_key_value_heads=8, head_dim=128, first_k_dense=0, n_routed_experts=128, num_experts_per_tok=8,
                     n_shared_experts=1, moe_intermediate_size=1536, router="softmax", vocab_size=151936, act="swiglu")


def k3_class_config() -> MoEConfig:
    """61 layers (first dense, FFN 18432), hidden 7168, 64 heads, MLA q_lora 1536 / kv_lora 512 / nope 128 / rope 64 / v 128,
    384 routed experts top-8 (sigmoid, group-limited 8 groups / 4 kept), 1 shared, expert FFN 2048, vocab 163840, 1 MTP layer."""
    return MoEConfig(name="k3-class", hidden_size=7168, num_hidden_layers=61, num_attention_heads=64, attention="mla",
                     q_lora_rank=1536, kv_lora_rank=512, qk_nope_head_dim=128, qk_rope_head_dim=64, v_head_dim=128,
                     first_k_dense=1, dense_intermediate_size=18432, n_routed_experts=384, num_experts_per_tok=8,
                     n_shared_experts=1, moe_intermediate_size=2048, router="sigmoid", n_group=8, topk_group=4,
                     routed_scaling_factor=2.5, vocab_size=163840, num_mtp_layers=1, act="swiglu", shared_expert_nvfp4=True)


def tiny_moe_config(attention: str = "mla", **kw) -> MoEConfig:
    base = dict(name=f"tiny-{attention}", hidden_size=512, num_hidden_layers=3, num_attention_heads=8, attention=attention,
                num_key_value_heads=2, head_dim=64, q_lora_rank=256, first_k_dense=1, dense_intermediate_size=1024,
                n_routed_experts=8, num_experts_per_tok=2, moe_intermediate_size=256, router="sigmoid" if attention == "mla" else "softmax",
                n_group=4 if attention == "mla" else 1, topk_group=2 if attention == "mla" else 1, routed_scaling_factor=2.5,
                vocab_size=2048, num_mtp_layers=1 if attention == "mla" else 0)
    base.update(kw)
    return MoEConfig(**base)
