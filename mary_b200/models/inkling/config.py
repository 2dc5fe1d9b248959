"""Inkling configuration as the checkpoint's ``config.json`` states it (src/models/inkling/config.rs:36-306).

The serving entry point reads it from FACTS in the pile (``format.jsonfacts``), never from a side file
(src/bin/inkling_forward.rs:2841-2854).  Two fields decide tensor NAME sets, not only sizes, so the layout depends on them:
``dense_mlp_idx`` (layers below it carry the dense MLP names) and ``shared_expert_sink`` (the router matrix then has
``n_routed_experts + n_shared_experts`` rows).  Sliding-window layers have head counts of their own (``swa_*``), which differ
from the global ones on the 66-layer model; a zero means "same as global"."""
from __future__ import annotations

from dataclasses import dataclass, field, fields

LOCAL, GLOBAL = "local", "global"


@dataclass
class InklingTextConfig:
    hidden_size: int
    num_hidden_layers: int
    num_attention_heads: int
    num_key_value_heads: int
    head_dim: int
    vocab_size: int
    d_rel: int
    rel_extent: int
    rms_norm_eps: float
    sconv_kernel_size: int
    sliding_window_size: int
    local_layer_ids: list
    dense_mlp_idx: int
    dense_intermediate_size: int
    intermediate_size: int
    n_routed_experts: int
    num_experts_per_tok: int
    n_shared_experts: int
    route_scale: float
    gate_activation: str
    swa_num_attention_heads: int = 0
    swa_num_key_value_heads: int = 0
    swa_head_dim: int = 0
    unpadded_vocab_size: int = 0
    use_embed_norm: bool = False
    use_sconv: bool = False
    shared_expert_sink: bool = False
    use_gate_bias: bool = False
    norm_after_topk: bool = False
    use_global_scale: bool = False
    log_scaling_n_floor: int = 0
    log_scaling_alpha: float = 0.0
    logits_mup_width_multiplier: float = 0.0
    model_max_length: int = 0

    def attn_kind(self, layer: int) -> str:
        return LOCAL if layer in self.local_layer_ids else GLOBAL

    def heads(self, kind: str) -> tuple[int, int, int]:
        """``(query heads, kv heads, head width)`` of a layer of this kind (config.rs:115-136)."""
        if kind == GLOBAL:
            return self.num_attention_heads, self.num_key_value_heads, self.head_dim
        return (self.swa_num_attention_heads or self.num_attention_heads, self.swa_num_key_value_heads or self.num_key_value_heads,
                self.swa_head_dim or self.head_dim)

    def q_dim(self, kind: str) -> int:
        h, _, d = self.heads(kind)
        return h * d

    def kv_dim(self, kind: str) -> int:
        _, kv, d = self.heads(kind)
        return kv * d

    def rel_dim(self, kind: str) -> int:
        return self.heads(kind)[0] * self.d_rel

    def norm_dim(self, kind: str) -> int:
        return self.heads(kind)[2]

    def rel_span(self, kind: str) -> int:
        """A local layer never sees past its window, so its bias table is ``sliding_window_size`` wide (config.rs:194-199)."""
        return self.sliding_window_size if kind == LOCAL else self.rel_extent

    def effective_vocab(self) -> int:
        return self.unpadded_vocab_size if 0 < self.unpadded_vocab_size <= self.vocab_size else self.vocab_size

    def gate_rows(self) -> int:
        return self.n_routed_experts + (self.n_shared_experts if self.shared_expert_sink else 0)

    def is_dense(self, layer: int) -> bool:
        return layer < self.dense_mlp_idx

    def op_cfg(self, kind: str) -> dict:
        """The dictionary the operators of ``models.inkling.ops`` / ``paged`` take for a layer of this kind."""
        h, kv, d = self.heads(kind)
        return dict(n_heads=h, n_kv_heads=kv, head_dim=d, d_rel=self.d_rel, window=self.sliding_window_size, eps=self.rms_norm_eps,
                    log_alpha=self.log_scaling_alpha, log_n_floor=max(self.log_scaling_n_floor, 1))


@dataclass
class InklingMtpConfig:
    num_nextn_predict_layers: int = 0
    chain_hidden_post_norm: bool = False
    local_layer_ids: list = field(default_factory=list)

    def attn_kind(self, layer: int) -> str:
        return LOCAL if layer in self.local_layer_ids else GLOBAL


@dataclass
class InklingAudioConfig:
    decoder_dmodel: int = 0
    n_mel_bins: int = 0
    mel_vocab_size: int = 0
    audio_mode: str = ""
    use_audio_norm: bool = False

    def encoder_rows(self) -> int:
        return self.n_mel_bins * self.mel_vocab_size


@dataclass
class InklingVisionConfig:
    decoder_dmodel: int = 0
    patch_size: int = 0
    temporal_patch_size: int = 1
    n_channels: int = 3
    n_layers: int = 0
    hidden_dims: list = field(default_factory=lambda: [128, 320, 4800])
    subpatch_size: int = 5

    def subpatch_elems(self) -> int:
        return self.subpatch_size ** 2 * self.n_channels

    def patch_elems(self) -> int:
        return self.patch_size ** 2 * self.n_channels * self.temporal_patch_size


@dataclass
class InklingConfig:
    text_config: InklingTextConfig
    mtp_config: InklingMtpConfig = field(default_factory=InklingMtpConfig)
    audio_config: InklingAudioConfig = field(default_factory=InklingAudioConfig)
    vision_config: InklingVisionConfig = field(default_factory=InklingVisionConfig)

    @staticmethod
    def from_json(d: dict) -> "InklingConfig":
        """``d``: the parsed ``config.json`` (e.g. ``jsonfacts.load_document(store, facts, "config.json")``)."""
        def take(cls, obj):
            names = {f.name for f in fields(cls)}
            kw = {k: v for k, v in (obj or {}).items() if k in names}
            try:
                return cls(**kw)
            except TypeError as ex:
                raise KeyError(f"{cls.__name__}: config.json lacks a required field: {ex}") from None
        return InklingConfig(take(InklingTextConfig, d.get("text_config")), take(InklingMtpConfig, d.get("mtp_config")),
                             take(InklingAudioConfig, d.get("audio_config")), take(InklingVisionConfig, d.get("vision_config")))

    def to_json(self) -> dict:
        from dataclasses import asdict
        return {"model_type": "inkling", "text_config": asdict(self.text_config), "mtp_config": asdict(self.mtp_config),
                "audio_config": asdict(self.audio_config), "vision_config": asdict(self.vision_config)}


def tiny_inkling_config(**kw) -> InklingConfig:
    """A small configuration with every structural feature of the released models: a dense first layer, local and global layers
    with DIFFERENT head counts, the shared-expert sink, log scaling, a padded vocabulary and two MTP heads."""
    t = dict(hidden_size=128, num_hidden_layers=4, num_attention_heads=4, num_key_value_heads=2, head_dim=32, swa_num_attention_heads=4,
             swa_num_key_value_heads=4, swa_head_dim=32, vocab_size=320, unpadded_vocab_size=300, d_rel=8, rel_extent=64, rms_norm_eps=1e-6,
             use_embed_norm=True, sconv_kernel_size=4, use_sconv=True, sliding_window_size=16, local_layer_ids=[0, 2], dense_mlp_idx=1,
             dense_intermediate_size=256, intermediate_size=128, n_routed_experts=8, num_experts_per_tok=2, n_shared_experts=2,
             shared_expert_sink=True, route_scale=2.0, use_gate_bias=True, gate_activation="sigmoid", norm_after_topk=True,
             use_global_scale=True, log_scaling_n_floor=32, log_scaling_alpha=0.1, logits_mup_width_multiplier=2.0, model_max_length=4096)
    t.update(kw)
    return InklingConfig(InklingTextConfig(**t), InklingMtpConfig(num_nextn_predict_layers=2, local_layer_ids=[]),
                         InklingAudioConfig(decoder_dmodel=t["hidden_size"], n_mel_bins=8, mel_vocab_size=4),
                         InklingVisionConfig(decoder_dmodel=t["hidden_size"], patch_size=40, temporal_patch_size=2, n_channels=3, n_layers=4,
                                             hidden_dims=[16, 24, 48], subpatch_size=5))
