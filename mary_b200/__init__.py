"""mary_b200 — a B200-native model-graph framework: content-addressed piles, config-free model loading,
generation and LoRA training for dense and sparse-MoE decoders on sm_100a."""
__version__ = "0.1.0"
