from .model import MistralConfig, MistralModel, init_random_, load_into, yarn_inv_freq  # noqa: F401
