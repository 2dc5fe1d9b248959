from .config import MoEConfig, inkling_style_config, k3_class_config, tiny_moe_config
from .model import MoEDecoder, NoParallel, init_random_

__all__ = ["MoEConfig", "MoEDecoder", "NoParallel", "init_random_", "inkling_style_config", "k3_class_config", "tiny_moe_config"]
