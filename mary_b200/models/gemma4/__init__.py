from .config import Gemma4TextConfig, gemma_12b_config, tiny_config
from .lm import GemmaLM
from .model import Gemma4Model

__all__ = ["Gemma4TextConfig", "Gemma4Model", "GemmaLM", "tiny_config", "gemma_12b_config"]
