from .model import BiQwenEmbedder, Qwen25VLConfig, TextModel, VisionTower, load_into, mrope_positions  # noqa: F401
