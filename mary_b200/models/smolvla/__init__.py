from .model import SmolVLA, SmolVLAConfig, TowerConfig, euler_sample, time_embedding  # noqa: F401
