from .model import SmolVLA, SmolVLAConfig, TowerConfig, euler_sample, load_into, time_embedding  # noqa: F401
