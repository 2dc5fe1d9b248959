from .model import Depformer, LmGen, MoshiConfig, StreamCache, init_random_, load_into  # noqa: F401
