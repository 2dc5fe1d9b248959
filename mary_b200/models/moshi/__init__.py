from .model import Depformer, LmGen, MoshiConfig, StreamCache, init_random_  # noqa: F401
