from .mimi import MimiCodec, MimiConfig, init_random_  # noqa: F401
