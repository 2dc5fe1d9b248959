from .clip import ClipConfig, ClipEmbedder, load_into  # noqa: F401
