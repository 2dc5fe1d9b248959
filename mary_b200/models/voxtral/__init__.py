from .model import VoxtralConfig, VoxtralModel, VoxtralListener, load_into, log_mel  # noqa: F401
