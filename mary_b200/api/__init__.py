"""In-process seams: the calls an application makes without going through a command line.

``local``  chat completion behind ``LocalTextEngine`` (src/local.rs)
``say``    one-shot speech synthesis with a cloned voice, F5-TTS + Vocos (src/say.rs)
``speak``  streaming speech synthesis, Qwen3-TTS talker + code predictor + codec (src/speak.rs)
``GemmaLM`` (``models.gemma4.lm``) is the fourth seam of the reference and lives with its model."""
from . import local, say, speak  # noqa: F401
