from .model import Depformer, LmGen, MoshiConfig, StreamCache, init_random_, load_into  # noqa: F401
from .voice_prompt import Prompt, VoicePrompt, wrap_with_system_tags  # noqa: F401
