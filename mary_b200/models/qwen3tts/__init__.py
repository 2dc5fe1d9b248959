from .codec import CodecConfig, CodecDecoder, CodecEncoder  # noqa: F401
from .model import (CodePredictor, Qwen3TTSConfig, SamplingParams, Talker, generate_frames, init_random_,  # noqa: F401
                    load_into, process_talker_logits)
