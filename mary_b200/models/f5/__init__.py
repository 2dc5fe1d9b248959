from .dit import CFM, DiT, F5Config, sway_times  # noqa: F401
from .spectral import istft_matmul, mel_spectrogram, stft_matmul  # noqa: F401
from .vocos import Vocos, VocosConfig  # noqa: F401
