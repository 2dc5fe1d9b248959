from .clip import ClipConfig, ClipEmbedder, load_into  # noqa: F401
from .nomic import NomicConfig, NomicTextEmbedder, NomicVisionConfig, NomicVisionEmbedder  # noqa: F401
from .siglip import SiglipConfig, SiglipEmbedder  # noqa: F401
from . import clip, nomic, siglip  # noqa: F401,E402
