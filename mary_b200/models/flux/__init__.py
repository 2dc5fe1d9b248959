from .pipeline import FluxPipeline, pack_latents, position_ids, unpack_latents  # noqa: F401
from .scheduler import FlowMatchEuler, empirical_mu  # noqa: F401
from .transformer import Flux2Config, Flux2Transformer  # noqa: F401
from .vae import Flux2VAE, VAEConfig  # noqa: F401
