"""Device-memory pool policy: which allocator configuration a serving process runs with and when cached blocks go back to the
driver.

The reference chooses its allocator before the CUDA client exists (``CUBECL_MEMORY_CONFIG=exclusive``: one allocation per
buffer, so a 9 GB expert slab does not pin a pool page for ever) and returns memory per layer or per stage under a
``CleanupPolicy`` (src/models/inkling/pool.rs:165-321), because prefill activations of a long prompt would otherwise stay cached
while the decode phase needs the room for KV.  The PyTorch caching allocator has the same failure shape — large, differently
sized blocks fragment it — and the same two remedies:

* ``MARY_POOL``: ``default`` leaves torch alone; ``expandable`` turns on expandable segments (blocks grow in place instead of
  fragmenting; the setting of choice for prefill chunks of varying length); ``exclusive`` disables the caching of large blocks
  (``max_split_size_mb`` at its minimum plus garbage collection at 0.6), the nearest twin of the reference's exclusive pool.
  The choice has to be made before the first CUDA allocation; ``choose_memory_config`` says so when it is too late.
* ``MARY_POOL_CLEANUP``: ``never`` | ``stage`` (after prefill, before the decode loop; after a finished request batch) |
  ``layer`` (after every decoder layer of a prefill chunk — slow, for prompts that only just fit).
"""
from __future__ import annotations

import enum
import os

from ..utils import flags


class CleanupPolicy(enum.Enum):
    NEVER = "never"
    STAGE = "stage"
    LAYER = "layer"

    @staticmethod
    def choose() -> "CleanupPolicy":
        v = flags.get("MARY_POOL_CLEANUP")
        try:
            return CleanupPolicy(v)
        except ValueError:
            raise ValueError(f"MARY_POOL_CLEANUP={v!r}: expected never | stage | layer") from None


_CONF = {"default": None,
         "expandable": "expandable_segments:True",
         "exclusive": "max_split_size_mb:20,garbage_collection_threshold:0.6"}


def choose_memory_config() -> str:
    """Apply ``MARY_POOL`` through ``PYTORCH_CUDA_ALLOC_CONF``.  Returns the policy name.  Must run before the first CUDA
    allocation of the process; afterwards the allocator has read its configuration and the call raises."""
    import torch
    name = flags.get("MARY_POOL")
    if name not in _CONF:
        raise ValueError(f"MARY_POOL={name!r}: expected one of {sorted(_CONF)}")
    conf = _CONF[name]
    if conf is None:
        return name
    if torch.cuda.is_available() and torch.cuda.is_initialized() and torch.cuda.memory_reserved() > 0:
        raise RuntimeError("MARY_POOL must be applied before the first CUDA allocation of the process")
    prior = os.environ.get("PYTORCH_CUDA_ALLOC_CONF")
    os.environ["PYTORCH_CUDA_ALLOC_CONF"] = conf if not prior else prior + "," + conf
    return name


class Pool:
    """Cleanup hooks the serving loops call at their boundaries; each is a no-op unless the policy asks for it."""

    def __init__(self, policy: CleanupPolicy | None = None):
        self.policy = policy or CleanupPolicy.choose()
        self.released = 0          # bytes handed back to the driver so far

    def _release(self):
        import torch
        if not torch.cuda.is_available():
            return
        before = torch.cuda.memory_reserved()
        torch.cuda.empty_cache()
        self.released += max(0, before - torch.cuda.memory_reserved())

    def after_layer(self):
        if self.policy is CleanupPolicy.LAYER:
            self._release()

    def after_stage(self):
        if self.policy in (CleanupPolicy.STAGE, CleanupPolicy.LAYER):
            self._release()

    def line(self) -> str:
        """One line for logs (the reference's ``pool_line``)."""
        import torch
        if not torch.cuda.is_available():
            return f"pool: policy {self.policy.value}, no CUDA device"
        g = 1 << 30
        return (f"pool: policy {self.policy.value}, reserved {torch.cuda.memory_reserved() / g:.2f} GiB, allocated "
                f"{torch.cuda.memory_allocated() / g:.2f} GiB, released {self.released / g:.2f} GiB")
