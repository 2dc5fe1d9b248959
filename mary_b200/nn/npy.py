""".npy / .npz readers for oracle goldens (src/nn/npy.rs, src/nn/npz.rs) — thin wrappers over NumPy that
refuse pickled payloads."""
from __future__ import annotations

import numpy as np


def load_npy(path) -> np.ndarray:
    return np.load(path, allow_pickle=False)


def load_npz(path) -> dict[str, np.ndarray]:
    with np.load(path, allow_pickle=False) as z:
        return {k: z[k] for k in z.files}
