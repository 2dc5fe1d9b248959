"""Model locations: an explicit path or ``$MARY_MODELS``; never a guessed default (src/paths.rs:18-56).
``model_opt`` + ``skip_reason`` let tests SKIP, not fail, when a model is absent."""
from __future__ import annotations

import os

from ..utils import flags
from pathlib import Path


def models_dir() -> Path | None:
    v = flags.get("MARY_MODELS") or None
    return Path(v) if v else None


def model_opt(name: str, explicit: str | None = None, env: str | None = None) -> Path | None:
    """explicit argument > per-model environment variable > ``$MARY_MODELS/name``."""
    for cand in (explicit, os.environ.get(env) if env else None):
        if cand:
            p = Path(cand)
            return p if p.exists() else None
    d = models_dir()
    if d is not None and (d / name).exists():
        return d / name
    return None


def skip_reason(name: str, env: str | None = None) -> str:
    where = f"${env} or " if env else ""
    return f"model {name!r} not found: set {where}$MARY_MODELS (no default location is guessed)"


def model(name: str, explicit: str | None = None, env: str | None = None) -> Path:
    p = model_opt(name, explicit, env)
    if p is None:
        raise FileNotFoundError(skip_reason(name, env))
    return p
