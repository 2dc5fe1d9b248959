"""Environment flags of the package in one typed registry.

The reference reads 106 environment variables, most of them once through ``OnceLock`` (``INK_*``, ``MARY_*``, ``K3*``; census in
src/bin/inkling_forward.rs:2869-3081,3397-3423 and the ``env::var`` call sites), with the house rule that a diagnostic arm is a
variable one has to type and that removed lanes are deleted, not hidden (:1044-1066).  Here every variable is declared once with
its type, default and meaning; readers call ``flags.get(name)``; ``mary flags`` prints the table with the values in effect.
Model hyper-parameters are never flags: they are facts in the pile."""
from __future__ import annotations

import os
from dataclasses import dataclass


@dataclass(frozen=True)
class Flag:
    name: str
    kind: type
    default: object
    doc: str


_FLAGS: dict[str, Flag] = {}
_CACHE: dict[str, object] = {}


def declare(name: str, kind: type, default, doc: str) -> Flag:
    f = Flag(name, kind, default, doc)
    _FLAGS[name] = f
    return f


def _parse(f: Flag, raw: str):
    if f.kind is bool:
        v = raw.strip().lower()
        if v in ("1", "true", "yes", "on"):
            return True
        if v in ("0", "false", "no", "off", ""):
            return False
        raise ValueError(f"{f.name}={raw!r}: expected 0/1")
    try:
        return f.kind(raw)
    except ValueError as ex:
        raise ValueError(f"{f.name}={raw!r}: expected {f.kind.__name__}") from ex


def get(name: str):
    """Value of a declared flag (environment, else default).  Read once per process, like the reference's ``OnceLock`` flags;
    an undeclared name is a programming error, a malformed value a loud ``ValueError``."""
    if name not in _CACHE:
        f = _FLAGS[name]
        raw = os.environ.get(name)
        _CACHE[name] = f.default if raw is None else _parse(f, raw)
    return _CACHE[name]


def reset() -> None:
    """Forget cached values (tests that change the environment)."""
    _CACHE.clear()


def table() -> list[tuple[str, str, object, object, str]]:
    return [(f.name, f.kind.__name__, f.default, get(f.name), f.doc) for f in sorted(_FLAGS.values(), key=lambda f: f.name)]


declare("MARY_MODELS", str, "", "directory that holds model piles and checkpoints; never guessed (format.paths)")
declare("MARY_GQA_TC", bool, True, "decode-shaped batches of grouped-query models (head dim 128 / 256, 16- or 32-token pages) run the tensor-core decode attention kernel")
declare("MARY_GEMM_SHORT", bool, False, "decode-shaped bf16 GEMMs use a short pipeline (two CTAs fit one SM), so that under MARY_PDL=1 the next GEMM sets up while this one drains")
declare("MARY_LAYER_STEP", bool, True, "one-token steps of one sequence through the dense pre-norm decoders take the five-launch fused layer step")
declare("MARY_PDL", bool, False, "launch the decode-path kernels with programmatic dependent launch")
declare("MARY_MULTIMEM", bool, True, "use the NVSwitch multicast address (multimem.ld_reduce / multimem.st) where the allocation has one")
declare("MARY_ONESHOT", bool, True, "small all-reduces take the one-barrier staged form")
declare("MARY_MOE_GLU_QUANT", bool, True, "with 32-token tiles the first expert GEMM of the planned MoE path quantises its GLU result in the epilogue (0: a second quantiser launch)")
declare("MARY_MOE_FUSED", bool, True, "decode-sized MoE layers take the four-launch pipeline (0: the planned path)")
declare("MARY_CANARY", bool, False, "guard bands around every output buffer the op wrappers allocate; utils.canary.check_all() verifies them")
declare("MARY_DEBUG_CHECKS", bool, False, "validate every batch description on the host before launch (lengths, page ids, page reuse)")
declare("MARY_NVTX", bool, False, "emit NVTX ranges per decoder layer and marks per kernel launch")
declare("MARY_BENCH_LIMIT_S", int, 540, "bench.py ends itself with a stack dump after this many seconds")
declare("MARY_POOL", str, "default", "device allocator policy: default | expandable | exclusive (runtime.pool)")
declare("MARY_POOL_CLEANUP", str, "never", "when cached allocator blocks are returned to the driver: never | stage | layer (runtime.pool)")
declare("MARY_WAIT_MS", int, 2000, "time limit of every device-side wait on another GPU, after which the kernel records a status and returns")
