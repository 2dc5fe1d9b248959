"""Dataset / Sample / TrainingRun / Preference schema (src/dataset.rs:1-75): attribute ids plus small
helpers.  The reference defines the schema only; here the LoRA trainer also records a ``TrainingRun``."""
from __future__ import annotations

from ..pile.trible import TribleBuilder, derived_id, v_f64, v_genid, v_u256
from .model import put_text

_A = lambda n: derived_id(b"mary_b200.dataset", n.encode())  # noqa: E731
DATASET_NAME, SAMPLE_OF, SAMPLE_TEXT, SAMPLE_TOKENS, SAMPLE_INDEX = (_A(n) for n in (
    "dataset_name", "sample_of", "sample_text", "sample_tokens", "sample_index"))
RUN_MODEL, RUN_DATASET, RUN_STEPS, RUN_FINAL_LOSS, RUN_ADAPTER = (_A(n) for n in (
    "run_model", "run_dataset", "run_steps", "run_final_loss", "run_adapter"))
PREF_PROMPT, PREF_CHOSEN, PREF_REJECTED = (_A(n) for n in ("pref_prompt", "pref_chosen", "pref_rejected"))


def put_dataset(store, tb: TribleBuilder, name: str, samples: list[str]) -> bytes:
    d = tb.entity([(DATASET_NAME, put_text(store, name))])
    for i, s in enumerate(samples):
        tb.entity([(SAMPLE_OF, v_genid(d)), (SAMPLE_INDEX, v_u256(i)), (SAMPLE_TEXT, put_text(store, s))])
    return d


def put_training_run(store, tb: TribleBuilder, model_root: bytes, steps: int, final_loss: float,
                     adapter: bytes | None = None, dataset: bytes | None = None) -> bytes:
    pairs = [(RUN_MODEL, v_genid(model_root)), (RUN_STEPS, v_u256(steps)), (RUN_FINAL_LOSS, v_f64(final_loss))]
    if adapter is not None:
        pairs.append((RUN_ADAPTER, v_genid(adapter)))
    if dataset is not None:
        pairs.append((RUN_DATASET, v_genid(dataset)))
    return tb.entity(pairs)


def put_preference(store, tb: TribleBuilder, prompt: str, chosen: str, rejected: str) -> bytes:
    return tb.entity([(PREF_PROMPT, put_text(store, prompt)), (PREF_CHOSEN, put_text(store, chosen)),
                      (PREF_REJECTED, put_text(store, rejected))])
