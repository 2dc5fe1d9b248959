"""Paired capability harness: does a runtime arm (quantised weights, fused kernels, another parallel layout) still answer like the
reference arm?  (golden/paired/paired_score.py of the reference: agreement / loss / McNemar exact with Wilson intervals, a ``--flip K``
synthetic-regression calibration, generation agreement, run-to-run stability.)

An ITEM is a prompt and a few candidate continuations (token ids); an ARM is a callable ``logits(ids) -> [len(ids), vocab]`` (any model
of the package wrapped by ``arm_from_model``).  An arm's answer to an item is the candidate with the highest summed log-probability.
The two arms are compared item by item (paired), which is far more sensitive than comparing two accuracies."""
from __future__ import annotations

import math
from dataclasses import dataclass

import numpy as np
import torch

from .metrics import wilson


@dataclass
class Item:
    prompt: list
    choices: list            # list of token-id lists
    label: int | None = None


def choice_scores(logits_fn, item: Item) -> np.ndarray:
    """Summed log-probability of every candidate continuation given the prompt."""
    out = []
    for ch in item.choices:
        ids = list(item.prompt) + list(ch)
        lp = torch.log_softmax(logits_fn(ids).float(), -1)
        pos = torch.arange(len(item.prompt) - 1, len(ids) - 1)
        out.append(float(lp[pos, torch.tensor(ch)].sum()))
    return np.asarray(out)


def mcnemar_exact(b: int, c: int) -> float:
    """Two-sided exact McNemar p-value from the discordant counts (``b``: only arm A right / chosen, ``c``: only arm B)."""
    n = b + c
    if n == 0:
        return 1.0
    k = min(b, c)
    tail = sum(math.comb(n, i) for i in range(k + 1)) / 2.0 ** n
    return min(1.0, 2.0 * tail)


def compare(scores_a, scores_b, labels=None) -> dict:
    """``scores_* [items, choices]``.  Agreement of the answers with a Wilson interval, mean absolute score gap, and — with labels —
    both accuracies and the exact McNemar test on the discordant items."""
    a, b = np.argmax(scores_a, 1), np.argmax(scores_b, 1)
    n = len(a)
    agree = int((a == b).sum())
    out = {"items": n, "agreement": agree / n, "agreement_ci95": wilson(agree, n),
           "mean_abs_score_gap": float(np.abs(np.asarray(scores_a) - np.asarray(scores_b)).mean())}
    if labels is not None:
        y = np.asarray(labels)
        ra, rb = a == y, b == y
        only_a, only_b = int((ra & ~rb).sum()), int((~ra & rb).sum())
        out.update(acc_a=float(ra.mean()), acc_b=float(rb.mean()), only_a=only_a, only_b=only_b, mcnemar_p=mcnemar_exact(only_a, only_b))
    return out


def flip(scores, k: int, seed: int = 0):
    """Synthetic regression for calibration: make ``k`` items answer differently (their best and second-best candidates swap)."""
    s = np.array(scores, dtype=np.float64, copy=True)
    rng = np.random.default_rng(seed)
    for i in rng.choice(len(s), size=min(k, len(s)), replace=False):
        order = np.argsort(-s[i])
        s[i, order[0]], s[i, order[1]] = s[i, order[1]], s[i, order[0]]
    return s


def generation_agreement(gen_a, gen_b) -> dict:
    """Token-level agreement of greedy continuations (lists of equal-length id lists): overall and up to the first divergence."""
    tot = same = prefix = 0
    for x, y in zip(gen_a, gen_b):
        n = min(len(x), len(y))
        eq = [int(p == q) for p, q in zip(x[:n], y[:n])]
        tot += n
        same += sum(eq)
        prefix += next((i for i, e in enumerate(eq) if not e), n)
    return {"tokens": tot, "agreement": same / max(tot, 1), "agreement_ci95": wilson(same, max(tot, 1)), "mean_common_prefix": prefix / max(len(gen_a), 1)}


def arm_from_model(model, page: int = 16, device="cpu", dtype=torch.float32):
    """Wrap a decoder of the package (``model(ids, meta, cache)`` with ``kv_spec()``) as a logits function over one sequence."""
    from ..runtime.batch import BatchMeta
    from ..runtime.kv_cache import PagedKVCache

    def logits(ids):
        spec = model.kv_spec()
        n = len(ids)
        cache = PagedKVCache(spec["num_layers"], n // page + 2, page, spec["kv_heads"], spec["head_dim"], dtype=dtype, device=device,
                             latent_dim=spec.get("latent_dim"))
        cache.alloc.extend(0, n)
        table, lens = cache.alloc.page_table([0])
        with torch.no_grad():
            return model(torch.as_tensor(ids, dtype=torch.int32, device=device), BatchMeta.build([n], lens, table, page, device=device), cache).cpu()
    return logits


def synthetic_items(vocab: int, n: int, prompt_len: int = 12, choices: int = 4, choice_len: int = 3, seed: int = 0) -> list:
    rng = np.random.default_rng(seed)
    return [Item(rng.integers(1, vocab, prompt_len).tolist(), [rng.integers(1, vocab, choice_len).tolist() for _ in range(choices)])
            for _ in range(n)]
