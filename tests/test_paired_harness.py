"""Paired capability harness on a synthetic model: an arm with rounded weights agrees with the reference arm, the flip calibration
shows that the harness WOULD see a regression of a few items, and the exact McNemar test behaves at its corner cases."""
import copy
import math

import numpy as np
import torch

from mary_b200.utils import paired as P


def test_mcnemar_exact_and_agreement_statistics():
    assert P.mcnemar_exact(0, 0) == 1.0 and P.mcnemar_exact(5, 5) == 1.0
    assert math.isclose(P.mcnemar_exact(0, 6), 2 * 0.5 ** 6) and P.mcnemar_exact(1, 9) < 0.05 < P.mcnemar_exact(2, 6)
    sa = np.array([[3.0, 1, 0], [0, 2, 1], [1, 0, 5], [2, 1, 0]])
    out = P.compare(sa, sa, labels=[0, 1, 2, 1])
    assert out["agreement"] == 1.0 and out["acc_a"] == 0.75 and out["mcnemar_p"] == 1.0 and out["agreement_ci95"][0] < 1.0
    fl = P.flip(sa, 2, seed=1)
    assert P.compare(sa, fl)["agreement"] == 0.5
    g = P.generation_agreement([[1, 2, 3, 4], [5, 6, 7, 8]], [[1, 2, 9, 4], [5, 6, 7, 8]])
    assert g["tokens"] == 8 and g["agreement"] == 7 / 8 and g["mean_common_prefix"] == 3.0


def test_rounded_weights_arm_agrees_and_flips_are_detected():
    from mary_b200.models.gemma4.config import Gemma4TextConfig
    from mary_b200.models.gemma4.model import Gemma4Model
    from mary_b200.models.gemma4.weights import init_random_
    cfg = Gemma4TextConfig(hidden_size=64, num_hidden_layers=2, num_attention_heads=2, head_dim=32, intermediate_size=96, vocab_size=128)
    ref = Gemma4Model(cfg)
    init_random_(ref, 0, std=0.08)
    low = copy.deepcopy(ref)
    for p in low.parameters():
        p.data = p.data.bfloat16().float()                      # the "runtime" arm: same model, weights rounded to bf16
    items = P.synthetic_items(cfg.vocab_size, 24, seed=3)
    a, b = P.arm_from_model(ref), P.arm_from_model(low)
    sa = np.stack([P.choice_scores(a, it) for it in items])
    sb = np.stack([P.choice_scores(b, it) for it in items])
    labels = sa.argmax(1)                                       # the reference arm defines the key on a synthetic pile
    out = P.compare(sa, sb, labels)
    assert out["agreement"] >= 0.9 and out["mean_abs_score_gap"] < 0.5 and out["mcnemar_p"] > 0.05
    # calibration: a regression of 8 of 24 items is seen
    bad = P.compare(sa, P.flip(sb, 8, seed=0), labels)
    assert bad["agreement"] <= out["agreement"] - 0.25 and bad["mcnemar_p"] < 0.05
    # run-to-run stability of one arm: bitwise
    assert np.array_equal(sb, np.stack([P.choice_scores(b, it) for it in items]))
