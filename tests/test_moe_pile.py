import numpy as np
import pytest
import torch

from mary_b200.models.moe import MoEDecoder, init_random_, tiny_moe_config
from mary_b200.models.moe.weights import load_from_pile, save_to_pile
from mary_b200.runtime.budget import AdmissionError, check, moe_bill, query_block
from mary_b200.utils.metrics import MetricsLog, wilson


def test_moe_model_roundtrips_through_a_pile_config_free(tmp_path):
    from mary_b200.pile import Pile, signing_key_file
    cfg = tiny_moe_config("mla", num_mtp_layers=0)
    m = MoEDecoder(cfg, dtype=torch.bfloat16)
    init_random_(m, 0)
    pile = Pile.open(str(tmp_path / "m.pile"))
    save_to_pile(pile, signing_key_file(str(tmp_path / "k")), m, "tiny")
    pile.close()
    pile = Pile.open(str(tmp_path / "m.pile"), create=False)
    m2 = load_from_pile(pile)                                   # hyper-parameters and placement come from facts
    assert m2.cfg == cfg
    for (n, a), (_, b) in zip(m.named_parameters(), m2.named_parameters()):
        assert torch.equal(a, b), n
    e1 = [x for x in m.modules() if hasattr(x, "experts") and x.experts is not None]
    e2 = [x for x in m2.modules() if hasattr(x, "experts") and x.experts is not None]
    for a, b in zip(e1, e2):
        assert torch.equal(a.experts.w13_q, b.experts.w13_q) and torch.equal(a.experts.w2_sf, b.experts.w2_sf)
        assert torch.allclose(a.experts.w13_s2, b.experts.w13_s2)
    # an expert-parallel rank asks the placement facts for its experts only
    class Par:
        rank = size = 0
        tp_rank, tp_size, ep_rank, ep_size, ep_mode = 0, 1, 1, 2, "replicated"
    m3 = load_from_pile(pile, par=Par())
    assert e1[0].experts.E == 8 and [x for x in m3.modules() if hasattr(x, "experts") and x.experts is not None][0].experts.E == 4
    # a tensor-parallel rank loads ITS shard from the pile: equal to cutting the full model in memory, for every rank
    from mary_b200.models.moe.shard import shard_from_full
    from mary_b200.parallel.group import ParallelGroup
    for vocab_parallel in (False, True):
        for r in range(2):
            par = ParallelGroup(rank=r, size=2, vocab_parallel=vocab_parallel)
            want, got = shard_from_full(m, par), load_from_pile(pile, par=ParallelGroup(rank=r, size=2, vocab_parallel=vocab_parallel))
            cut = 0
            for (n, a), (_, b) in zip(want.named_parameters(), got.named_parameters()):
                assert a.shape == b.shape and torch.equal(a, b), n
                cut += int(a.numel() < dict(m.named_parameters())[n].numel())
            assert cut >= 4                                                  # attention, dense FFN (and the head) really are slices
            for a, b in zip([x for x in want.modules() if getattr(x, "experts", None) is not None],
                            [x for x in got.modules() if getattr(x, "experts", None) is not None]):
                assert a.experts.E == b.experts.E and torch.equal(a.experts.w13_q, b.experts.w13_q) and torch.equal(a.experts.w2_sf, b.experts.w2_sf)
    pile.close()


def test_admission_bill_and_metrics():
    from mary_b200.models.moe import k3_class_config
    cfg = k3_class_config()
    bill = moe_bill(cfg, world=8, batch=128, max_len=5120, rows_per_step=384, capacity=180 << 30)
    assert 60 << 30 < bill.weights < 90 << 30          # ~540 GB of NVFP4 experts over 8 ranks plus bf16 attention
    check(bill)
    with pytest.raises(AdmissionError, match="does not fit"):
        check(moe_bill(cfg, world=1, batch=128, max_len=5120, rows_per_step=384, capacity=180 << 30))
    assert query_block(64, 4096) == (4 << 30) // (64 * 4096 * 4)
    lo, hi = wilson(71, 100)
    assert lo < 0.71 < hi and hi - lo < 0.2
    log = MetricsLog()
    log.emit("step", tokens_out=128, seconds=0.1, accepted=30, drafted=256)
    log.emit("request", ttft_s=0.5)
    s = log.summary()
    assert abs(s["tokens_per_s"] - 1280) < 1e-6 and abs(s["acceptance"] - 30 / 256) < 1e-9


def test_moe_forward_cli_serves_a_pile_and_maintenance_commands(tmp_path, capsys):
    """The serving CLI loads a persisted decoder config-free and decodes batched slots with MTP speculation; its tokens equal
    plain greedy decoding; ``mary branches|verify|stats`` read the same pile."""
    from mary_b200.cli import mary, moe_forward
    from mary_b200.models.moe.weights import save_to_pile
    from mary_b200.pile import Pile, signing_key_file
    torch.manual_seed(0)
    cfg = tiny_moe_config("mla")
    m = MoEDecoder(cfg, dtype=torch.bfloat16)
    init_random_(m, 0)
    path = str(tmp_path / "m.pile")
    pile = Pile.open(path)
    save_to_pile(pile, signing_key_file(str(tmp_path / "key")), m, name="tiny-moe")
    pile.close()
    outs = {}
    for spec in (0, 2):
        assert moe_forward.main(["--pile", path, "--ids", "5,6,7,8,9;11,12,13,14,15", "--max-new", "6", "--spec", str(spec), "--device", "cpu"]) == 0
        outs[spec] = [l for l in capsys.readouterr().out.strip().splitlines() if l]
    assert len(outs[0]) == 2 and outs[0] == outs[2]                    # speculation never changes the tokens
    assert all(len(l.split(",")) == 6 for l in outs[0])
    assert mary.main(["branches", "--pile", path]) == 0
    assert mary.main(["verify", "--pile", path, "--deep"]) == 0
    assert "0 problems" in capsys.readouterr().out
    assert mary.main(["stats", "--pile", path]) == 0
