"""The Inkling decoder on the paged runtime against the reference operators, layout and configuration (CPU, f32)."""
import numpy as np
import pytest
import torch

from mary_b200.models.inkling import layout as L
from mary_b200.models.inkling.config import InklingConfig, tiny_inkling_config
from mary_b200.models.inkling.decoder import RING, InklingDecoder, conv_ring, reference_forward
from mary_b200.ops import reference as ref
from mary_b200.runtime.batch import BatchMeta
from mary_b200.runtime.kv_cache import PagedKVCache


def _decoder(quantized=None, **kw):
    cfg = tiny_inkling_config(**kw)
    return InklingDecoder(cfg, quantized=quantized, dtype=torch.float32, device="cpu", max_slots=4).init_random_(0)


def _cache(dec, pages=32):
    s = dec.kv_spec()
    return PagedKVCache(s["num_layers"], pages, 16, s["kv_heads"], s["head_dim"], dtype=torch.float32)


def _meta(cache, q_lens, seqs):
    table, lens = cache.alloc.page_table(seqs)
    return BatchMeta.build(q_lens, lens, table, 16, "cpu")


def test_config_round_trips_through_json_facts_and_decides_name_sets():
    from mary_b200.format import jsonfacts
    from mary_b200.pile import MemoryBlobStore, TribleBuilder
    cfg = tiny_inkling_config()
    st, tb = MemoryBlobStore(), TribleBuilder()
    jsonfacts.save_document(st, tb, "config.json", cfg.to_json())
    back = InklingConfig.from_json(jsonfacts.load_document(st, tb.build(), "config.json"))     # config from FACTS, no side file
    assert back.text_config == cfg.text_config and back.mtp_config == cfg.mtp_config
    t = back.text_config
    assert t.gate_rows() == 10 and t.effective_vocab() == 300 and t.heads("local") == (4, 4, 32) and t.heads("global") == (4, 2, 32)
    assert t.rel_span("local") == 16 and t.rel_span("global") == 64 and t.is_dense(0) and not t.is_dense(1)
    with pytest.raises(KeyError, match="required"):
        InklingConfig.from_json({"text_config": {"hidden_size": 8}})


def test_layout_is_a_bijection_and_the_header_gate_catches_mutants():
    cfg = tiny_inkling_config()
    ss = L.slots(cfg, {2, 3})                                   # layer 1 keeps bf16 experts, like layer 2 of the released small model
    names = [n for _, n, _, _ in ss]
    assert len(set(names)) == len(names) == 150
    for slot, name, _, _ in ss:
        assert L.parse(name) == slot and L.tensor_name(slot) == name
    assert "model.llm.layers.1.mlp.experts.w13_weight.scale" not in names and "model.llm.layers.2.mlp.experts.w13_weight.scale" in names
    assert L.describe(cfg, {2}, ("llm", 1, "mlp", "moe", "gate_weight"))[0] == (10, 128)          # the sink widens the router
    assert L.describe(cfg, {2}, ("llm", 0, "attn", "wk"))[0] == (128, 128) and L.describe(cfg, {2}, ("llm", 1, "attn", "wk"))[0] == (64, 128)
    hdr = {n: (sh, dt) for _, n, sh, dt in ss}
    assert L.check_headers(cfg, hdr) == []
    for mutate, expect in ((lambda h: h.pop("model.llm.layers.2.mlp.experts.w2_weight.scale2"), "sidecars"),
                           (lambda h: h.update({"model.llm.layers.9.attn.wq_du.weight": ((128, 128), "BF16")}), "no such slot"),
                           (lambda h: h.update({"model.mtp.layers.0.transformer_block.mlp.gate.weight": ((10, 128), "BF16")}), "no such slot"),
                           (lambda h: h.update({"model.llm.layers.1.attn.wq_du.weight": ((64, 128), "BF16")}), "expected"),
                           (lambda h: h.update({"model.visual.layers.0.attn.wq_du.weight": ((1,), "BF16")}), "unmapped")):
        h2 = dict(hdr)
        mutate(h2)
        bad = L.check_headers(cfg, h2, {2, 3})
        assert bad and any(expect in b for b in bad), (expect, bad)
    assert L.parse("model.llm.layers.3.attn.wq_du.weight.extra") is None and L.parse("model.mtp.layers.0.attn_norm.weight") is None


def test_conv_ring_equals_the_sequential_convolution_over_chunks():
    torch.manual_seed(0)
    C, taps = 12, 4
    w = torch.randn(C, taps) * 0.3
    lens = [37, 5, 21]
    xs = [torch.randn(n, C) for n in lens]
    want = [ref.short_conv(x, w, None)[0] for x in xs]
    ring = torch.zeros(4, RING, C)
    cache = PagedKVCache(1, 16, 16, 1, 4, dtype=torch.float32)
    done, got = [0, 0, 0], [[], [], []]
    for chunk in ([20, 5, 1], [1, 0, 3], [16, 0, 17]):           # prefill chunks (one longer than the ring), decode rows, speculative rows
        seqs = [s for s in range(3) if chunk[s]]
        for s in seqs:
            cache.alloc.extend(s, chunk[s])
        meta = _meta(cache, [chunk[s] for s in seqs], seqs)
        x = torch.cat([xs[s][done[s]:done[s] + chunk[s]] for s in seqs])
        y = conv_ring(x, w, ring, torch.tensor(seqs), meta)
        o = 0
        for s in seqs:
            got[s].append(y[o:o + chunk[s]])
            o += chunk[s]
            done[s] += chunk[s]
    for s in range(3):
        assert torch.allclose(torch.cat(got[s]), want[s], atol=1e-5)


@pytest.mark.parametrize("quantized", [set(), None, {2}])
def test_paged_decoder_matches_the_reference_operators(quantized):
    """Prefill in two chunks and three decode steps of two sequences of different lengths in ONE flattened batch: logits equal
    the one-sequence-at-a-time reference (whole sequence at once)."""
    dec = _decoder(quantized)
    cache = _cache(dec)
    rng = np.random.default_rng(1)
    toks = [rng.integers(0, 300, 27).tolist(), rng.integers(0, 300, 12).tolist()]
    want = [reference_forward(dec, t)[0] for t in toks]
    got = [[], []]
    done = [0, 0]
    for chunk in ([20, 5], [4, 4], [1, 1], [1, 1], [1, 1]):
        for s in range(2):
            cache.alloc.extend(s, chunk[s])
        meta = _meta(cache, chunk, [0, 1])
        ids = torch.tensor(sum((toks[s][done[s]:done[s] + chunk[s]] for s in range(2)), []), dtype=torch.int32)
        lg = dec(ids, meta, cache)
        o = 0
        for s in range(2):
            got[s].append(lg[o:o + chunk[s]])
            o += chunk[s]
            done[s] += chunk[s]
    for s in range(2):
        g = torch.cat(got[s])
        w = want[s][:g.shape[0]]
        assert g.shape[1] == 300
        tol = 2e-3 if quantized == set() else 0.08           # NVFP4 layers quantise activations per call: chunking changes nothing, rounding order a little
        assert (g - w).abs().max() <= tol * w.abs().max(), ((g - w).abs().max(), w.abs().max())


def test_rejected_speculative_rows_leave_no_trace():
    """Feed three rows, keep one (the cache length goes back by two), continue: every later logit equals the run that never saw
    the rejected rows — K / V pages and all four convolution rings included (src/models/inkling/burn.rs:2957-2985)."""
    rng = np.random.default_rng(2)
    toks = rng.integers(0, 300, 14).tolist()
    bad = [7, 9]
    outs = []
    for speculate in (False, True):
        dec = _decoder(set())
        cache = _cache(dec)
        cache.alloc.extend(0, 10)
        dec(torch.tensor(toks[:10], dtype=torch.int32), _meta(cache, [10], [0]), cache)
        if speculate:
            cache.alloc.extend(0, 3)
            dec(torch.tensor([toks[10]] + bad, dtype=torch.int32), _meta(cache, [3], [0]), cache)
            cache.alloc.truncate(0, 11)                       # one row kept
            start = 11
        else:
            start = 10
        rows = []
        for p in range(start, 14):
            cache.alloc.extend(0, 1)
            rows.append(dec(torch.tensor([toks[p]], dtype=torch.int32), _meta(cache, [1], [0]), cache))
        outs.append(torch.cat(rows)[-3:])
    assert torch.allclose(outs[0], outs[1], atol=1e-5)


def test_speculative_decoding_with_mtp_heads_emits_the_greedy_tokens():
    from mary_b200.runtime.spec_decode import SpecDecoder
    rng = np.random.default_rng(3)
    prompts = rng.integers(0, 300, (2, 9))
    outs = []
    for k in (0, 2):
        dec = _decoder(set())
        cache = _cache(dec, pages=16)
        sd = SpecDecoder(dec, cache, 2, spec_k=k, max_len=64, device="cpu", use_graph=False)
        first = sd.prefill(prompts, chunk=4)
        seqs = [[int(t)] for t in first.tolist()]
        while min(len(s) for s in seqs) < 10:
            sd.step()
            for b in range(2):
                seqs[b].extend(sd.emitted[b, :int(sd.n_emitted[b])].tolist())
        outs.append([s[:10] for s in seqs])
    assert outs[0] == outs[1]


def test_checkpoint_dictionary_fills_every_slot():
    dec = _decoder({2, 3})
    have = set(dec.P) | {f"model.llm.layers.{i}.mlp.experts.{m}_weight" for i in (1, 2, 3) for m in ("w13", "w2")}
    need = {n for s, n, _, _ in dec.expected() if not ("expert" in s and s[-1] != "weight")}
    assert need == have
    with pytest.raises(KeyError):
        dec.set_tensor("model.llm.layers.0.attn.nonsense.weight", torch.zeros(1))


def test_decoder_round_trips_through_a_pile_with_config_from_facts(tmp_pile):
    """Save to a pile (NVFP4 blobs with placement facts, bf16 leaves, config as facts), load config-free through the Weights
    facade, same logits; the facade counts what it copied and refuses a share that cannot fit before copying."""
    from mary_b200.models.inkling.source import Weights
    from mary_b200.models.inkling.weights import load_from_pile, save_to_pile
    from mary_b200.runtime.budget import AdmissionError
    pile, key = tmp_pile
    dec = _decoder({2, 3})
    save_to_pile(pile, key, dec)
    dec2, w = load_from_pile(pile, dtype=torch.float32)
    assert dec2.quantized == {2, 3} and dec2.cfg.text_config == dec.cfg.text_config
    ids = torch.tensor(np.random.default_rng(0).integers(0, 300, 11), dtype=torch.int32)
    outs = []
    for d in (dec, dec2):
        c = _cache(d)
        c.alloc.extend(0, 11)
        outs.append(d(ids, _meta(c, [11], [0]), c))
    assert (outs[0] - outs[1]).abs().max() <= 0.05 * outs[0].abs().max()       # bf16 storage of the dense tensors of an f32 model
    assert w.stats.tensors > 100 and w.stats.bytes_requested > 0 and w.held("model.llm.embed.weight") > 0 and "GiB requested" in w.io_table()
    assert w.stored("model.llm.embed.weight") == 320 * 128 * 2 and w.document("config.json")["model_type"] == "inkling"
    with pytest.raises(AdmissionError, match="share"):
        Weights.open(pile).admit(w.names(), 0, 1 << 20)
    assert (2, 0) in w.index.experts_in_layers(2, 3)         # placement is a query over facts


def test_moe_forward_serves_an_inkling_pile(tmp_pile, capsys):
    """The serving entry point picks the architecture from the pile's config facts and decodes with the MTP heads drafting."""
    from mary_b200.cli import moe_forward
    from mary_b200.models.inkling.weights import save_to_pile
    pile, key = tmp_pile
    dec = _decoder(set())
    save_to_pile(pile, key, dec)
    path = pile.path
    pile.close()
    outs = []
    for spec in ("0", "2"):
        assert moe_forward.main(["--pile", path, "--ids", "5,6,7,8,9", "--max-new", "6", "--spec", spec, "--device", "cpu"]) == 0
        outs.append(capsys.readouterr().out.strip().splitlines()[-1])
    assert outs[0] == outs[1] and len(outs[0].split(",")) == 6
