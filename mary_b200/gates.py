"""Gate commands: small self-contained checks that print PASS / FAIL and carry a positive control.

The reference's main correctness mechanism is a family of ``*_gate`` binaries (src/bin/fp4quant_gate.rs, mxfp4_gate.rs,
inkling_fp4_expert_gate.rs, inkling_layout_gate.rs, inkling_layer_gate.rs, k3_router_gate.rs, k3_tokenizer_gate.rs,
inkling_meta_gate.rs) with a stated tolerance policy — bitwise where the result is an integer, an f64 arbiter over the same
quantised operands for GEMMs — and MUTANTS that show each gate can fail (``--mutate``, golden/mutate_k3_router_gate.py,
scripts/k3_mla_mutants.py), plus a determinism reproducer (golden/determinism/{cmp,nanscan}.py).  The real checkpoints those
binaries read are not available here, so every gate builds its operands from a seed; the rules checked are the same.

``mary gate NAME [--mutate]`` runs one, ``mary gate all`` every one.  With ``--mutate`` the operands or the rule are perturbed
and the command succeeds only if the gate then FAILS."""
from __future__ import annotations

import numpy as np
import torch

GATES = {}


def gate(name):
    def deco(fn):
        GATES[name] = fn
        return fn
    return deco


@gate("fp4quant")
def fp4quant(mutate: bool) -> list[str]:
    """NVFP4 activation quantiser, bit for bit: ties on every code threshold go away from zero, signed zero survives, a zero block
    has scale byte 0, the scale clamps at 448 (src/models/inkling/fp4quant.rs:10-54).  On a GPU the kernel's bytes are compared too."""
    from .nn.fp4 import e4m3_decode, quantize_act_nvfp4
    from .ops import reference as ref
    bad = []
    x = np.zeros((4, 64), dtype=np.float32)
    x[0, :16] = [6, .25, .75, 1.25, 1.75, 2.5, 3.5, 5, -.25, -.75, -1.25, -1.75, -2.5, -3.5, -5, 0.0]
    x[1, :16] = 3e4
    x[2, 0], x[2, 1] = -1e-30, 6.0            # block scale 1.0; the tiny negative rounds to zero but keeps its sign
    x[3] = np.random.default_rng(0).standard_normal(64) * 3
    codes, scales = quantize_act_nvfp4(x)
    want0 = [0x17, 0x32, 0x54, 0x76, 0xA9, 0xCB, 0xED, 0x0F]
    if mutate:
        want0[1] = 0x22                           # as if the tie at 1.25 went TOWARD zero
    if codes[0, :8].tolist() != want0:
        bad.append(f"tie row: {[hex(c) for c in codes[0, :8]]}")
    if e4m3_decode(scales[1, :1])[0] != 448.0:
        bad.append("scale does not clamp at 448")
    if scales[0, 1] != 0 or codes[0, 8:16].any():
        bad.append("a zero block must have scale byte 0 and codes 0")
    if codes[2, 0] & 0xF != 0x8:
        bad.append("a negative value that rounds to zero keeps its sign bit")
    tc, ts = ref.quantize_nvfp4(torch.from_numpy(x).bfloat16())
    xb = torch.from_numpy(x).bfloat16().float().numpy()
    nc, ns = quantize_act_nvfp4(xb)
    if not (np.array_equal(tc.numpy(), nc) and np.array_equal(ts.numpy(), ns)):
        bad.append("torch twin differs from the NumPy quantiser")
    if torch.cuda.is_available():
        from .ops import cuda_moe
        from .ops.moe import unswizzle_scales
        gc, gsf, grm = cuda_moe.quantize_rows(torch.from_numpy(x).bfloat16().cuda(), nt=128, rowmajor=True)
        if not (np.array_equal(gc.cpu().numpy(), nc) and np.array_equal(grm.cpu().numpy(), ns)):
            bad.append("GPU kernel bytes differ")
        if not np.array_equal(unswizzle_scales(gsf.cpu(), 4, 4).numpy(), ns):
            bad.append("GPU scale tile layout differs")
    return bad


@gate("mxfp4")
def mxfp4(mutate: bool) -> list[str]:
    """MXFP4 decode and the EXACT relabel to NVFP4 (global = 2^(e_max - 8), power-of-two E4M3 block scales, duplicated for both
    16-halves), refused when the exponent span exceeds 18 octaves (src/nn/mxfp4.rs:257-361)."""
    from .nn.fp4 import decode_mxfp4, decode_nvfp4, quantize_mxfp4, transcode_mxfp4_to_nvfp4
    bad = []
    rng = np.random.default_rng(1)
    w = rng.standard_normal((8, 128)).astype(np.float32) * np.exp2(rng.integers(-6, 6, (8, 1))).astype(np.float32)
    codes, sc = quantize_mxfp4(w)
    a = decode_mxfp4(codes, sc)
    c2, s2, g = transcode_mxfp4_to_nvfp4(codes, sc)
    b = decode_nvfp4(c2, s2, g)
    if mutate:
        b = b * np.float32(1.0 + 2 ** -20)
    if not np.array_equal(a, b):
        bad.append(f"relabel is not exact: max diff {np.abs(a - b).max()}")
    wide = sc.copy()
    wide[0, 0], wide[1, 0] = 100, 140                     # 40 octaves apart
    try:
        transcode_mxfp4_to_nvfp4(codes, wide)
        bad.append("a 40-octave span was not refused")
    except ValueError:
        pass
    return bad


@gate("nvfp4-expert")
def nvfp4_expert(mutate: bool) -> list[str]:
    """Expert MLP against an f64 arbiter over the SAME quantised operands (src/bin/inkling_fp4_expert_gate.rs:10-25).  The CPU
    lane must agree to f32 accuracy with the arbiter before the bf16 rounding of its outputs; on a GPU the tensor-core lane is
    held to half a bf16 ulp of it."""
    from .ops import reference as ref
    from .ops.moe import NVFP4Experts, experts_forward
    bad = []
    torch.manual_seed(2)
    E, H, F, T, k = 4, 256, 128, 24, 2
    dev = "cuda" if torch.cuda.is_available() else "cpu"
    ex = NVFP4Experts.random(E, H, F, dev, std=0.05, seed=2)
    x = torch.randn(T, H, device=dev).bfloat16()
    idx = torch.stack([torch.randperm(E)[:k] for _ in range(T)]).int().to(dev)
    w = torch.rand(T, k, device=dev)
    got = experts_forward(x, idx, w, ex).float().cpu()
    xd = ref.dequantize_nvfp4(*ref.quantize_nvfp4(x.cpu())).double()
    out = torch.zeros(T, H, dtype=torch.float64)
    for e in range(E):
        t, j = (idx.cpu() == e).nonzero(as_tuple=True)
        if not len(t):
            continue
        w13 = ex.dense("w13", e).double()
        h = torch.nn.functional.silu(xd[t] @ w13[:F].T) * (xd[t] @ w13[F:].T)
        hd = ref.dequantize_nvfp4(*ref.quantize_nvfp4(h.float().bfloat16())).double()
        y = (hd @ ex.dense("w2", e).double().T).float().bfloat16().double()
        out.index_put_((t,), y * w.cpu().double()[t, j][:, None], accumulate=True)
    if mutate:
        out[0, 0] += 0.05
    rel = ((got.double() - out).abs().max() / out.abs().max()).item()
    if rel > 2 ** -7:
        bad.append(f"expert MLP differs from the f64 arbiter by {rel:.3e}")
    return bad


@gate("inkling-layout")
def inkling_layout(mutate: bool) -> list[str]:
    """Name <-> slot bijection of the four towers and the header gate (src/bin/inkling_layout_gate.rs)."""
    from .models.inkling import layout as L
    from .models.inkling.config import tiny_inkling_config
    cfg = tiny_inkling_config()
    ss = L.slots(cfg, {2, 3})
    bad = [f"{n} does not round-trip" for s, n, _, _ in ss if L.parse(n) != s or L.tensor_name(s) != n]
    hdr = {n: (sh, dt) for _, n, sh, dt in ss}
    if mutate:
        hdr.pop("model.llm.layers.2.mlp.experts.w13_weight.scale")
    return bad + L.check_headers(cfg, hdr, {2, 3})


@gate("inkling-layer")
def inkling_layer(mutate: bool) -> list[str]:
    """The paged Inkling decoder against the reference operators, every layer's hidden state (src/bin/inkling_layer_gate.rs,
    inkling_stack_gate.rs).  The mutant swaps the short convolution's tap order."""
    from .models.inkling.config import tiny_inkling_config
    from .models.inkling.decoder import InklingDecoder, reference_forward
    from .runtime.batch import BatchMeta
    from .runtime.kv_cache import PagedKVCache
    dec = InklingDecoder(tiny_inkling_config(), quantized=set(), dtype=torch.float32, device="cpu", max_slots=2).init_random_(0)
    toks = np.random.default_rng(0).integers(0, 300, 21).tolist()
    want, _ = reference_forward(dec, toks)
    if mutate:
        n = "model.llm.layers.1.attn.k_sconv.weight"
        dec.set_tensor(n, dec.P[n].flip(-1))
    s = dec.kv_spec()
    cache = PagedKVCache(s["num_layers"], 8, 16, s["kv_heads"], s["head_dim"], dtype=torch.float32)
    got, done = [], 0
    for n in (16, 4, 1):
        cache.alloc.extend(0, n)
        table, lens = cache.alloc.page_table([0])
        got.append(dec(torch.tensor(toks[done:done + n], dtype=torch.int32), BatchMeta.build([n], lens, table, 16, "cpu"), cache))
        done += n
    rel = ((torch.cat(got) - want).abs().max() / want.abs().max()).item()
    return [f"logits differ from the reference operators by {rel:.3e}"] if rel > 2e-3 else []


@gate("k3-router")
def k3_router(mutate: bool) -> list[str]:
    """``noaux_tc``: select on ``sigmoid + bias``, weigh with the UNBIASED scores renormalised by ``sum + 1e-20`` times the factor
    (src/models/k3/router.rs:9-15).  The mutant weighs with the biased scores (golden/mutate_k3_router_gate.py)."""
    from .ops import reference as ref
    torch.manual_seed(4)
    T, E, k = 32, 64, 6
    lg, bias = torch.randn(T, E), torch.randn(E) * 0.5
    idx, w = ref.router_sigmoid_topk(lg, bias, k, 1, 1, 2.5, True)
    s = torch.sigmoid(lg)
    sel = s + bias
    want_idx = torch.stack([torch.tensor(sorted(range(E), key=lambda e: (-sel[t, e].item(), e))[:k]) for t in range(T)])
    base = (sel if mutate else s).gather(1, want_idx)
    want_w = base / (base.sum(-1, keepdim=True) + 1e-20) * 2.5
    bad = []
    if not torch.equal(idx.long(), want_idx):
        bad.append("selection differs from top-k of sigmoid + bias with ties to the lower index")
    if not torch.allclose(w.float(), want_w, atol=1e-6):
        bad.append("weights are not the unbiased scores renormalised")
    if torch.cuda.is_available():
        from .ops import cuda as K
        gi, gw = K.router_topk(lg.cuda(), k, "sigmoid", bias.cuda(), 1, 1, 2.5, True)
        if not (torch.equal(gi.cpu().long(), want_idx) and torch.allclose(gw.cpu(), want_w, atol=1e-5)):
            bad.append("GPU router differs")
    return bad


@gate("tokenizer")
def tokenizer(mutate: bool) -> list[str]:
    """Tokenizer as a fact graph: rebuilt without JSON, it encodes id for id like the original (src/bin/k3_tokenizer_gate.rs,
    inkling_tokenizer_gate.rs).  The mutant drops one merge before the comparison."""
    import json
    from tokenizers import Tokenizer, decoders, models, pre_tokenizers
    from .format.tokenizer import build_tokenizer, save_tokenizer_json
    from .pile import MemoryBlobStore, TribleBuilder
    vocab = {"<unk>": 0, "h": 1, "e": 2, "l": 3, "o": 4, "he": 5, "ll": 6, "hell": 7, "hello": 8, "Ġ": 9, "w": 10}
    merges = [("h", "e"), ("l", "l"), ("he", "ll"), ("hell", "o")]
    tok = Tokenizer(models.BPE(vocab=vocab, merges=merges, unk_token="<unk>"))
    tok.pre_tokenizer = pre_tokenizers.ByteLevel(add_prefix_space=False)
    tok.decoder = decoders.ByteLevel()
    st, tb = MemoryBlobStore(), TribleBuilder()
    doc = json.loads(tok.to_str())
    if mutate:
        doc["model"]["merges"] = doc["model"]["merges"][:-1]
    save_tokenizer_json(st, tb, "gate", json.dumps(doc))
    rebuilt = build_tokenizer(st, tb.build())
    bad = []
    for s in ("hello", "hello hello", "hellow"):
        if rebuilt.encode(s).ids != tok.encode(s).ids:
            bad.append(f"{s!r}: {rebuilt.encode(s).ids} != {tok.encode(s).ids}")
    return bad


@gate("json")
def json_meta(mutate: bool) -> list[str]:
    """A checkpoint's JSON sidecars as facts: the canonical serialisation of the round trip equals the source byte for byte
    (src/bin/inkling_meta_gate.rs)."""
    import json
    from .format import jsonfacts
    from .models.inkling.config import tiny_inkling_config
    from .pile import MemoryBlobStore, TribleBuilder
    doc = tiny_inkling_config().to_json()
    doc["eos_token_id"], doc["architectures"], doc["ratio"] = [1, 1], ["InklingForCausalLM"], 16.0
    st, tb = MemoryBlobStore(), TribleBuilder()
    jsonfacts.save_document(st, tb, "config.json", doc)
    back = jsonfacts.load_document(st, tb.build(), "config.json")
    if mutate:
        back["ratio"] = 16
    a, b = json.dumps(doc, sort_keys=True), json.dumps(back, sort_keys=True)
    return [] if a == b else ["round trip is not exact: " + next(f"{x!r} != {y!r}" for x, y in zip(a.split(","), b.split(",")) if x != y)]


@gate("determinism")
def determinism(mutate: bool) -> list[str]:
    """Run-to-run stability (golden/determinism/cmp.py, nanscan.py): the same decode steps from the same state, twice — emitted
    tokens and logits must be bit-identical and free of NaN / Inf.  The reference traced its own flips (43 of 503 positions) to the
    GPU reading reclaimed file pages; here weights live in device memory, so any flip is a kernel's.  On a GPU the check runs the
    MoE decoder's step (stream-K GEMMs included: their partial sums are added in arrival order, so the LOGITS may differ in the
    last bit; the gate reports that separately and fails only on a token flip or a non-finite value)."""
    from .models.moe import MoEDecoder, init_random_, tiny_moe_config
    from .runtime.batch import BatchMeta
    from .runtime.kv_cache import PagedKVCache
    dev = "cuda" if torch.cuda.is_available() else "cpu"
    cfg = tiny_moe_config("mla")
    m = MoEDecoder(cfg, dtype=torch.bfloat16 if dev == "cuda" else torch.float32, device=dev)
    init_random_(m, 0)
    ids = torch.tensor(np.random.default_rng(0).integers(0, cfg.vocab_size, 40), dtype=torch.int32, device=dev)
    runs = []
    for rep in range(2):
        spec = m.kv_spec()
        cache = PagedKVCache(spec["num_layers"], 8, 16, spec["kv_heads"], spec["head_dim"], dtype=m.dtype, device=dev, latent_dim=spec.get("latent_dim"))
        cache.alloc.extend(0, 40)
        table, lens = cache.alloc.page_table([0])
        with torch.no_grad():
            lg = m(ids, BatchMeta.build([40], lens, table, 16, dev), cache).float().cpu()
        if mutate and rep == 1:
            lg[7, lg[7].argmax()] = float("nan")
        runs.append(lg)
    bad = []
    for i, lg in enumerate(runs):
        if not torch.isfinite(lg).all():
            bad.append(f"run {i}: {int((~torch.isfinite(lg)).sum())} non-finite logits")
    flips = int((runs[0].argmax(-1) != runs[1].argmax(-1)).sum())
    if flips:
        bad.append(f"{flips} of {runs[0].shape[0]} positions flip their arg-max between two runs")
    if not torch.equal(runs[0], runs[1]) and not bad:
        ulp = (runs[0] - runs[1]).abs().max().item()
        print(f"  note: logits differ in the last bits between runs (max {ulp:.3e}); tokens are stable")
    return bad


def run(name: str, mutate: bool = False) -> int:
    names = list(GATES) if name == "all" else [name]
    rc = 0
    for n in names:
        if n not in GATES:
            print(f"unknown gate {n!r}; known: {', '.join(GATES)}")
            return 2
        bad = GATES[n](mutate)
        if mutate:
            ok = bool(bad)
            print(f"{n}: mutant {'caught' if ok else 'NOT caught'}" + (f" ({bad[0]})" if bad else ""))
        else:
            ok = not bad
            print(f"{n}: {'PASS' if ok else 'FAIL'}")
            for b in bad[:10]:
                print(f"  {b}")
        rc |= 0 if ok else 1
    return rc
