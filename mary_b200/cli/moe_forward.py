"""``moe_forward --pile P (--ids 1,2,3[;4,5] | --prompt "...") [--max-new N] [--slots B] [--spec K] [--device cuda] [--trace]``

The serving entry point for the sparse-MoE decoders (Inkling- and K3-style), the counterpart of the reference's
``inkling_forward`` binary (src/bin/inkling_forward.rs): config-free load from a pile, batched decode over ``--slots``
sequences (the reference's ``INK_SLOTS``), MTP speculative decoding with ``--spec`` drafts per step (``INK_MTP``), one CUDA
graph per step on a GPU, and a per-op device-time table with ``--trace`` (the reference's ``stage_sync!`` buckets).  Under
``torchrun`` with several ranks the experts are spread expert-parallel and attention tensor-parallel over the ranks.
Without a tokenizer in the pile, feed ids; several prompts are separated by ``;`` and must have equal lengths (one batch)."""
from __future__ import annotations

import argparse
import sys
import time

import numpy as np
import torch


def main(argv=None) -> int:
    ap = argparse.ArgumentParser(prog="moe_forward")
    ap.add_argument("--pile", required=True)
    ap.add_argument("--ids")
    ap.add_argument("--prompt")
    ap.add_argument("--max-new", type=int, default=32)
    ap.add_argument("--slots", type=int, default=None, help="sequences decoded together (prompts are repeated to fill them)")
    ap.add_argument("--spec", type=int, default=None, help="drafts per step (default: the model's MTP depth, at most 2)")
    ap.add_argument("--device", default="cuda" if torch.cuda.is_available() else "cpu")
    ap.add_argument("--trace", action="store_true")
    ap.add_argument("--metrics", help="append JSON-lines run metrics (steps, requests, acceptance) to this file")
    a = ap.parse_args(argv)
    if argv is None:                                  # run as a program: any uncaught exception on any thread ends the process
        from ..utils import fatal
        fatal.arm()
    from ..runtime import budget
    from ..runtime.pool import Pool, choose_memory_config
    from ..utils.metrics import MetricsLog
    choose_memory_config()
    pool, mlog = Pool(), MetricsLog(a.metrics)
    from ..models.moe.weights import load_from_pile
    from ..pile import Pile
    from ..runtime.kv_cache import PagedKVCache
    from ..runtime.spec_decode import SpecDecoder
    dev = torch.device(a.device)
    dtype = torch.bfloat16 if dev.type == "cuda" else torch.float32
    t0 = time.time()
    pile = Pile.open(a.pile, create=False)
    # the architecture is a FACT in the pile (config.json's model_type), not a flag
    from ..format.persist import load_config, read_model_pile
    from ..format.selection import SelectedModelIndex
    facts0 = read_model_pile(pile)
    arch = load_config(pile, facts0, SelectedModelIndex.from_snapshot(pile, facts0).roots[0]).get("model_type", "mary_moe")
    weights = None
    if arch == "inkling":
        from ..models.inkling.weights import load_from_pile as load_inkling
        model, weights = load_inkling(pile, device=dev, dtype=dtype, max_slots=max(a.slots or 1, 1))
        cfg = model.t
        cfg.num_mtp_layers, cfg.attention, cfg.name = model.n_mtp, "gqa", "inkling"
    else:
        model = load_from_pile(pile, device=dev, dtype=dtype)
        cfg = model.cfg
    print(f"loaded {cfg.name} ({cfg.num_hidden_layers} layers, {cfg.n_routed_experts} experts) in {time.time() - t0:.2f} s", file=sys.stderr)
    if weights is not None:
        print(weights.io_table(), file=sys.stderr)
    tok = None
    if a.prompt is not None:
        from ..format.persist import read_model_pile
        from ..format.tokenizer import build_tokenizer
        tok = build_tokenizer(pile, read_model_pile(pile))
        prompts = [tok.encode(a.prompt, add_special_tokens=False).ids]
    else:
        prompts = [[int(x) for x in p.split(",")] for p in (a.ids or "1").split(";")]
    if len({len(p) for p in prompts}) != 1:
        print("all prompts of one batch must have the same length", file=sys.stderr)
        return 2
    B = a.slots or len(prompts)
    prompts = np.asarray([prompts[i % len(prompts)] for i in range(B)])
    k = min(cfg.num_mtp_layers, 2) if a.spec is None else a.spec
    if k and not cfg.num_mtp_layers:
        print("this model has no MTP layer: --spec 0", file=sys.stderr)
        return 2
    spec = model.kv_spec()
    max_len = prompts.shape[1] + (a.max_new + 2) * (1 + k) + 16
    pages = B * ((max_len + 15) // 16) + 2
    if dev.type == "cuda":
        # admission: the cache and the widest prefill chunk are priced against what is free BEFORE anything is allocated
        free, _ = torch.cuda.mem_get_info(dev)
        if isinstance(spec["kv_heads"], list):
            kv = sum(budget.kv_bytes(1, pages * 16, 2 * h * d * 2) for h, d in zip(spec["kv_heads"], spec["head_dim"]))
        else:
            row = 576 * 2 if cfg.attention == "mla" else 2 * spec["kv_heads"] * spec["head_dim"] * 2
            kv = budget.kv_bytes(spec["num_layers"], pages * 16, row)
        if kv > free:
            raise budget.AdmissionError(f"the paged cache of {B} x {max_len} tokens needs {kv / 2**30:.2f} GiB, {free / 2**30:.2f} GiB are free")
        if arch != "inkling":
            budget.check_prefill(cfg, min(512, prompts.shape[1]) * B, free - kv)
    cache = PagedKVCache(spec["num_layers"], pages, 16, spec["kv_heads"], spec["head_dim"], dtype=dtype, device=dev,
                         latent_dim=spec.get("latent_dim"))
    dec = SpecDecoder(model, cache, B, spec_k=k, max_len=(max_len + 15) // 16 * 16, device=dev, use_graph=dev.type == "cuda" and not a.trace)
    t0 = time.time()
    first = dec.prefill(prompts)
    out = [[int(t)] for t in first.tolist()]
    ttft = time.time() - t0
    pool.after_stage()                                # prefill activations go back before the decode loop captures its graph
    for b in range(B):
        mlog.emit("request", slot=b, prompt_tokens=int(prompts.shape[1]), ttft_s=ttft)
    if dev.type == "cuda":
        dec.capture()
    tracer = None
    if a.trace and dev.type == "cuda":
        from ..utils.trace import Tracer
        tracer = Tracer().__enter__()
    t0 = time.time()
    steps = 0
    while min(len(o) for o in out) < a.max_new:
        ts = time.time()
        dec.step()
        steps += 1
        em, ne = dec.emitted.cpu().numpy(), dec.n_emitted.cpu().numpy()
        for b in range(B):
            out[b].extend(int(t) for t in em[b, :ne[b]])
        mlog.emit("step", seconds=time.time() - ts, tokens_out=int(ne.sum()), accepted=int(ne.sum()) - B, drafted=B * k, slots=B)
    dt = time.time() - t0
    if tracer is not None:
        tracer.__exit__(None, None, None)
        print(tracer.report(), file=sys.stderr)
    for o in out[:len(set(map(tuple, prompts.tolist())))] if a.slots else out:
        o = o[:a.max_new]
        print(tok.decode(o) if tok is not None else ",".join(map(str, o)))
    n = sum(len(o) - 1 for o in out)
    print(f"ttft {ttft * 1e3:.1f} ms; {steps} steps, {n / max(dt, 1e-9):.1f} tok/s over {B} slot(s), "
          f"{n / max(steps * B, 1):.2f} tokens per sequence-step", file=sys.stderr)
    if a.metrics:
        print("metrics: " + str(mlog.summary()), file=sys.stderr)
    print(pool.line(), file=sys.stderr)
    pile.close()
    return 0


if __name__ == "__main__":
    sys.exit(main())
