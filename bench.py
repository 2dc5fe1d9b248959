"""Headline benchmark: decode throughput of the Kimi-K3-class MLA + NVFP4-MoE decoder with 2-token MTP speculation.

``python bench.py --gpus N --steps K --warmup W`` (N > 1 under ``torch.distributed.run``, one rank per GPU).
Metric: confirmed tokens per second of the whole job, device-timed with CUDA events over exactly K decode steps after W
warm-up steps, maximum over ranks.  Weights are random-init of the named architecture, token ids synthetic; the latent KV
cache of the 4096-token contexts is filled with synthetic rows (prefill is outside the timed region; a real prefill of
the same architecture is timed separately for TTFT).  On fewer GPUs than the 540 GB of NVFP4 experts need, MoE layers
share physical expert slabs cyclically — every layer still streams a full slab (far larger than L2) and does the full
arithmetic, only the resident set is smaller; the JSON line says so."""
from __future__ import annotations

import argparse
import json
import os
import subprocess
import sys
import threading
import time

import numpy as np
import torch

ROOT = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, ROOT)


class ClockSampler:
    """Samples SM clocks and throttle reasons of one GPU through NVML (read-only queries, every 20 ms, in a thread) while the
    timed region runs; falls back to an ``nvidia-smi`` loop when the NVML binding is unavailable."""
    Q = ("clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.hw_slowdown,clocks_event_reasons.hw_thermal_slowdown,"
         "clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap")
    BITS = {0x8: "hw_slowdown", 0x40: "hw_thermal_slowdown", 0x20: "sw_thermal_slowdown", 0x4: "sw_power_cap"}

    def __init__(self, index: int):
        self.index, self.rows, self.proc, self.nvml = index, [], None, None
        self.sm, self.reasons, self.max_sm, self._stop = [], set(), None, threading.Event()

    def start(self):
        try:
            import pynvml
            pynvml.nvmlInit()
            try:
                uuid = str(torch.cuda.get_device_properties(self.index).uuid)
                h = pynvml.nvmlDeviceGetHandleByUUID(("GPU-" + uuid) if not uuid.startswith("GPU-") else uuid)
            except Exception:
                h = pynvml.nvmlDeviceGetHandleByIndex(self.index)
            self.max_sm = float(pynvml.nvmlDeviceGetMaxClockInfo(h, pynvml.NVML_CLOCK_SM))
            reasons_fn = getattr(pynvml, "nvmlDeviceGetCurrentClocksEventReasons", None) or pynvml.nvmlDeviceGetCurrentClocksThrottleReasons
            self.nvml = pynvml

            def loop():
                while not self._stop.is_set():
                    try:
                        self.sm.append(float(pynvml.nvmlDeviceGetClockInfo(h, pynvml.NVML_CLOCK_SM)))
                        mask = int(reasons_fn(h))
                        self.reasons.update(n for bit, n in self.BITS.items() if mask & bit)
                    except Exception:
                        pass
                    self._stop.wait(0.02)
            self.thread = threading.Thread(target=loop, daemon=True)
            self.thread.start()
            return
        except Exception:
            self.nvml = None
        try:
            self.proc = subprocess.Popen(["nvidia-smi", f"--id={self.index}", f"--query-gpu={self.Q}", "--format=csv,noheader,nounits",
                                          "-lms", "100"], stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True)
            self.thread = threading.Thread(target=self._read, daemon=True)
            self.thread.start()
        except Exception:
            self.proc = None

    def _read(self):
        for line in self.proc.stdout:
            self.rows.append([c.strip() for c in line.split(",")])

    def stop(self) -> dict:
        if self.nvml is not None:
            self._stop.set()
            self.thread.join(timeout=1)
            sm = sorted(self.sm)
            return {"sm_mhz": sm[len(sm) // 2] if sm else None, "sm_max_mhz": self.max_sm, "reasons": sorted(self.reasons),
                    "samples": len(sm), "source": "nvml"}
        if self.proc is None:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["nvidia-smi unavailable"]}
        self.proc.terminate()
        try:
            self.proc.wait(timeout=2)
        except Exception:
            pass
        sm = sorted(float(r[0]) for r in self.rows if r and r[0].replace(".", "").isdigit())
        mx = [float(r[1]) for r in self.rows if len(r) > 1 and r[1].replace(".", "").isdigit()]
        names = ["hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"]
        reasons = sorted({n for r in self.rows if len(r) >= 7 for n, v in zip(names, r[3:7]) if v.lower().startswith("active")})
        return {"sm_mhz": sm[len(sm) // 2] if sm else None, "sm_max_mhz": max(mx) if mx else None, "reasons": reasons,
                "samples": len(sm), "source": "nvidia-smi"}


def reference_arm(args):
    if int(os.environ.get("RANK", "0")) != 0:          # launched one process per GPU like the own arm: one line, from rank 0
        return
    print(json.dumps({"impl": "reference", "unavailable":
                      "the reference is a Rust crate (Cargo.toml) whose path dependencies ../triblespace-rs and ../cubecl-fork are "
                      "not in the tree and no cargo/rustc exists in this image; pip cannot install it (no setup.py/pyproject.toml)"}))


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=20)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--impl", default="ours")
    ap.add_argument("--arm", default="both", choices=["both", "ours", "library"],
                    help="ours: the product arm only; library: only the same-box library baseline (torch.matmul / torch._grouped_mm / NCCL, none "
                         "of this package's kernels); both: the product arm, then the library arm on the same GPUs, and vs_baseline = ours / library")
    ap.add_argument("--library-steps", type=int, default=4, help="timed steps of the library arm (after 2 warm-up steps)")
    ap.add_argument("--library-limit", type=float, default=240.0, help="seconds after which a stalled library arm is abandoned")
    ap.add_argument("--model", default="k3", choices=["k3", "inkling", "gemma12b", "tiny"],
                    help="k3 is the headline; the others time the remaining workload configurations with the same harness")
    ap.add_argument("--ep", default="auto", choices=["auto", "replicated", "a2a"],
                    help="expert parallel layout for N > 1: replicated tokens + tensor-parallel attention + reduction, or home-rank "
                         "tokens (data-parallel attention) + all-to-all dispatch / combine; auto = all-to-all from 4 ranks up "
                         "(measured on 8 GPUs: 34.8 ms/step against 43.5 ms/step)")
    ap.add_argument("--batch", type=int, default=None)
    ap.add_argument("--ctx", type=int, default=None)
    ap.add_argument("--spec", type=int, default=None)
    ap.add_argument("--comm", default="auto", choices=["auto", "fused", "nccl", "sp"],
                    help="fused: own all-reduce kernels over peer memory; sp: GEMM->reduce-scatter epilogue + fused norm/all-gather (dense decoders); nccl: library arm")
    ap.add_argument("--layers", type=int, default=None, help="debug only: fewer layers (the JSON line then names a reduced config)")
    ap.add_argument("--from-pile", default=None, metavar="PATH",
                    help="MoE decoders: take the weights from a pile instead of initialising them on the device; rank 0 writes the pile first "
                         "when PATH does not exist (the whole single-rank model must fit one GPU for that, so combine with --layers for k3); "
                         "every rank then loads ITS shard config-free (placement facts for experts, the cutting rule for tensor parallelism)")
    ap.add_argument("--no-graph", action="store_true")
    ap.add_argument("--replicated-head", action="store_true", help="keep the whole LM head on every rank (default: vocabulary-parallel head)")
    ap.add_argument("--no-ttft", action="store_true")
    ap.add_argument("--ttft-limit", type=float, default=150.0, help="seconds after which a stalled TTFT measurement is abandoned")
    ap.add_argument("--ttft-layout", default="cp", choices=["cp", "zigzag", "each"],
                    help="all-to-all layout only: cp = one context with its rows split over the ranks (contiguous chunks), zigzag = the same with "
                         "load-balanced chunk pairs (not yet measured on GPUs), each = every rank prefills its own context")
    ap.add_argument("--prefill-chunk", type=int, default=4096, help="tokens per prefill chunk of the TTFT measurement")
    ap.add_argument("--trace", action="store_true", help="print a per-op device-time table of one eager step and exit")
    ap.add_argument("--profile-step", action="store_true",
                    help="run one eager step between cudaProfilerStart/Stop and exit (for ncu --profile-from-start off)")
    ap.add_argument("--trace-prefill", action="store_true", help="print a per-op device-time table of one real prefill of one context and exit")
    args = ap.parse_args()
    if args.impl == "reference":
        return reference_arm(args)
    W = max(args.warmup, 3)
    # a benchmark that stops making progress must end by itself: dump the stacks and exit after the limit
    import faulthandler
    from mary_b200.utils import flags
    faulthandler.dump_traceback_later(flags.get("MARY_BENCH_LIMIT_S"), exit=True)

    def say(msg):
        if os.environ.get("RANK", "0") == "0":
            print(f"[bench {time.strftime('%H:%M:%S')}] {msg}", file=sys.stderr, flush=True)

    from mary_b200.parallel.group import ParallelGroup, init_distributed
    rank, world, local = init_distributed()
    import torch.distributed as dist
    dev = torch.device("cuda", local)
    from mary_b200.models.moe import MoEDecoder, init_random_, inkling_style_config, k3_class_config, tiny_moe_config
    from mary_b200.ops import cuda as K
    from mary_b200.runtime.kv_cache import PagedKVCache
    from mary_b200.runtime.spec_decode import SpecDecoder

    is_gemma = args.model == "gemma12b"
    if is_gemma:
        from mary_b200.models.gemma4 import Gemma4Model, gemma_12b_config
        cfg = gemma_12b_config()
        cfg.name, cfg.num_mtp_layers, cfg.attention = "gemma-4-12b-style", 0, "gqa"
    else:
        cfg = {"k3": k3_class_config, "inkling": inkling_style_config, "tiny": tiny_moe_config}[args.model]()
    pdl = bool(int(os.environ["MARY_PDL"])) if os.environ.get("MARY_PDL", "") in ("0", "1") else (is_gemma and world == 1)
    if pdl != bool(int(os.environ.get("MARY_PDL", "0") or 0)):
        # a dense decoder's step is a chain of small GEMMs, where programmatic dependent launch gains (10.2 -> 9.4 ms measured);
        # with the expert pipeline in the chain it loses, and it has not run with the peer-flag kernels of the multi-GPU layouts
        from mary_b200.ops import cuda as _K
        _K.set_pdl(pdl)
    B = args.batch or {"k3": 128, "inkling": 64, "tiny": 8, "gemma12b": 32}[args.model]
    ctx = args.ctx or {"k3": 4096, "inkling": 1024, "tiny": 256, "gemma12b": 2048}[args.model]
    k = args.spec if args.spec is not None else (2 if cfg.num_mtp_layers else 0)
    if args.ep == "auto":
        args.ep = "a2a" if world >= 4 else "replicated"
    a2a = args.ep == "a2a" and world > 1 and not is_gemma
    if a2a:
        assert B % world == 0
        B_local = B // world
    else:
        B_local = B
    reduced = False
    if args.layers:
        cfg.num_hidden_layers, reduced = args.layers, True

    if args.comm == "auto":       # dense decoder: reduce-scatter / all-gather arm (measured faster at 2 and 8 GPUs); MoE decoders: all-reduce kernels
        args.comm = "sp" if (is_gemma and world > 1) else "fused"
    say(f"model {cfg.name}, {world} rank(s), batch {B}, ctx {ctx}, spec {k}, comm {args.comm}")
    lib_layout = "single" if world == 1 else ("a2a" if a2a else "replicated")
    if args.arm == "library":
        assert args.model == "k3", "the library arm restates the K3-class decoder"
        from mary_b200.library_arm import run_library_arm
        sampler = ClockSampler(local)
        sampler.start()
        res = run_library_arm(cfg, rank, world, lib_layout, B_local, ctx, k, args.steps, W, dev, limit_s=args.library_limit)
        clocks = sampler.stop()
        if rank == 0:
            print(json.dumps({"metric": "decode tok/s (max over ranks), K3-class MLA + MoE, 2-token MTP speculation", "impl": "library",
                              "value": round(res["tokens_per_s"], 2), "unit": "tokens/s", "n_gpus": world, "steps": args.steps, "warmup": W,
                              "ms_per_step": round(res["ms_per_step"], 4), "higher_is_better": True, "scaling": "strong",
                              "dtype": "bf16 activations, bf16 experts", "data": "synthetic token ids, random-init weights, synthetic KV context",
                              "config": {"model": cfg.name, "layers": cfg.num_hidden_layers, "global_batch": B, "seq_len": ctx, "spec_tokens": k,
                                         "parallelism": lib_layout}, "library": res, "clocks": clocks,
                              "e2e": {"value": round(res["e2e_tokens_per_s"], 2), "unit": "tokens/s"}}))
        if world > 1:
            dist.destroy_process_group()
        return
    if world > 1 and args.comm == "nccl":
        # the library arm is launched op by op: recording NCCL collectives into the step graph is not relied upon here
        args.no_graph = True
    symm = None
    if world > 1 and args.comm == "fused":
        try:
            from mary_b200.parallel.symm import SymmetricHeap
            symm = SymmetricHeap(rank, world, dev, max_bytes=max(B * (1 + k), args.prefill_chunk) * cfg.hidden_size * 4)   # decode rows or one prefill chunk
        except Exception as ex:  # the fused path must never be silently absent
            raise RuntimeError(f"fused communication requested but the symmetric heap failed: {ex}") from ex
    par = ParallelGroup(rank, world, "fused" if symm else "nccl", symm=symm, ep_mode="a2a" if a2a else "replicated",
                        vocab_parallel=not args.replicated_head)
    if world > 1 and args.comm == "sp":
        assert is_gemma, "--comm sp is the dense decoders' arm"
        from mary_b200.parallel.sp import SequenceParallel
        par.sp = SequenceParallel.distributed(rank, world, max(B * (1 + k), args.prefill_chunk), cfg.hidden_size, dev)
    if a2a:
        from mary_b200.parallel.ep import distributed_factory
        par.ep_factory = distributed_factory(rank, world, dev, t_cap=B_local * (1 + k))
        par.ep_decode_cap, par.ep_prefill_cap = B_local * (1 + k), args.prefill_chunk

    # ---------------------------------------------------------------- model
    t0 = time.time()
    from_pile = None
    if args.from_pile and not is_gemma:
        from mary_b200.models.moe.weights import load_from_pile, save_to_pile
        from mary_b200.pile import Pile, signing_key_file
        if rank == 0 and not os.path.exists(args.from_pile):
            say(f"writing {args.from_pile}")
            full = MoEDecoder(cfg, dtype=torch.bfloat16, device=dev)
            init_random_(full, seed=0)
            pile = Pile.open(args.from_pile)
            save_to_pile(pile, signing_key_file(args.from_pile + ".key"), full, name=cfg.name)
            pile.close()
            del full
            torch.cuda.empty_cache()
        if world > 1:
            dist.barrier()
        pile = Pile.open(args.from_pile, create=False)
        from_pile = load_from_pile(pile, par=par, device=dev)
        pile.close()
        say(f"loaded this rank's shard from {args.from_pile} in {time.time() - t0:.1f} s")
    model = from_pile if from_pile is not None else (
        Gemma4Model(cfg, tp=par, dtype=torch.bfloat16, device=dev) if is_gemma else MoEDecoder(cfg, par=par, dtype=torch.bfloat16, device=dev))
    B_global, B = B, B_local
    # every step can commit up to 1 + k tokens; the decoder runs the eager census step, the capture warm-up, W warm-up steps,
    # the timed steps and the same number again in the end-to-end loop, all from the same context
    steps_total = W + 2 * args.steps + 8
    max_len = ctx + (steps_total + 8) * (1 + k) + 16
    max_len = (max_len + 15) // 16 * 16
    n_cache_layers = cfg.num_hidden_layers + cfg.num_mtp_layers
    # latent (MLA) caches use 32-token pages: the attention kernel then fetches a whole 32-key stage with one TMA operation;
    # the GQA decoders keep the 16-token pages their workload names
    page = 32 if getattr(cfg, "attention", "") == "mla" else 16
    max_len = (max_len + 31) // 32 * 32
    pages = B * (max_len // page) + 8
    if is_gemma:
        from mary_b200.models.gemma4.weights import init_random_ as gemma_init
        gemma_init(model, 0)
        slabs = n_moe = 0
    else:
        kv_bytes = pages * page * (576 if cfg.attention == "mla" else 2 * max(cfg.num_key_value_heads // par.tp_size, 1) * cfg.head_dim) * 2 * n_cache_layers
        e_local = cfg.n_routed_experts // world
        slab_bytes = e_local * (3 * cfg.hidden_size * cfg.moe_intermediate_size) * (0.5 + 1 / 16) + 1
        free, total = torch.cuda.mem_get_info(dev)
        n_moe = sum(1 for i in range(cfg.num_hidden_layers) if not cfg.is_dense(i)) + cfg.num_mtp_layers
        budget = free - kv_bytes - 12 * (1 << 30)
        slabs = int(max(1, min(n_moe, budget // slab_bytes)))
        if from_pile is None:
            init_random_(model, seed=0, expert_slabs=slabs)
        else:
            slabs = n_moe                                # every layer's experts came from the pile
    # non-expert weights must be identical on every rank that replicates them; experts differ per rank by construction
    spec = model.kv_spec()
    cache = PagedKVCache(spec["num_layers"], pages, page, spec["kv_heads"], spec["head_dim"], dtype=torch.bfloat16, device=dev,
                         latent_dim=spec.get("latent_dim"))
    g = torch.Generator(device=dev).manual_seed(1234)
    for t in cache.k:
        t.normal_(0.0, 1.0, generator=g)
    if cache.v is not cache.k:
        for t in cache.v:
            t.normal_(0.0, 1.0, generator=g)
    dec = SpecDecoder(model, cache, B, spec_k=k, max_len=max_len, device=dev, use_graph=not args.no_graph)
    rng = np.random.default_rng(0)
    dec.set_context(np.full(B, ctx), rng.integers(0, cfg.vocab_size, B), rng.integers(0, cfg.vocab_size, (B, max(k, 1)))[:, :k])
    build_s = time.time() - t0
    say(f"model and cache built in {build_s:.1f} s ({slabs} expert slabs resident)")

    if args.trace_prefill:
        from mary_b200.utils.trace import Tracer
        pc = PagedKVCache(spec["num_layers"], (ctx + 64) // page + 2, page, spec["kv_heads"], spec["head_dim"], dtype=torch.bfloat16,
                          device=dev, latent_dim=spec.get("latent_dim"))
        pd = SpecDecoder(model, pc, 1, spec_k=k, max_len=ctx + 32, device=dev, use_graph=False)
        prompt = rng.integers(0, cfg.vocab_size, (1, ctx))
        pd.prefill(prompt, chunk=args.prefill_chunk)
        torch.cuda.synchronize()
        torch.cuda.profiler.start()          # a profiler started with its capture off sees exactly this prefill
        with Tracer() as tr:
            pd.prefill(prompt, chunk=args.prefill_chunk)
        torch.cuda.synchronize()
        torch.cuda.profiler.stop()
        if rank == 0:
            print(tr.report())
        return
    if args.profile_step:
        with torch.no_grad():
            for _ in range(2):
                dec._step_device()
            torch.cuda.synchronize()
            torch.cuda.profiler.start()
            dec._step_device()
            torch.cuda.synchronize()
            torch.cuda.profiler.stop()
        if world > 1:
            dist.destroy_process_group()
        return
    if args.trace:
        from mary_b200.utils.trace import Tracer
        with torch.no_grad():
            for _ in range(2):
                dec._step_device()
            torch.cuda.synchronize()
            with Tracer() as tr:
                dec._step_device()
        if rank == 0:
            print(tr.report())
        return

    # ---------------------------------------------------------------- capture + launch census
    K.LAUNCHES = 0
    with torch.no_grad():
        dec._step_device()
    torch.cuda.synchronize()
    launches_per_step = K.LAUNCHES
    dec.set_context(np.full(B, ctx), rng.integers(0, cfg.vocab_size, B), rng.integers(0, cfg.vocab_size, (B, max(k, 1)))[:, :k])
    say(f"eager step done ({launches_per_step} launches); capturing")
    dec.capture(warmup=1)
    say("captured" if dec.graph is not None else "running without a graph")
    st = K.last_status()
    if st:
        raise RuntimeError(f"kernel status {st} during warm-up")

    def barrier():
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()

    # ---------------------------------------------------------------- device-timed region
    total_emitted = torch.zeros((), dtype=torch.int64, device=dev)
    for _ in range(W):
        dec.step()
    barrier()
    sampler = ClockSampler(local)
    sampler.start()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    barrier()
    marks = [torch.cuda.Event(enable_timing=True) for _ in range(args.steps)]
    e0.record()
    for i in range(args.steps):
        dec.step()
        total_emitted += dec.n_emitted.sum()
        marks[i].record()                            # one event per step: the percentiles below are percentiles of real steps
    e1.record()
    barrier()
    ms = e0.elapsed_time(e1)
    step_ms = np.array([a.elapsed_time(b) for a, b in zip([e0] + marks[:-1], marks)])
    clocks = sampler.stop()
    say(f"timed region: {ms / args.steps:.3f} ms/step")
    em_t = total_emitted.clone()
    if a2a:
        dist.all_reduce(em_t)                        # every rank decodes its own sequences
    emitted = int(em_t.item())
    t_ms = torch.tensor([ms], dtype=torch.float64, device=dev)
    if world > 1:
        dist.all_reduce(t_ms, op=dist.ReduceOp.MAX)
    ms = float(t_ms.item())
    value = emitted / (ms / 1e3)

    # ---------------------------------------------------------------- end to end through the public loop
    R = 1 + k
    fed_pin = torch.empty(B, R, dtype=torch.int32).pin_memory()
    outs = (torch.empty(B, R, dtype=torch.int32).pin_memory(), torch.empty(B, dtype=torch.int32).pin_memory(),
            torch.empty(B, R, dtype=torch.int32).pin_memory())
    fed_pin.copy_(dec.fed.cpu())
    barrier()
    e2e_tokens = 0
    t_start = time.perf_counter()
    for _ in range(args.steps):
        dec.step_host(fed_pin, outs)                 # H2D of the fed tokens, one step, D2H of tokens / counts / next feed
        e2e_tokens += int(outs[1].sum())
        fed_pin.copy_(outs[2])
    barrier()
    e2e_s = time.perf_counter() - t_start
    if a2a:
        tt = torch.tensor([e2e_tokens], dtype=torch.int64, device=dev)
        dist.all_reduce(tt)
        e2e_tokens = int(tt.item())
    t_e = torch.tensor([e2e_s], dtype=torch.float64, device=dev)
    if world > 1:
        dist.all_reduce(t_e, op=dist.ReduceOp.MAX)
    e2e_value = e2e_tokens / float(t_e.item())
    status = K.last_status()
    say(f"end-to-end loop done, kernel status {status}")

    baseline = {"state": "not run"}
    graph_used = dec.graph is not None
    head_kind = "vocabulary-parallel" if getattr(model, "vocab_parallel", False) else "replicated"

    def emit_line(ttft, ttft_note):
        if rank == 0:
            tok_per_seq_step = emitted / (B_global * args.steps)
            base_ok = isinstance(baseline.get("tokens_per_s"), float)
            line = {
                "metric": "decode tok/s (max over ranks), K3-class MLA + NVFP4 MoE, 2-token MTP speculation" if args.model == "k3" else f"decode tok/s {cfg.name}",
                "value": round(value, 2), "unit": "tokens/s", "n_gpus": world, "steps": args.steps, "warmup": W,
                "ms_per_step": round(ms / args.steps, 4), "higher_is_better": True, "scaling": "strong",
                "vs_baseline": round(value / baseline["tokens_per_s"], 3) if base_ok else None,
                "baseline_ms_per_step": round(baseline["ms_per_step"], 4) if base_ok else None,
                "baseline": dict(baseline, what="same-box library arm of this repository (torch.matmul, torch._grouped_mm, NCCL; bf16 experts, "
                                              "eager launches), same model, batch, context, speculation and layout; the reference itself cannot "
                                              "be built here and publishes no number at this configuration"),
                "dtype": "bf16 activations, NVFP4 experts", "data": "synthetic token ids, random-init weights" + (" written to and loaded from a pile" if from_pile is not None else "") + ", synthetic KV context",
                "impl": "ours",
                "config": {"model": cfg.name + (" (REDUCED layers: debug)" if reduced else ""), "layers": cfg.num_hidden_layers,
                           "global_batch": B_global, "seq_len": ctx, "spec_tokens": k,
                           "parallelism": ("single" if world == 1 else f"tp{world}" if is_gemma else
                                           f"ep{world}-all-to-all+dp{world}-attention" if a2a else f"ep{world}+tp{world}-attention"),
                           "kv_page_tokens": page, "comm": ("sp: gemm->reduce-scatter + fused norm/all-gather" if par.sp is not None else par.mode) if world > 1 else "none", "cuda_graph": graph_used, "dependent_launch": pdl,
                           "lm_head": head_kind,
                           "expert_slabs_resident": slabs, "moe_layers": n_moe,
                           "l2": "each step streams >100x the 126 MB L2 (expert slabs, KV pages), so no flush is needed between steps",
                           "accepted_drafts_per_step": round(tok_per_seq_step - 1, 4)},
                "tpot_ms_mean": round(ms / args.steps / max(tok_per_seq_step, 1e-9), 4),
                "step_ms_p50": round(float(np.percentile(step_ms, 50)), 4), "step_ms_p99": round(float(np.percentile(step_ms, 99)), 4),
                "tpot_ms_p50": round(float(np.percentile(step_ms, 50)) / max(tok_per_seq_step, 1e-9), 4),
                "tpot_ms_p99": round(float(np.percentile(step_ms, 99)) / max(tok_per_seq_step, 1e-9), 4),
                "tpot_note": "percentiles of this rank's per-step CUDA-event times divided by the mean tokens emitted per sequence and step",
                "ttft_ms_p50_one_context": ttft,
                "ttft_note": ttft_note,
                "clocks": clocks,
                "e2e": {"value": round(e2e_value, 2), "unit": "tokens/s", "h2d_bytes_per_step": B * R * 4,
                        "d2h_bytes_per_step": B * R * 4 * 2 + B * 4,
                        "vs_baseline": round(e2e_value / baseline["e2e_tokens_per_s"], 3) if base_ok else None},
                "gpu_launches": launches_per_step * args.steps,
                "kernel_status": status, "build_seconds": round(build_s, 1),
            }
            print(json.dumps(line))

    # the decode result must not be lost to a stalled prefill: if the TTFT measurement has not finished in time, the line is printed
    # without it and the process ends
    done = threading.Event()

    def give_up():
        if not done.is_set():
            emit_line(f"failed: no result within {args.ttft_limit} s", "abandoned")
            sys.stdout.flush()
            os._exit(0)
    stall = threading.Timer(args.ttft_limit, give_up)
    stall.daemon = True
    stall.start()
    # ---------------------------------------------------------------- TTFT: a real prefill of one context
    ttft, ttft_note = None, "median of 3 runs; one context, all ranks"
    pc = pd = None
    if not args.no_ttft:
        try:
            pc = PagedKVCache(spec["num_layers"], (ctx + 64) // page + 2, page, spec["kv_heads"], spec["head_dim"], dtype=torch.bfloat16,
                              device=dev, latent_dim=spec.get("latent_dim"))
            prompt = rng.integers(0, cfg.vocab_size, (1, ctx))
            ts = []
            if a2a and args.ttft_layout == "zigzag":
                # the same context-parallel prefill with load-balanced chunks: rank r takes chunks r and 2 * world - 1 - r of the prompt
                from mary_b200.parallel.cp import ContextParallel
                cp = ContextParallel(rank, world, zigzag=True)
                par.cp = cp
                pc.alloc.extend(0, ctx)
                table, _ = pc.alloc.page_table([0])
                ids_all = torch.as_tensor(prompt[0], dtype=torch.int32, device=dev)
                for _ in range(3):
                    barrier()
                    a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
                    a.record()
                    with torch.no_grad():
                        meta = cp.begin(ctx, table, page, device=dev)
                        idx = torch.cat([torch.arange(lo, hi, device=dev) for lo, hi in (cp.chunks[c] for c in cp.my_chunks())])
                        head = torch.tensor([idx.numel() - 1], device=dev)     # the vocabulary projection for the last local row only
                        tok, h = model.verify(ids_all[idx], meta, pc, rows=head)
                        if k:
                            nxt = torch.where(idx + 1 < ctx, ids_all[(idx + 1).clamp_max(ctx - 1)], tok[-1].to(torch.int32))
                            model.draft(0, h, nxt, meta, pc, rows=head)
                    cp.end()
                    b.record()
                    barrier()
                    ts.append(a.elapsed_time(b))
                ttft_note = f"one context, rows split over {world} ranks in zigzag chunks (context-parallel prefill)"
            elif a2a and args.ttft_layout == "cp":
                # data-parallel attention + expert-parallel all-to-all: ONE context, its rows cut into contiguous chunks, one per rank
                # (context parallelism: after every layer's cache append the earlier chunks' latent rows are gathered into the local
                # cache, attention stays a local kernel); the time is that of the slowest rank, which holds the last chunk
                from mary_b200.parallel.cp import ContextParallel
                cp = ContextParallel(rank, world)
                par.cp = cp
                pc.alloc.extend(0, ctx)
                table, _ = pc.alloc.page_table([0])
                ids_all = torch.as_tensor(prompt[0], dtype=torch.int32, device=dev)
                for _ in range(3):
                    barrier()
                    a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
                    a.record()
                    with torch.no_grad():
                        meta = cp.begin(ctx, table, page, device=dev)
                        lo, hi = cp.bounds[rank]
                        head = torch.tensor([hi - lo - 1], device=dev)         # the vocabulary projection for the last local row only
                        tok, h = model.verify(ids_all[lo:hi], meta, pc, rows=head)
                        if k:                                   # the draft layer's cache rows of this chunk, as the plain prefill fills them
                            nxt = torch.cat([ids_all[lo + 1:hi], ids_all[hi:hi + 1] if hi < ctx else tok[-1:].to(torch.int32)])
                            model.draft(0, h, nxt, meta, pc, rows=head)
                    cp.end()
                    b.record()
                    barrier()
                    ts.append(a.elapsed_time(b))
                ttft_note = f"one context, rows split over {world} ranks (context-parallel prefill)"
            else:          # tensor-parallel attention: all ranks work on the same rows; "each": every rank prefills a context of its own
                pd = SpecDecoder(model, pc, 1, spec_k=k, max_len=ctx + 32, device=dev, use_graph=False)
                for _ in range(3):
                    barrier()
                    a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
                    a.record()
                    pd.prefill(prompt, chunk=args.prefill_chunk)
                    b.record()
                    barrier()
                    ts.append(a.elapsed_time(b))
                if a2a:
                    ttft_note = f"{world} contexts prefilled concurrently, one per rank"
            t_loc = torch.tensor([sorted(ts)[1]], device=dev)
            if world > 1:
                import torch.distributed as dist
                dist.all_reduce(t_loc, op=dist.ReduceOp.MAX)
            ttft = float(t_loc[0])
        except Exception as ex:
            ttft = f"failed: {type(ex).__name__}: {ex}"

    done.set()
    stall.cancel()
    # ---------------------------------------------------------------- the library arm on the same GPUs (the denominator of vs_baseline)
    if args.arm == "both" and args.model == "k3" and not reduced:
        done2 = threading.Event()

        def give_up2():
            if not done2.is_set():
                baseline.update(state=f"abandoned: no result within {args.library_limit} s")
                emit_line(ttft, ttft_note)
                sys.stdout.flush()
                os._exit(0)
        stall2 = threading.Timer(args.library_limit, give_up2)
        stall2.daemon = True
        stall2.start()
        try:
            import gc
            dec.graph = None
            pc = pd = None
            par.cp = None
            del dec, cache, model
            par.__dict__.pop("_fused_moe", None)
            gc.collect()
            torch.cuda.empty_cache()
            from mary_b200.library_arm import run_library_arm
            say("library arm")
            baseline.update(run_library_arm(cfg, rank, world, lib_layout, B, ctx, k, args.library_steps, 2, dev, limit_s=args.library_limit), state="ok")
            say(f"library arm: {baseline['ms_per_step']:.2f} ms/step")
        except Exception as ex:
            baseline.update(state=f"failed: {type(ex).__name__}: {ex}")
        done2.set()
        stall2.cancel()
    emit_line(ttft, ttft_note)
    faulthandler.cancel_dump_traceback_later()
    if world > 1:
        dist.destroy_process_group()


if __name__ == "__main__":
    main()
