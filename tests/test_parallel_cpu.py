"""Tensor/expert-parallel execution on CPU ranks (gloo): the sharded model must reproduce the single-rank model."""
import os
import socket

import numpy as np
import pytest
import torch
import torch.multiprocessing as mp


def _free_port():
    s = socket.socket()
    s.bind(("127.0.0.1", 0))
    p = s.getsockname()[1]
    s.close()
    return p


def _once_more(test):
    """Multi-process tests rendezvous on a port that was free a moment ago and wait on queues with a time limit: one retry with a
    fresh port absorbs a lost race for the port or a slow start of the child interpreters on a loaded machine."""
    import functools

    @functools.wraps(test)
    def run(*a, **kw):
        try:
            return test(*a, **kw)
        except Exception:
            for child in mp.active_children():                      # ranks of the failed attempt must not outlive it
                child.terminate()
                child.join(10)
            return test(*a, **kw)
    return run


def _logits(model, ids, n):
    from mary_b200.runtime.batch import BatchMeta
    from mary_b200.runtime.kv_cache import PagedKVCache
    spec = model.kv_spec()
    cache = PagedKVCache(spec["num_layers"], 16, 16, spec["kv_heads"], spec["head_dim"], dtype=torch.float32,
                         latent_dim=spec.get("latent_dim"))
    cache.alloc.extend(0, n)
    table, lens = cache.alloc.page_table([0])
    meta = BatchMeta.build([n], lens, table, 16)
    with torch.no_grad():
        return model(ids, meta, cache)


def _worker(rank, world, port, attention, out, shared_fp4=False):
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port), RANK=str(rank), WORLD_SIZE=str(world))
    import torch.distributed as dist
    dist.init_process_group("gloo", rank=rank, world_size=world)
    from mary_b200.models.moe import MoEDecoder, init_random_, tiny_moe_config
    from mary_b200.models.moe.shard import shard_from_full
    from mary_b200.parallel.group import ParallelGroup
    torch.manual_seed(0)
    cfg = tiny_moe_config(attention, shared_expert_nvfp4=shared_fp4)
    full = MoEDecoder(cfg, dtype=torch.float32)
    init_random_(full, 0)
    par = ParallelGroup(rank, world, "nccl", vocab_parallel=(attention == "mla"))      # MLA cases also shard the LM head by rows
    shard = shard_from_full(full, par)
    assert shard.vocab_parallel == (attention == "mla")
    ids = torch.arange(1, 20, dtype=torch.int32)
    lg = _logits(shard, ids, 19)
    if shard.vocab_parallel:
        x = torch.randn(5, cfg.hidden_size, generator=torch.Generator().manual_seed(3))
        assert torch.equal(shard.head_argmax(x), full.head_argmax(x))
    if rank == 0:
        ref = _logits(full, ids, 19)
        # a rounding-level difference in the hidden state can flip one expert choice of one token (a discontinuity of
        # top-k routing, not an error), so rows are judged individually
        row_err = (lg - ref).abs().amax(-1)
        out.put((float(row_err.median()), float((row_err < 2e-2 * ref.abs().max()).float().mean()), float(ref.abs().max()), par.calls))
    dist.barrier()
    dist.destroy_process_group()


@pytest.mark.parametrize("attention,shared_fp4", [("mla", False), ("gqa", False), ("mla", True)])
@_once_more
def test_tp_ep_two_cpu_ranks_match_single_rank(attention, shared_fp4):
    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    port = _free_port()
    procs = [ctx.Process(target=_worker, args=(r, 2, port, attention, q, shared_fp4)) for r in range(2)]
    for p in procs:
        p.start()
    med, frac_ok, scale, calls = q.get(timeout=240)
    for p in procs:
        p.join(60)
        assert p.exitcode == 0
    assert med < 1e-2 * scale and frac_ok >= 0.85, (med, frac_ok, scale)
    assert calls > 0                      # the group really reduced partial sums


def test_balanced_split_minimises_the_heaviest_stage():
    from mary_b200.parallel.pp import balanced_split
    assert balanced_split([1, 1, 1, 1], 2) == [(0, 2), (2, 4)]
    r = balanced_split([10, 1, 1, 1, 1, 10], 3)
    assert r[0][0] == 0 and r[-1][1] == 6 and all(a[1] == b[0] for a, b in zip(r, r[1:]))
    assert max(sum([10, 1, 1, 1, 1, 10][lo:hi]) for lo, hi in r) == 10
    assert balanced_split([5], 1) == [(0, 1)]


def _pp_worker(rank, world, port, cohorts, out):
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port), RANK=str(rank), WORLD_SIZE=str(world))
    import torch.distributed as dist
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        from mary_b200.models.moe import MoEDecoder, init_random_, tiny_moe_config
        from mary_b200.parallel.pp import PipeChannel, PipelineStage, balanced_split
        from mary_b200.runtime.batch import BatchMeta
        from mary_b200.runtime.kv_cache import PagedKVCache
        torch.manual_seed(0)
        cfg = tiny_moe_config("gqa")
        m = MoEDecoder(cfg, dtype=torch.float32)
        init_random_(m, 0)
        B, L, n_new = 2, 9, 5
        rng = np.random.default_rng(5)
        prompts = [rng.integers(0, cfg.vocab_size, (B, L)) for _ in range(cohorts)]
        spec = m.kv_spec()
        caches = []
        for c in range(cohorts):
            ca = PagedKVCache(spec["num_layers"], B * 2 + 1, 16, spec["kv_heads"], spec["head_dim"], dtype=torch.float32)
            for s in range(B):
                ca.alloc.extend(s, L + n_new)
            caches.append(ca)

        def make_meta(c, q, kv_len):
            table, _ = caches[c].alloc.page_table(list(range(B)))
            return BatchMeta.build([q] * B, [kv_len] * B, table, 16), caches[c]

        ranges = balanced_split([1] * cfg.num_hidden_layers, world)
        st = PipelineStage(m, ranges, rank, PipeChannel(cfg.hidden_size, B * L, torch.float32, "cpu"))
        res = st.generate(prompts, n_new, make_meta)
        if rank == 0:
            # single-process greedy on fresh caches
            want = []
            for c in range(cohorts):
                ca = PagedKVCache(spec["num_layers"], B * 2 + 1, 16, spec["kv_heads"], spec["head_dim"], dtype=torch.float32)
                for s in range(B):
                    ca.alloc.extend(s, L + n_new)
                table, _ = ca.alloc.page_table(list(range(B)))
                fed, kv, toks = torch.as_tensor(prompts[c], dtype=torch.int32), 0, [[] for _ in range(B)]
                for _ in range(n_new):
                    q = fed.shape[1]
                    meta = BatchMeta.build([q] * B, [kv + q] * B, table, 16)
                    with torch.no_grad():
                        t = m.greedy(fed.reshape(-1), meta, ca, torch.arange(B) * q + (q - 1))
                    kv += q
                    for b in range(B):
                        toks[b].append(int(t[b]))
                    fed = t.to(torch.int32).view(B, 1)
                want.append(toks)
            out.put((res, want))
    finally:
        dist.destroy_process_group()


@pytest.mark.parametrize("cohorts", [1, 3])
@_once_more
def test_layer_pipeline_two_stages_with_cohorts_matches_single_process(cohorts):
    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    port = _free_port()
    ps = [ctx.Process(target=_pp_worker, args=(r, 2, port, cohorts, q)) for r in range(2)]
    for p in ps:
        p.start()
    res, want = q.get(timeout=240)
    for p in ps:
        p.join(60)
    assert res == want


def _vocab_worker(rank, world, port, out):
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port), RANK=str(rank), WORLD_SIZE=str(world))
    import torch.distributed as dist
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        from mary_b200.parallel.vocab import VocabParallelHead
        torch.manual_seed(0)
        W = torch.randn(512, 64)
        W[300] = W[17]                                          # a duplicated row: exact ties between shards
        x = torch.randn(40, 64)
        x[0] = W[17] * 3
        head = VocabParallelHead(VocabParallelHead.shard(W, rank, world), rank, world, softcap=30.0)
        ids, val = head.argmax(x)
        draws = torch.stack([head.sample(x[:4], 0.7, top_k=5, seed=3, step=s) for s in range(200)])
        if rank == 0:
            out.put((ids, val, draws, W, x))
    finally:
        dist.destroy_process_group()


@_once_more
def test_vocab_parallel_head_matches_full_argmax_and_samples_inside_top_k():
    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    port = _free_port()
    ps = [ctx.Process(target=_vocab_worker, args=(r, 2, port, q)) for r in range(2)]
    for p in ps:
        p.start()
    ids, val, draws, W, x = q.get(timeout=120)
    for p in ps:
        p.join(30)
    logits = 30.0 * torch.tanh((x @ W.T) / 30.0)
    from mary_b200.ops import reference as ref
    assert torch.equal(ids, ref.argmax_first(logits))
    assert ids[0] == 17                                           # the tie between rows 17 and 300 goes to the lower index
    assert torch.allclose(val, logits.max(-1).values, atol=1e-5)
    top5 = torch.topk(logits[:4], 5, dim=-1).indices
    for r in range(4):
        seen = set(draws[:, r].tolist())
        assert seen <= set(top5[r].tolist()) and len(seen) >= 2  # draws stay inside the global top-k and do vary


def _cp_worker(rank, world, port, out, zigzag=False):
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port), RANK=str(rank), WORLD_SIZE=str(world))
    import torch.distributed as dist
    dist.init_process_group("gloo", rank=rank, world_size=world)
    from mary_b200.models.gemma4.config import Gemma4TextConfig
    from mary_b200.models.gemma4.model import Gemma4Model, _NoTP
    from mary_b200.models.gemma4.weights import init_random_
    from mary_b200.parallel.cp import ContextParallel
    from mary_b200.runtime.batch import BatchMeta
    from mary_b200.runtime.kv_cache import PagedKVCache
    cfg = Gemma4TextConfig(hidden_size=64, num_hidden_layers=4, num_attention_heads=2, head_dim=32, intermediate_size=96, vocab_size=100,
                           sliding_window=8, num_kv_shared_layers=2)
    m = Gemma4Model(cfg)
    init_random_(m, 0, std=0.05)
    n = 37                                                          # ragged: chunks of 13, 13, 11
    ids = torch.randint(0, 100, (n,), dtype=torch.int32, generator=torch.Generator().manual_seed(1))
    spec = m.kv_spec()

    def fresh():
        c = PagedKVCache(spec["num_layers"], 4, 16, spec["kv_heads"], spec["head_dim"], dtype=torch.float32)
        c.alloc.extend(0, n)
        return c, c.alloc.page_table([0])
    cache, (table, lens) = fresh()
    with torch.no_grad():
        want = m(ids, BatchMeta.build([n], lens, table, 16), cache)
    tp = _NoTP()
    tp.cp = ContextParallel(rank, world, zigzag=zigzag)
    for layer in m.layers:
        layer.tp = tp
    m.tp = tp
    cache, (table, lens) = fresh()
    meta = tp.cp.begin(n, table, 16)
    with torch.no_grad():
        mine = m(tp.cp.rows(ids), meta, cache)
        got = tp.cp.gather_rows(mine)
    if zigzag:
        idx = torch.cat([torch.arange(a, b) for a, b in (tp.cp.chunks[c] for c in tp.cp.my_chunks())])
        out.put((rank, float((got - want).abs().max()), mine.shape[0] == len(idx), float((mine - want[idx]).abs().max())))
    else:
        lo, hi = tp.cp.bounds[rank]
        out.put((rank, float((got - want).abs().max()), mine.shape[0] == hi - lo, float((mine - want[lo:hi]).abs().max())))
    dist.barrier()
    dist.destroy_process_group()


@_once_more
def test_context_parallel_prefill_equals_the_single_rank_prefill():
    world = 3
    ctx = mp.get_context("spawn")
    out = ctx.Queue()
    port = _free_port()
    ps = [ctx.Process(target=_cp_worker, args=(r, world, port, out)) for r in range(world)]
    [p.start() for p in ps]
    res = sorted(out.get(timeout=120) for _ in range(world))
    [p.join(60) for p in ps]
    for rank, err_all, rows_ok, err_mine in res:
        assert rows_ok and err_all < 1e-5 and err_mine < 1e-5, res


@_once_more
def test_zigzag_context_parallel_prefill_equals_the_single_rank_prefill():
    """Rank r takes chunks r and 2 * world - 1 - r of the prompt (two batch entries on one page-table row): same logits as one rank,
    and every rank attends to the same number of half-chunks."""
    world = 3
    ctx = mp.get_context("spawn")
    out = ctx.Queue()
    port = _free_port()
    ps = [ctx.Process(target=_cp_worker, args=(r, world, port, out, True)) for r in range(world)]
    [p.start() for p in ps]
    res = sorted(out.get(timeout=120) for _ in range(world))
    [p.join(60) for p in ps]
    for rank, err_all, rows_ok, err_mine in res:
        assert rows_ok and err_all < 1e-5 and err_mine < 1e-5, res
    from mary_b200.parallel.cp import ContextParallel
    import numpy as np
    work = []
    for r in range(4):
        cp = ContextParallel(r, 4, zigzag=True)
        cp.begin(4096, np.arange(256, dtype=np.int32)[None], 16)
        work.append(sum((b - a) * (a + b) / 2 for a, b in (cp.chunks[c] for c in cp.my_chunks())))      # keys seen, summed over the rank's queries
    assert max(work) / min(work) < 1.01
    flat = []
    for r in range(4):
        cp = ContextParallel(r, 4)
        cp.begin(4096, np.arange(256, dtype=np.int32)[None], 16)
        a, b = cp.bounds[r]
        flat.append((b - a) * (a + b) / 2)
    assert max(flat) / min(flat) > 6                                    # the contiguous layout: the last rank does 7x the first rank's attention


def _cp_mla_worker(rank, world, port, out, zigzag=False):
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port), RANK=str(rank), WORLD_SIZE=str(world))
    import torch.distributed as dist
    dist.init_process_group("gloo", rank=rank, world_size=world)
    from mary_b200.models.moe import MoEDecoder, init_random_, tiny_moe_config
    from mary_b200.parallel.cp import ContextParallel
    from mary_b200.runtime.batch import BatchMeta
    from mary_b200.runtime.kv_cache import PagedKVCache
    cfg = tiny_moe_config("mla")
    m = MoEDecoder(cfg, dtype=torch.float32)                           # every rank holds the whole model: attention is data-parallel
    init_random_(m, 0)
    n = 2 * 56                                                          # 56 rows per rank: above the prefill threshold of the MLA block
    ids = torch.randint(0, cfg.vocab_size, (n,), dtype=torch.int32, generator=torch.Generator().manual_seed(2))
    spec = m.kv_spec()

    def fresh():
        c = PagedKVCache(spec["num_layers"], 9, 16, spec["kv_heads"], spec["head_dim"], dtype=torch.float32, latent_dim=spec.get("latent_dim"))
        c.alloc.extend(0, n)
        return c, c.alloc.page_table([0])
    cache, (table, lens) = fresh()
    with torch.no_grad():
        want_tok, want_h = m.verify(ids, BatchMeta.build([n], lens, table, 16), cache)
    cp = ContextParallel(rank, world, zigzag=zigzag)
    m.par.cp = cp
    cache, (table, lens) = fresh()
    meta = cp.begin(n, table, 16)
    with torch.no_grad():
        tok, h = m.verify(cp.rows(ids), meta, cache)
    cp.end()
    idx = torch.cat([torch.arange(a, b) for a, b in (cp.chunks[c] for c in cp.my_chunks())]) if zigzag else torch.arange(*cp.bounds[rank])
    # routing is discontinuous: judge rows individually, as the tensor-parallel tests do
    row_err = (h - want_h[idx]).abs().amax(-1) / want_h.abs().max()
    out.put((rank, float((row_err < 1e-3).float().mean()), float((tok == want_tok[idx]).float().mean())))
    # outside begin() .. end() the hook is inert: a plain decode step of one row runs without any collective
    cache.alloc.extend(0, 1)
    table, lens = cache.alloc.page_table([0])
    with torch.no_grad():
        m.verify(ids[:1], BatchMeta.build([1], lens, table, 16), cache)
    dist.barrier()
    dist.destroy_process_group()


@pytest.mark.parametrize("zigzag", [False, True])
@_once_more
def test_context_parallel_prefill_of_the_latent_attention_decoder(zigzag):
    world = 2
    ctx = mp.get_context("spawn")
    out = ctx.Queue()
    port = _free_port()
    ps = [ctx.Process(target=_cp_mla_worker, args=(r, world, port, out, zigzag)) for r in range(world)]
    [p.start() for p in ps]
    res = sorted(out.get(timeout=180) for _ in range(world))
    [p.join(60) for p in ps]
    for rank, rows_ok, toks_ok in res:
        assert rows_ok >= 0.95 and toks_ok >= 0.95, res


def _lora_tp_worker(rank, world, port, tp_size, out):
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port), RANK=str(rank), WORLD_SIZE=str(world))
    import torch.distributed as dist
    dist.init_process_group("gloo", rank=rank, world_size=world)
    from mary_b200.models.gemma4 import Gemma4Model, tiny_config
    from mary_b200.models.gemma4.weights import init_random_, shard_from_full
    from mary_b200.parallel.group import ParallelGroup
    from mary_b200.train.lora import LoraWeights
    from mary_b200.train.trainer import LoraTrainer
    torch.manual_seed(0)
    cfg = tiny_config()
    full = Gemma4Model(cfg, dtype=torch.float32)
    init_random_(full, 0)
    full_lora = LoraWeights.init_gemma4(full, rank=4, alpha=8.0, seed=1)
    g = torch.Generator().manual_seed(2)
    for ad in full_lora.adapters.values():
        ad.B.data.normal_(0.0, 0.05, generator=g)                         # non-zero B: every factor gets a gradient
    dp_size = world // tp_size
    tp_rank, dp_rank = rank % tp_size, rank // tp_size
    tp_groups = [dist.new_group(list(range(d * tp_size, (d + 1) * tp_size))) for d in range(dp_size)]
    dp_groups = [dist.new_group(list(range(t, world, tp_size))) for t in range(tp_size)]
    par = ParallelGroup(tp_rank, tp_size, "nccl", group=tp_groups[dp_rank])
    model = shard_from_full(full, par)
    lora = LoraWeights.shard_from_full(full_lora, model, full)
    tr = LoraTrainer(model, rank=4, alpha=8.0, lr=1e-2, dp_size=dp_size, lora=lora, overlap=False,
                     reduce_fn=(lambda t: dist.all_reduce(t, group=dp_groups[tp_rank])) if dp_size > 1 else None,
                     tp_reduce_fn=(lambda t: dist.all_reduce(t, group=tp_groups[dp_rank])) if tp_size > 1 else None)
    ids_all = torch.randint(0, cfg.vocab_size, (dp_size, 2, 24), generator=torch.Generator().manual_seed(3))
    # the same computation on ONE rank: the full model over all replicas' sequences, plain autograd
    ref_tr = LoraTrainer(full, rank=4, alpha=8.0, lr=1e-2, lora=full_lora, overlap=False)
    ref_tr.opt.zero_grad()
    ref_loss = sum(ref_tr.fwd.loss(ids_all[d]) for d in range(dp_size)) / dp_size
    ref_loss.backward()
    ref_grads = {k: (ad.A.grad.clone(), ad.B.grad.clone()) for k, ad in full_lora.adapters.items()}
    tr.opt.zero_grad()
    loss = tr.fwd.loss(ids_all[dp_rank])
    loss.backward()
    worst = 0.0
    for i, (L, Fl) in enumerate(zip(model.layers, full.layers)):
        D = L.D
        kv0 = (tp_rank * Fl.n_kv) // tp_size if Fl.n_kv >= tp_size else 0
        rows = {"q_proj": (tp_rank * L.n_q * D, L.n_q * D), "k_proj": (kv0 * D, L.n_kv * D), "v_proj": (kv0 * D, L.n_kv * D),
                "gate_proj": (tp_rank * L.F, L.F), "up_proj": (tp_rank * L.F, L.F)}
        cols = {"o_proj": (tp_rank * L.n_q * D, L.n_q * D), "down_proj": (tp_rank * L.F, L.F)}
        for p in ("q_proj", "k_proj", "v_proj", "o_proj", "gate_proj", "up_proj", "down_proj"):
            ad = lora.get(i, p)
            ga, gb = ref_grads[f"{i}_{p}"]
            if p in rows:
                o, k = rows[p]
                want_a, want_b = ga, gb[o:o + k]
            else:
                o, k = cols[p]
                want_a, want_b = ga[:, o:o + k], gb
            # after the hooks: gradients are summed over the data-parallel replicas (the step divides by dp_size)
            for got, want in ((ad.A.grad / dp_size, want_a), (ad.B.grad / dp_size, want_b)):
                worst = max(worst, float((got - want).abs().max() / want.abs().max().clamp_min(1e-9)))
    losses = [torch.zeros(()) for _ in range(world)]
    dist.all_gather(losses, loss.detach())
    mean_loss = float(sum(losses[d * tp_size] for d in range(dp_size)) / dp_size)
    # two optimiser steps keep the replicas in lockstep: replicated factors stay identical over the tensor-parallel group
    tr.step(ids_all[dp_rank])
    tr.step(ids_all[dp_rank])
    a0 = lora.get(0, "q_proj").A.detach().clone()
    gathered = [torch.zeros_like(a0) for _ in range(world)]
    dist.all_gather(gathered, a0)
    drift = max(float((t - gathered[0]).abs().max()) for t in gathered)
    if rank == 0:
        out.put((worst, mean_loss, float(ref_loss.detach()), drift, tr.reduced_bytes))
    dist.barrier()
    dist.destroy_process_group()


@pytest.mark.parametrize("world,tp_size", [(2, 2), (4, 2)])
@_once_more
def test_lora_training_under_tensor_and_data_parallelism_has_the_single_rank_gradients(world, tp_size):
    """LoRA training with the base model cut over a tensor-parallel group (and replicated over a data-parallel one): loss and EVERY
    adapter gradient equal plain autograd on the unsharded model — shards compare with their slice, replicated factors after the
    group sum; the replicas stay in lockstep over optimiser steps."""
    ctx = mp.get_context("spawn")
    out = ctx.Queue()
    port = _free_port()
    procs = [ctx.Process(target=_lora_tp_worker, args=(r, world, port, tp_size, out)) for r in range(world)]
    for p in procs:
        p.start()
    worst, loss, ref_loss, drift, reduced = out.get(timeout=240)
    for p in procs:
        p.join(60)
    assert abs(loss - ref_loss) < 1e-4 * max(1.0, abs(ref_loss)), (loss, ref_loss)
    assert worst < 2e-3, worst
    assert drift == 0.0 and reduced > 0
