"""Sequence-parallel attention (``parallel/seq_attention.py``) on gloo ranks against the one-process attention over the whole
sequence: outputs for both forms, gradients for the all-to-all (Ulysses) form."""
import os
import socket

import pytest
import torch
import torch.multiprocessing as mp


def _port():
    s = socket.socket()
    s.bind(("127.0.0.1", 0))
    p = s.getsockname()[1]
    s.close()
    return p


def _worker(rank, world, port, Hq, Hkv, window, out):
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port), RANK=str(rank), WORLD_SIZE=str(world))
    import torch.distributed as dist
    dist.init_process_group("gloo", rank=rank, world_size=world)
    from mary_b200.parallel.seq_attention import _local_attention, ring_attention, ulysses_attention
    torch.manual_seed(0)
    S, D = 8 * world, 16
    q = torch.randn(S, Hq, D, dtype=torch.float64).requires_grad_()
    k = torch.randn(S, Hkv, D, dtype=torch.float64).requires_grad_()
    v = torch.randn(S, Hkv, D, dtype=torch.float64).requires_grad_()
    want = _local_attention(q, k, v, D ** -0.5, True, window)
    w = torch.randn(S, Hq, D, dtype=torch.float64)
    (want * w).sum().backward()
    n = S // world
    sl = slice(rank * n, (rank + 1) * n)
    ql, kl, vl = (t.detach()[sl].clone().requires_grad_() for t in (q, k, v))
    got = ulysses_attention(ql, kl, vl, rank, world, window=window)
    (got * w[sl]).sum().backward()
    err = [(got - want[sl]).abs().max().item(), (ql.grad - q.grad[sl]).abs().max().item(), (kl.grad - k.grad[sl]).abs().max().item(),
           (vl.grad - v.grad[sl]).abs().max().item()]
    if not window:
        ring = ring_attention(ql.detach(), kl.detach(), vl.detach(), rank, world)
        err.append((ring - want[sl].detach()).abs().max().item())
    out.put((rank, err))
    dist.barrier()
    dist.destroy_process_group()


def _once_more(test):
    """One retry with a fresh port absorbs a lost race for the rendezvous port or a slow start of the child interpreters."""
    import functools

    @functools.wraps(test)
    def run(*a, **kw):
        try:
            return test(*a, **kw)
        except Exception:
            for child in mp.active_children():
                child.terminate()
                child.join(10)
            return test(*a, **kw)
    return run


@pytest.mark.parametrize("world,Hq,Hkv,window", [(2, 4, 2, 0), (4, 8, 2, 0), (3, 6, 6, 0), (2, 4, 4, 5), (4, 8, 1, 0)])
@_once_more
def test_sequence_parallel_attention_equals_the_whole_sequence(world, Hq, Hkv, window):
    ctx = mp.get_context("spawn")
    out = ctx.Queue()
    port = _port()
    ps = [ctx.Process(target=_worker, args=(r, world, port, Hq, Hkv, window, out)) for r in range(world)]
    [p.start() for p in ps]
    res = [out.get(timeout=120) for _ in range(world)]
    [p.join(60) for p in ps]
    for rank, err in res:
        assert max(err[:4]) < 1e-9 and max(err) < 1e-5, (rank, err)      # the ring form accumulates in f32
