"""The allocation-free attention entry point, called through its exported C symbol.

Some users of this library cannot allocate device memory when they call it — a server that already gave all free memory
to its KV cache, code inside a stream capture, a host whose allocator belongs to someone else.  For them the library
carries its own fixed scratch array and exposes ``mary_paged_attention_noalloc``.  This test drives that symbol with
ctypes (no wrapper in between), twice in a row, and compares each result with the regular entry point, which is given a
torch-allocated scratch buffer.  It also checks that an oversized request is refused with the documented status."""
import ctypes

import pytest
import torch

pytestmark = pytest.mark.gpu


def _problem(seed, Hq=16, Hkv=8, D=128):
    from mary_b200.runtime.batch import BatchMeta
    from mary_b200.runtime.kv_cache import PagedKVCache
    torch.manual_seed(seed)
    lens = [700, 33, 1500, 257]
    cache = PagedKVCache(1, sum((l + 15) // 16 for l in lens) + 2, 16, Hkv, D, dtype=torch.bfloat16, device="cuda")
    for s, l in enumerate(lens):
        cache.alloc.extend(s, l)
    table, kl = cache.alloc.page_table(list(range(len(lens))))
    meta = BatchMeta.build([1] * len(lens), kl, table, 16, "cuda")
    cache.k[0].normal_()
    cache.v[0].normal_()
    q = torch.randn(len(lens), Hq, D, device="cuda").bfloat16()
    return cache, meta, q, Hq, Hkv, D


def _args(lib, cache, meta, q, out, Hq, Hkv, D, nsplit):
    NB = meta.num_seqs
    blk_seq = torch.arange(NB, dtype=torch.int32, device="cuda")
    blk_q0 = torch.arange(NB, dtype=torch.int32, device="cuda")
    kc, vc = cache.k[0], cache.v[0]
    p = lambda t: ctypes.c_void_p(t.data_ptr())  # noqa: E731
    keep = (blk_seq, blk_q0)
    a = [p(q), p(kc), p(vc), p(out), p(meta.page_table), p(meta.kv_len), p(meta.q_start), p(blk_seq), p(blk_q0),
         ctypes.c_int(NB), ctypes.c_int(meta.page_table.shape[1]), ctypes.c_int(16),
         ctypes.c_int64(kc.stride(1)), ctypes.c_int64(kc.stride(0)), ctypes.c_int64(vc.stride(1)), ctypes.c_int64(vc.stride(0)),
         ctypes.c_int(Hq), ctypes.c_int(Hkv), ctypes.c_int(D), ctypes.c_int(D), ctypes.c_int(1), ctypes.c_int(nsplit),
         ctypes.c_int(0), ctypes.c_float(D ** -0.5), ctypes.c_float(0.0)]
    return a, keep, NB


def test_noalloc_entry_point_matches_regular_entry_point_twice():
    from mary_b200 import _native
    lib = _native.kernels()
    lib.mary_paged_attention_noalloc.restype = ctypes.c_int
    lib.mary_paged_attention.restype = ctypes.c_int
    lib.mary_paged_attention_scratch_floats.restype = ctypes.c_int64
    lib.mary_status_string.restype = ctypes.c_char_p
    lib.mary_noalloc_scratch_bytes.restype = ctypes.c_int64
    assert lib.mary_noalloc_scratch_bytes() == 16 << 20
    stream = ctypes.c_void_p(torch.cuda.current_stream().cuda_stream)
    # calls in a row share the built-in array; the third one has 256-wide heads, whose kernel needs more dynamic shared
    # memory than the 48 KB default, so it exercises the per-device raise of that limit on a later call
    for call, (seed, nsplit, shape) in enumerate(((1, 4, (16, 8, 128)), (2, 6, (16, 8, 128)), (3, 3, (8, 4, 256)))):
        cache, meta, q, Hq, Hkv, D = _problem(seed, *shape)
        got = torch.full((meta.num_seqs, Hq, D), float("nan"), dtype=torch.bfloat16, device="cuda")
        want = torch.full_like(got, float("nan"))
        a, keep, NB = _args(lib, cache, meta, q, got, Hq, Hkv, D, nsplit)
        if call == 1:
            # same head shape as the call before: nothing is left to set up, so the device's free memory must not move
            torch.cuda.synchronize()
            free_before = torch.cuda.mem_get_info()[0]
        rc = lib.mary_paged_attention_noalloc(*a, stream)
        assert rc == 0, lib.mary_status_string(rc).decode()
        if call == 1:
            torch.cuda.synchronize()
            assert torch.cuda.mem_get_info()[0] == free_before, "the allocation-free entry point changed the free device memory"
        n = lib.mary_paged_attention_scratch_floats(NB, Hkv, nsplit, D)
        scratch = torch.empty(n, dtype=torch.float32, device="cuda")
        b, keep2, _ = _args(lib, cache, meta, q, want, Hq, Hkv, D, nsplit)
        rc = lib.mary_paged_attention(*b, ctypes.c_void_p(scratch.data_ptr()), stream)
        assert rc == 0
        torch.cuda.synchronize()
        assert not torch.isnan(got).any()
        rel = ((got.float() - want.float()).abs().max() / want.float().abs().max()).item()
        assert rel < 2e-2, (call, rel)
        # and both agree with the fp32 reference of the op
        from mary_b200.ops import reference as ref
        oracle = ref.paged_attention(q, cache.k[0], cache.v[0], meta, D ** -0.5)
        assert ((got.float() - oracle.float()).abs().max() / oracle.float().abs().max()).item() < 2e-2


def test_noalloc_entry_point_refuses_oversized_requests():
    from mary_b200 import _native
    lib = _native.kernels()
    lib.mary_paged_attention_noalloc.restype = ctypes.c_int
    lib.mary_status_string.restype = ctypes.c_char_p
    cache, meta, q, Hq, Hkv, D = _problem(3)
    out = torch.zeros(meta.num_seqs, Hq, D, dtype=torch.bfloat16, device="cuda")
    a, keep, NB = _args(lib, cache, meta, q, out, Hq, Hkv, D, 4)
    a[9] = ctypes.c_int(4096)                 # claim 4096 query blocks: 4096*8*4*16*130*4 bytes is far above 16 MiB
    rc = lib.mary_paged_attention_noalloc(*a, ctypes.c_void_p(torch.cuda.current_stream().cuda_stream))
    assert rc == 7
    assert b"16 MiB" in lib.mary_status_string(rc)
    torch.cuda.synchronize()
    assert out.abs().max().item() == 0        # nothing was launched
