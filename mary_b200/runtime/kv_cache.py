"""Paged KV cache: native page allocator (``_core.so``) + the device tensors that hold the pages.

Pages are 16 tokens by default.  One cache instance serves all layers: ``k[layer]`` / ``v[layer]`` have shape
``[num_pages, page_size, kv_heads, head_dim]``; MLA models use a single latent tensor per layer
(``[num_pages, page_size, kv_lora + rope_dim]``).  A sequence's page list is shared by every layer."""
from __future__ import annotations

import ctypes

import numpy as np
import torch

from .. import _native


def _declare(lib):
    if getattr(lib, "_kv_declared", False):
        return
    c = ctypes
    lib.kv_create.restype = c.c_void_p
    lib.kv_create.argtypes = [c.c_int32, c.c_int32]
    lib.kv_destroy.argtypes = [c.c_void_p]
    lib.kv_free_pages.argtypes = [c.c_void_p]
    lib.kv_peak_used.restype = c.c_int64
    lib.kv_peak_used.argtypes = [c.c_void_p]
    lib.kv_seq_len.restype = c.c_int64
    lib.kv_seq_len.argtypes = [c.c_void_p, c.c_int64]
    lib.kv_extend.restype = c.c_int64
    lib.kv_extend.argtypes = [c.c_void_p, c.c_int64, c.c_int64]
    lib.kv_truncate.restype = c.c_int64
    lib.kv_truncate.argtypes = [c.c_void_p, c.c_int64, c.c_int64]
    lib.kv_release.argtypes = [c.c_void_p, c.c_int64]
    lib.kv_pages.argtypes = [c.c_void_p, c.c_int64, c.c_void_p, c.c_int32]
    lib.kv_page_table.argtypes = [c.c_void_p, c.c_void_p, c.c_int32, c.c_void_p, c.c_int32, c.c_void_p]
    lib.sched_create.restype = c.c_void_p
    lib.sched_create.argtypes = [c.c_void_p, c.c_int32, c.c_int32, c.c_int32]
    lib.sched_destroy.argtypes = [c.c_void_p]
    lib.sched_add.argtypes = [c.c_void_p, c.c_int64, c.c_void_p, c.c_int32, c.c_int32]
    lib.sched_add.restype = c.c_int32
    lib.sched_num_waiting.argtypes = [c.c_void_p]
    lib.sched_num_running.argtypes = [c.c_void_p]
    lib.sched_set_drafts.argtypes = [c.c_void_p, c.c_int64, c.c_void_p, c.c_int32]
    lib.sched_next.argtypes = [c.c_void_p] + [c.c_void_p] * 9
    lib.sched_commit.argtypes = [c.c_void_p, c.c_int64, c.c_int32, c.c_int32, c.c_int32, c.c_int32]
    lib.sched_is_finished.argtypes = [c.c_void_p, c.c_int64]
    lib.sched_remove.argtypes = [c.c_void_p, c.c_int64]
    lib._kv_declared = True


class OutOfPages(RuntimeError):
    pass


class PageAllocator:
    def __init__(self, num_pages: int, page_size: int = 16):
        self.lib = _native.core()
        _declare(self.lib)
        self.num_pages, self.page_size = num_pages, page_size
        self.h = self.lib.kv_create(num_pages, page_size)

    def extend(self, seq: int, tokens: int) -> int:
        n = self.lib.kv_extend(self.h, seq, tokens)
        if n < 0:
            raise OutOfPages(f"sequence {seq}: no free pages for {tokens} more tokens "
                             f"({self.free_pages} of {self.num_pages} pages free)")
        return n

    def truncate(self, seq: int, new_len: int) -> None:
        if self.lib.kv_truncate(self.h, seq, new_len) < 0:
            raise ValueError(f"cannot truncate sequence {seq} to {new_len}")

    def release(self, seq: int) -> None:
        self.lib.kv_release(self.h, seq)

    def seq_len(self, seq: int) -> int:
        return self.lib.kv_seq_len(self.h, seq)

    @property
    def free_pages(self) -> int:
        return self.lib.kv_free_pages(self.h)

    @property
    def peak_used(self) -> int:
        return self.lib.kv_peak_used(self.h)

    def pages(self, seq: int) -> list[int]:
        buf = np.empty(self.num_pages, dtype=np.int32)
        n = self.lib.kv_pages(self.h, seq, buf.ctypes.data, buf.size)
        if n < 0:
            raise KeyError(seq)
        return buf[:n].tolist()

    def page_table(self, seqs, max_pages: int | None = None):
        """``(table int32[n, max_pages] padded with -1, kv_lens int32[n])`` as NumPy arrays."""
        s = np.asarray(seqs, dtype=np.int64)
        if max_pages is None:
            max_pages = max(1, max((self.seq_len(int(x)) + self.page_size - 1) // self.page_size for x in s))
        table = np.empty((len(s), max_pages), dtype=np.int32)
        lens = np.empty(len(s), dtype=np.int32)
        rc = self.lib.kv_page_table(self.h, s.ctypes.data, len(s), table.ctypes.data, max_pages, lens.ctypes.data)
        if rc != 0:
            raise ValueError("page table: unknown sequence or max_pages too small")
        return table, lens

    def __del__(self):
        try:
            self.lib.kv_destroy(self.h)
        except Exception:
            pass


class Q8Pages:
    """The pages of one layer's K (or V) as 8-bit codes: ``codes [pages, page, Hkv, D]`` unsigned bytes and ``sz [pages, page, Hkv, 2]``
    f32 ``(scale, zero)`` per (token, kv head); element = ``code * scale + zero``, ``scale = (max - min) / 255``, ``zero = min`` — the
    grouping and rounding of the reference's device cache quantiser (src/models/gemma/gpu_quant.rs:28-166), which packs four codes
    per 32-bit word where this keeps plain bytes.  Half the bytes of a bf16 cache plus 8 bytes per (token, head)."""

    def __init__(self, num_pages: int, page_size: int, kv_heads: int, head_dim: int, device="cpu"):
        self.codes = torch.zeros(num_pages, page_size, kv_heads, head_dim, dtype=torch.uint8, device=device)
        self.sz = torch.zeros(num_pages, page_size, kv_heads, 2, dtype=torch.float32, device=device)
        self.sz[..., 0] = 1.0

    shape = property(lambda self: self.codes.shape)
    device = property(lambda self: self.codes.device)
    is_cuda = property(lambda self: self.codes.is_cuda)

    def dim(self) -> int:
        return 4

    def nbytes(self) -> int:
        return self.codes.numel() + self.sz.numel() * 4

    @staticmethod
    def quantize(rows):
        """``rows [..., D]`` -> ``(codes uint8, sz [..., 2] f32)`` by the rule above (round half up, as the device kernel)."""
        x = rows.float()
        lo, hi = x.min(-1, keepdim=True).values, x.max(-1, keepdim=True).values
        rng = hi - lo
        sc = torch.where(rng > 0, rng / 255.0, torch.ones_like(rng))
        codes = torch.floor((x - lo) / sc + 0.5).clamp(0, 255).to(torch.uint8)
        return codes, torch.cat([sc, lo], -1)

    def append(self, rows, slots) -> None:
        """Quantise ``rows [T, Hkv, D]`` into the flat slots ``slots [T]`` (page * page_size + offset)."""
        codes, sz = self.quantize(rows)
        self.codes.view(-1, *self.codes.shape[2:])[slots.long()] = codes
        self.sz.view(-1, *self.sz.shape[2:])[slots.long()] = sz

    def dequantize(self, pages=None, dtype=torch.bfloat16):
        """bf16 pages ``[n, page, Hkv, D]`` of the listed pages (all when ``None``)."""
        c = self.codes if pages is None else self.codes[pages.long()]
        z = self.sz if pages is None else self.sz[pages.long()]
        return (c.float() * z[..., :1] + z[..., 1:]).to(dtype)


class PagedKVCache:
    """Device storage for the pages of every layer.  ``kv_dtype="int8"`` keeps K and V as :class:`Q8Pages`."""

    def __init__(self, num_layers: int, num_pages: int, page_size: int, kv_heads: int | list[int], head_dim: int | list[int],
                 dtype=torch.bfloat16, device="cpu", latent_dim: int | None = None, alias_v_to_k: bool = False, kv_dtype: str | None = None):
        self.alloc = PageAllocator(num_pages, page_size)
        self.page_size, self.num_pages, self.num_layers = page_size, num_pages, num_layers
        self.latent = latent_dim is not None
        heads = kv_heads if isinstance(kv_heads, list) else [kv_heads] * num_layers
        dims = head_dim if isinstance(head_dim, list) else [head_dim] * num_layers
        self.kv_dtype = kv_dtype
        if kv_dtype not in (None, "int8"):
            raise ValueError(f"kv_dtype {kv_dtype!r}: only None (the activation dtype) and 'int8' are implemented")
        if kv_dtype == "int8":
            if self.latent or alias_v_to_k:
                raise ValueError("the 8-bit cache holds separate K and V pages of attention heads, not a latent or aliased cache")
            self.k = [Q8Pages(num_pages, page_size, heads[i], dims[i], device) for i in range(num_layers)]
            self.v = [Q8Pages(num_pages, page_size, heads[i], dims[i], device) for i in range(num_layers)]
        elif self.latent:
            self.k = [torch.zeros(num_pages, page_size, latent_dim, dtype=dtype, device=device) for _ in range(num_layers)]
            self.v = self.k
        else:
            self.k = [torch.zeros(num_pages, page_size, heads[i], dims[i], dtype=dtype, device=device) for i in range(num_layers)]
            self.v = self.k if alias_v_to_k else [torch.zeros_like(t) for t in self.k]

    def bytes(self) -> int:
        if self.kv_dtype == "int8":
            return sum(t.nbytes() for t in self.k) + sum(t.nbytes() for t in self.v)
        n = sum(t.numel() * t.element_size() for t in self.k)
        return n if (self.latent or self.v is self.k) else 2 * n
