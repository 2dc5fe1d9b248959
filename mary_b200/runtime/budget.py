"""Memory admission: price a serving configuration before any allocation and refuse what cannot fit.

Reference: src/models/inkling/budget.rs (per-buffer cap, query blocking against a score budget :226-270, prefill activation
pricing, ``check`` :677) and the copy_share admission gate (src/models/inkling/pile.rs:1192-1650).  Here the quantities are
the weights resident on the rank, the paged KV cache and the activation high-water mark of one step; ``check`` raises
``AdmissionError`` with the full bill instead of letting the allocator fail half-way through start-up."""
from __future__ import annotations

from dataclasses import dataclass


class AdmissionError(RuntimeError):
    pass


@dataclass
class Bill:
    weights: int
    kv_cache: int
    activations: int
    workspace: int
    capacity: int

    @property
    def total(self) -> int:
        return self.weights + self.kv_cache + self.activations + self.workspace

    def lines(self) -> str:
        g = 1 << 30
        return (f"weights {self.weights / g:.2f} GiB + kv cache {self.kv_cache / g:.2f} GiB + activations {self.activations / g:.2f} GiB "
                f"+ workspace {self.workspace / g:.2f} GiB = {self.total / g:.2f} GiB of {self.capacity / g:.2f} GiB")


def kv_bytes(num_layers: int, tokens: int, row_bytes: int) -> int:
    return num_layers * tokens * row_bytes


def moe_bill(cfg, world: int, batch: int, max_len: int, rows_per_step: int, capacity: int, expert_slabs: int | None = None) -> Bill:
    H, F = cfg.hidden_size, cfg.moe_intermediate_size
    n_moe = sum(1 for i in range(cfg.num_hidden_layers) if not cfg.is_dense(i)) + cfg.num_mtp_layers
    slabs = n_moe if expert_slabs is None else min(expert_slabs, n_moe)
    experts = slabs * (cfg.n_routed_experts // world) * 3 * H * F * (0.5 + 1 / 16)
    if cfg.attention == "mla":
        attn = (cfg.q_lora_rank + 576) * H + (cfg.num_attention_heads // world) * (192 * cfg.q_lora_rank + 2 * 128 * 512 + 128 * H)
        row = 576 * 2
    else:
        attn = ((cfg.num_attention_heads + 2 * cfg.num_key_value_heads) // world) * cfg.head_dim * H + (cfg.num_attention_heads // world) * cfg.head_dim * H
        row = 2 * max(cfg.num_key_value_heads // world, 1) * cfg.head_dim * 2
    dense = cfg.first_k_dense * 3 * H * cfg.dense_intermediate_size // world + n_moe * (cfg.n_routed_experts * H + 3 * H * F * cfg.n_shared_experts // world)
    layers = cfg.num_hidden_layers + cfg.num_mtp_layers
    weights = int(experts + 2 * (layers * attn + dense + 2 * cfg.vocab_size * H))
    kv = kv_bytes(layers, batch * max_len, row)
    act = rows_per_step * (H * 2 * 8 + cfg.vocab_size * 4) + rows_per_step * (cfg.num_experts_per_tok + 1) * (H + F) * 3
    return Bill(weights, kv, int(act), 2 << 30, capacity)


def check(bill: Bill, headroom: float = 0.03) -> Bill:
    if bill.total > bill.capacity * (1.0 - headroom):
        raise AdmissionError("configuration does not fit: " + bill.lines())
    return bill


def query_block(n_heads: int, n_keys: int, score_budget_bytes: int = 4 << 30, bytes_per_score: int = 4) -> int:
    """Largest number of query rows whose ``[heads, rows, keys]`` score block stays inside the budget (budget.rs:226-270);
    the flash kernels here never materialise scores, this sizes the PyTorch reference paths."""
    return max(1, score_budget_bytes // max(1, n_heads * n_keys * bytes_per_score))
