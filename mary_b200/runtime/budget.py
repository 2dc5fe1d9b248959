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


# ---------------------------------------------------------------------------------------------------------------------
# Prefill: what a chunk of `tokens` rows holds while the stack runs (src/models/inkling/budget.rs:523-590).  Three shapes:
# what every layer reads and none frees (the residual stream and its normed copy), what each layer KEEPS (its cache rows,
# already billed by the paged cache here, so only the rows of this chunk that are not yet paged count), and what ONE layer
# holds while it runs — layers run one after the other and free their working set, so the widest layer binds, not the sum.
def attention_activation_bytes(cfg, tokens: int, world: int = 1) -> int:
    heads = max(cfg.num_attention_heads // world, 1)
    if cfg.attention == "mla":
        # q_a/kv_a row, q_b rows, absorbed queries (576 wide), latent outputs (512 wide), un-absorbed outputs; the expanded
        # prefill path additionally holds K (192) and V (128) of the visible context per head
        per = (cfg.q_lora_rank + 576) + heads * (192 + 576 + 512 + 128) + heads * (192 + 128)
    else:
        kv = max(cfg.num_key_value_heads // world, 1)
        per = (heads + 2 * kv) * cfg.head_dim + 2 * heads * cfg.head_dim
    return tokens * per * 2


def mlp_activation_bytes(cfg, layer: int, tokens: int, world: int = 1) -> int:
    H = cfg.hidden_size
    if cfg.is_dense(layer):
        return tokens * (2 * cfg.dense_intermediate_size // world + cfg.dense_intermediate_size // world + H) * 2
    k1 = cfg.num_experts_per_tok + cfg.n_shared_experts
    rows = padded_routed_rows(cfg, tokens, world)
    F = cfg.moe_intermediate_size
    # NVFP4 codes + scales of the gathered rows and of the intermediate, the bf16 expert outputs, the router logits
    return int(rows * (H * (0.5 + 1 / 16) + F * (0.5 + 1 / 16) + H * 2)) + tokens * (cfg.n_routed_experts * 4 + k1 * 12)


def padded_routed_rows(cfg, tokens: int, world: int = 1, tile: int = 128) -> int:
    """Upper bound of the padded rows one rank's grouped GEMM sees: every entry plus one ragged tile per local expert."""
    entries = tokens * (cfg.num_experts_per_tok + cfg.n_shared_experts)
    e_local = cfg.n_routed_experts // world + cfg.n_shared_experts
    return entries + min(entries, e_local) * (tile - 1)


def prefill_activation_bytes(cfg, tokens: int, world: int = 1, layers: range | None = None) -> int:
    layers = range(cfg.num_hidden_layers) if layers is None else layers
    carried = 2 * tokens * cfg.hidden_size * 2
    widest = max((max(attention_activation_bytes(cfg, tokens, world), mlp_activation_bytes(cfg, l, tokens, world)) for l in layers), default=0)
    head = tokens * 8                                   # the arg-max head keeps (value, index) per row, never the logits
    return carried + widest + head


def largest_buffer(cfg, tokens: int, world: int = 1) -> int:
    """The largest SINGLE allocation of a prefill chunk (a maximum, never a sum: budget.rs:593-660)."""
    H, F = cfg.hidden_size, cfg.moe_intermediate_size
    rows = padded_routed_rows(cfg, tokens, world)
    cands = [tokens * H * 2, rows * H * 2, rows * H // 2, rows * F * 2, tokens * cfg.n_routed_experts * 4]
    if cfg.attention == "mla":
        cands.append(tokens * max(cfg.num_attention_heads // world, 1) * 576 * 2)
    if cfg.first_k_dense:
        cands.append(tokens * 2 * cfg.dense_intermediate_size // world * 2)
    return max(cands)


def longest_sequence(cfg, cap: int, world: int = 1) -> int:
    """The longest prefill chunk whose activations fit under ``cap`` bytes; bisected (every term is non-decreasing in tokens)."""
    lo, hi = 0, 1 << 24
    while lo < hi:
        mid = (lo + hi + 1) // 2
        if prefill_activation_bytes(cfg, mid, world) <= cap:
            lo = mid
        else:
            hi = mid - 1
    return lo


def check_prefill(cfg, tokens: int, free_bytes: int, world: int = 1) -> int:
    """Refuse a prefill chunk this device cannot hold BEFORE the first allocation (budget.rs:677): the allocator's own refusal
    would come half-way through the stack.  Returns the priced bytes."""
    want = prefill_activation_bytes(cfg, tokens, world)
    if want > free_bytes:
        g = 1 << 30
        raise AdmissionError(f"a prefill chunk of {tokens} rows needs {want / g:.2f} GiB of activations (largest single buffer "
                             f"{largest_buffer(cfg, tokens, world) / g:.2f} GiB) and {free_bytes / g:.2f} GiB are free; the longest chunk that "
                             f"fits is {longest_sequence(cfg, free_bytes, world)} rows")
    return want
