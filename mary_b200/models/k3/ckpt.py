"""Streaming reader for a K3-class checkpoint: ``model.safetensors.index.json`` + N safetensors shards (96 shards and 1.5 TB for
the released model) (src/models/k3/ckpt.rs).

Nothing here holds a model.  Every accessor reads exactly one tensor's byte range with ``pread`` and returns it; shard HEADERS are
cached (they are small and there are few), tensor bytes never are.  A caller that wants one layer asks for one layer and drops it.

Two properties make a wrong load loud instead of plausible:

* both directions of the index are checked: the index names a shard for a tensor, and that shard's own header must name the tensor
  back, so a stale index is an error and not a different weight;
* dtypes are asserted, never coerced: :meth:`bf16` refuses an F32 tensor and the reverse.  The checkpoint mixes them on purpose
  (``A_log``, ``dt_bias``, the three ``*_conv1d.weight`` and ``o_norm.weight`` are F32 among BF16 neighbours).

On top of the raw accessors: MXFP4 expert planes decoded to f32 or relabelled exactly to NVFP4 for the tcgen05 block-scaled GEMM,
per-layer parameter dictionaries in the shape :mod:`mary_b200.models.k3.ops` takes, and :meth:`headers` for the layout gate."""
from __future__ import annotations

import json
import os
import struct

import numpy as np
import torch

from ...nn.fp4 import decode_mxfp4, transcode_mxfp4_to_nvfp4
from . import layout


class CheckpointError(ValueError):
    pass


class K3Checkpoint:
    def __init__(self, directory: str):
        self.dir = str(directory)
        with open(os.path.join(self.dir, "model.safetensors.index.json")) as f:
            self.weight_map: dict = json.load(f)["weight_map"]
        self._headers: dict = {}                       # shard -> (entries, data base offset)
        self._fds: dict = {}
        cfg = os.path.join(self.dir, "config.json")
        self.dims = None
        if os.path.exists(cfg):
            with open(cfg) as f:
                self.dims = layout.K3Dims.from_json(json.load(f))

    def __len__(self) -> int:
        return len(self.weight_map)

    def has(self, name: str) -> bool:
        return name in self.weight_map

    def shards(self) -> list:
        return sorted(set(self.weight_map.values()))

    def close(self) -> None:
        for fd in self._fds.values():
            os.close(fd)
        self._fds.clear()

    # ---- headers ------------------------------------------------------------------------------------------------------------------

    def _shard(self, shard: str):
        if shard not in self._headers:
            fd = os.open(os.path.join(self.dir, shard), os.O_RDONLY)
            (n,) = struct.unpack("<Q", os.pread(fd, 8, 0))
            entries = json.loads(os.pread(fd, n, 8).decode("utf-8"))
            entries.pop("__metadata__", None)
            self._fds[shard] = fd
            self._headers[shard] = (entries, 8 + n)
        return self._headers[shard]

    def headers(self) -> dict:
        """``{name: (dtype, shape)}`` over every shard's OWN header (what the layout gate compares against), after checking that the
        index and the headers name the same tensors in the same shards."""
        out = {}
        for shard in self.shards():
            entries, _ = self._shard(shard)
            for name, e in entries.items():
                if self.weight_map.get(name) != shard:
                    raise CheckpointError(f"{name} is in {shard}'s header but the index says {self.weight_map.get(name)}")
                out[name] = (e["dtype"], tuple(e["shape"]))
        missing = set(self.weight_map) - set(out)
        if missing:
            raise CheckpointError(f"{len(missing)} indexed tensors are in no shard header, e.g. {sorted(missing)[:3]}")
        return out

    # ---- raw tensors --------------------------------------------------------------------------------------------------------------

    def raw(self, name: str):
        """``(dtype string, shape, bytes)`` of one tensor: one ``pread`` of exactly its byte range."""
        shard = self.weight_map.get(name)
        if shard is None:
            raise CheckpointError(f"{name} is not in model.safetensors.index.json")
        entries, base = self._shard(shard)
        e = entries.get(name)
        if e is None:
            raise CheckpointError(f"{name} is absent from {shard}'s own header")
        a, b = e["data_offsets"]
        if b <= a:
            raise CheckpointError(f"{name}: empty tensor in {shard}")
        buf = os.pread(self._fds[shard], b - a, base + a)
        if len(buf) != b - a:
            raise CheckpointError(f"{name}: short read in {shard} ({len(buf)} of {b - a} bytes)")
        return e["dtype"], tuple(e["shape"]), buf

    def _typed(self, name: str, want: str, np_dtype):
        dt, shape, buf = self.raw(name)
        if dt != want:
            raise CheckpointError(f"{name} is {dt}, expected {want}")
        return np.frombuffer(buf, dtype=np_dtype).reshape(shape)

    def bf16(self, name: str) -> torch.Tensor:
        """A BF16 tensor as ``torch.bfloat16`` (the bits, unchanged)."""
        a = self._typed(name, "BF16", np.uint16)
        return torch.from_numpy(a.copy()).view(torch.bfloat16)

    def f32(self, name: str) -> torch.Tensor:
        return torch.from_numpy(self._typed(name, "F32", np.float32).copy())

    def u8(self, name: str) -> np.ndarray:
        return self._typed(name, "U8", np.uint8)

    def slot(self, slot: tuple):
        """Read by slot, checking the stored shape and dtype against the layout's description."""
        if self.dims is None:
            raise CheckpointError("no config.json beside the index: slots cannot be described")
        spec = layout.describe(self.dims, slot)
        if spec is None:
            raise CheckpointError(f"slot {slot} does not exist under this config")
        name = layout.tensor_name(slot)
        dt, shape, _ = self.raw_info(name)
        if (tuple(shape), dt) != (tuple(spec[0]), spec[1]):
            raise CheckpointError(f"{name}: stored {dt}{list(shape)}, layout says {spec[1]}{list(spec[0])}")
        return {"BF16": self.bf16, "F32": self.f32, "U8": self.u8}[dt](name)

    def raw_info(self, name: str):
        shard = self.weight_map.get(name)
        if shard is None:
            raise CheckpointError(f"{name} is not in model.safetensors.index.json")
        e = self._shard(shard)[0].get(name)
        if e is None:
            raise CheckpointError(f"{name} is absent from {shard}'s own header")
        return e["dtype"], tuple(e["shape"]), e["data_offsets"]

    # ---- MXFP4 experts ------------------------------------------------------------------------------------------------------------

    def mxfp4_parts(self, prefix: str):
        """``(codes[rows, cols/2] u8, exponents[rows, cols/32] u8)`` with the two shapes checked against each other."""
        codes = self.u8(prefix + ".weight_packed")
        scale = self.u8(prefix + ".weight_scale")
        if codes.ndim != 2 or scale.shape != (codes.shape[0], codes.shape[1] * 2 // layout.MXFP4_BLOCK):
            raise CheckpointError(f"{prefix}: packed {codes.shape} and scale {scale.shape} do not describe one matrix")
        return codes, scale

    def mxfp4_plane(self, prefix: str) -> torch.Tensor:
        """One expert matrix decoded to f32 ``[rows, cols]`` (low nibble first, one E8M0 exponent per 32 inputs)."""
        codes, scale = self.mxfp4_parts(prefix)
        return torch.from_numpy(decode_mxfp4(codes, scale))

    def _expert_prefix(self, layer: int, expert: int) -> str:
        return f"language_model.model.layers.{layer}.block_sparse_moe.experts.{expert}"

    def expert(self, layer: int, expert: int) -> dict:
        """``{"w1": gate[F, L], "w3": up[F, L], "w2": down[L, F]}`` in f32 for one routed expert."""
        p = self._expert_prefix(layer, expert)
        return {m: self.mxfp4_plane(f"{p}.{m}") for m in ("w1", "w3", "w2")}

    def expert_nvfp4(self, layer: int, expert: int) -> dict:
        """The same expert relabelled EXACTLY to NVFP4 (codes unchanged, E8M0 block exponents rewritten as E4M3 powers of two under
        one f32 global scale per matrix): ``{mat: (codes, e4m3 scales [rows, cols/16], scale2)}``, the operand form of the tcgen05
        block-scaled grouped GEMM.  A matrix whose exponent span does not fit E4M3 raises ``SpanError``."""
        p = self._expert_prefix(layer, expert)
        return {m: transcode_mxfp4_to_nvfp4(*self.mxfp4_parts(f"{p}.{m}")) for m in ("w1", "w3", "w2")}

    # ---- per-layer parameter dictionaries ----------------------------------------------------------------------------------------

    def _L(self, layer: int) -> str:
        return f"language_model.model.layers.{layer}"

    def layer_norms(self, layer: int) -> dict:
        L = self._L(layer)
        return {"input_layernorm": self.bf16(f"{L}.input_layernorm.weight"),
                "post_attention_layernorm": self.bf16(f"{L}.post_attention_layernorm.weight"),
                "attn_res_norm1": self.bf16(f"{L}.self_attention_res_norm.weight"),
                "attn_res_q1": self.bf16(f"{L}.self_attention_res_proj.weight")[0],
                "attn_res_norm2": self.bf16(f"{L}.mlp_res_norm.weight"),
                "attn_res_q2": self.bf16(f"{L}.mlp_res_proj.weight")[0]}

    def kda_weights(self, layer: int) -> dict:
        """The KDA sublayer's parameters.  ``A_log`` ships ``[head_dim]`` with only the first ``num_heads`` entries live; the padding
        is DROPPED here (a zero there would mean decay rate 1, no decay).  The depthwise taps lose their singleton axis."""
        S = self._L(layer) + ".self_attn"
        nh = self.dims.linear.num_heads if self.dims is not None else None
        a_log = self.f32(f"{S}.A_log")
        if nh is not None:
            if bool((a_log[nh:] != 0).any()):
                raise CheckpointError(f"{S}.A_log: entries past the {nh} heads are not zero padding")
            a_log = a_log[:nh]
        p = {k: self.bf16(f"{S}.{k}.weight") for k in ("q_proj", "k_proj", "v_proj", "f_a_proj", "f_b_proj", "b_proj", "g_proj",
                                                        "o_proj")}
        for k in ("q", "k", "v"):
            p[k + "_conv"] = self.f32(f"{S}.{k}_conv1d.weight")[:, 0, :]
        p["A_log"], p["dt_bias"], p["o_norm"] = a_log, self.f32(f"{S}.dt_bias"), self.f32(f"{S}.o_norm.weight")
        return p

    def mla_weights(self, layer: int) -> dict:
        S = self._L(layer) + ".self_attn"
        return {k: self.bf16(f"{S}.{k}.weight") for k in ("q_a_proj", "q_a_layernorm", "q_b_proj", "kv_a_proj_with_mqa",
                                                          "kv_a_layernorm", "kv_b_proj", "g_proj", "o_proj")}

    def mlp_weights(self, prefix: str) -> dict:
        return {k: self.bf16(f"{prefix}.{k}.weight") for k in ("gate_proj", "up_proj", "down_proj")}

    def moe_block_weights(self, layer: int) -> dict:
        """Everything of a sparse block EXCEPT the routed experts (those stream one at a time through :meth:`expert`)."""
        M = self._L(layer) + ".block_sparse_moe"
        p = {"gate": self.bf16(f"{M}.gate.weight"), "gate_bias": self.f32(f"{M}.gate.e_score_correction_bias"),
             "down_in": self.bf16(f"{M}.routed_expert_down_proj.weight"), "up_out": self.bf16(f"{M}.routed_expert_up_proj.weight")}
        if self.has(f"{M}.routed_expert_norm.weight"):
            p["latent_norm"] = self.bf16(f"{M}.routed_expert_norm.weight")
        if self.has(f"{M}.shared_experts.gate_proj.weight"):
            p["shared"] = self.mlp_weights(f"{M}.shared_experts")
        return p

    def gate(self) -> dict:
        """The layout gate on this checkpoint: see :func:`mary_b200.models.k3.layout.check_headers`."""
        if self.dims is None:
            raise CheckpointError("no config.json beside the index")
        return layout.check_headers(self.dims, self.headers())


# ---- expert address book (src/bin/k3_expert_index.rs) --------------------------------------------------------------------------

_EXPERT_MEMBERS = tuple(f"{m}.weight_{h}" for m in ("w1", "w2", "w3") for h in ("packed", "scale"))


def expert_index(ck: K3Checkpoint) -> dict:
    """Where every routed expert's bytes live: ``{(layer, expert): (shard, absolute file offset, length, contiguous)}`` through the
    real name -> shard -> offset path, plus the gate's findings.  Streaming is the only way a model of this size runs on one
    host, and a loader wants ONE read per expert, so three properties are checked instead of assumed: the count is
    ``sparse layers x experts``; every expert totals the byte count the layout predicts; the six members of an expert
    (w1 / w2 / w3 x codes + exponents) sit back to back in one shard.  Offsets in a shard's header are relative to the END of
    the header; the ones returned here are absolute."""
    d = ck.dims
    if d is None:
        raise CheckpointError("no config.json beside the index")
    lat, f = d.moe_hidden_size, d.moe_intermediate_size
    want_bytes = 3 * (lat * f // 2 + lat * f // layout.MXFP4_BLOCK)
    book, wrong_size, split = {}, [], []
    sparse = [i for i in range(d.num_hidden_layers) if d.is_moe_layer(i)]
    for i in sparse:
        for e in range(d.num_experts):
            pre = ck._expert_prefix(i, e)
            spans, shards = [], set()
            for m in _EXPERT_MEMBERS:
                name = f"{pre}.{m}"
                if not ck.has(name):
                    break
                shard = ck.weight_map[name]
                _, base = ck._shard(shard)
                a, b = ck.raw_info(name)[2]
                spans.append((base + a, base + b))
                shards.add(shard)
            if len(spans) != len(_EXPERT_MEMBERS):
                continue
            spans.sort()
            total = sum(b - a for a, b in spans)
            contiguous = len(shards) == 1 and all(spans[j][1] == spans[j + 1][0] for j in range(len(spans) - 1))
            book[(i, e)] = (next(iter(shards)) if len(shards) == 1 else None, spans[0][0], total, contiguous)
            if total != want_bytes:
                wrong_size.append((i, e, total))
            if not contiguous:
                split.append((i, e))
    resident: dict = {}
    for name, shard in ck.weight_map.items():
        if ".experts." in name:
            continue
        a, b = ck.raw_info(name)[2]
        slot = layout.parse(name)
        group = "unmapped" if slot is None else slot[0] if slot[0] != "layer" else "layer." + ".".join(str(x) for x in slot[2:4] if isinstance(x, str))
        resident[group] = resident.get(group, 0) + (b - a)
    return {"book": book, "expected": len(sparse) * d.num_experts, "expert_bytes": want_bytes, "wrong_size": wrong_size, "split": split,
            "resident": resident, "ok": len(book) == len(sparse) * d.num_experts and not wrong_size and not split}


def read_expert_bytes(ck: K3Checkpoint, entry) -> bytes:
    """One ``pread`` covering a whole contiguous expert (an entry of :func:`expert_index`'s book)."""
    shard, off, n, contiguous = entry
    if not contiguous:
        raise CheckpointError("expert is split or interleaved: a single read cannot cover it")
    ck._shard(shard)
    buf = os.pread(ck._fds[shard], n, off)
    if len(buf) != n:
        raise CheckpointError(f"short read in {shard}")
    return buf


def fetch_sweep(ck: K3Checkpoint, book: dict, levels=(1, 4, 16), per_level: int = 32) -> list:
    """Expert fetch bandwidth through the address book at several concurrency levels: ``[(threads, experts, seconds, GB/s)]``.
    Each level reads experts no earlier level touched (the page cache is not bypassed: this is the path a loader sees)."""
    import time
    from concurrent.futures import ThreadPoolExecutor
    keys = [k for k in sorted(book) if book[k][3]]
    out, pos = [], 0
    for n in levels:
        batch = keys[pos:pos + per_level]
        pos += len(batch)
        if not batch:
            break
        t0 = time.perf_counter()
        with ThreadPoolExecutor(max_workers=n) as pool:
            got = sum(pool.map(lambda k: len(read_expert_bytes(ck, book[k])), batch))
        dt = time.perf_counter() - t0
        out.append((n, len(batch), dt, got / dt / 1e9))
    return out
