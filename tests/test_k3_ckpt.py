"""K3 checkpoint layout (names <-> slots, written twice) and the streaming sharded reader, on a synthetic checkpoint."""
import json
import os

import numpy as np
import pytest
import torch

from mary_b200.format.safetensors import save_file
from mary_b200.models.k3 import layout
from mary_b200.models.k3.ckpt import CheckpointError, K3Checkpoint
from mary_b200.nn.fp4 import quantize_mxfp4, decode_mxfp4, decode_nvfp4

CFG = {"text_config": {"hidden_size": 64, "intermediate_size": 96, "num_hidden_layers": 4, "num_attention_heads": 4,
                       "num_key_value_heads": 4, "vocab_size": 50, "first_k_dense_replace": 1, "moe_layer_freq": 1, "num_experts": 4,
                       "num_shared_experts": 1, "moe_intermediate_size": 64, "routed_expert_hidden_size": 32,
                       "latent_moe_use_norm": True, "q_lora_rank": 24, "kv_lora_rank": 16, "qk_nope_head_dim": 8,
                       "qk_rope_head_dim": 4, "v_head_dim": 8,
                       "linear_attn_config": {"kda_layers": [1, 2, 3], "full_attn_layers": [4], "head_dim": 8, "num_heads": 4,
                                              "short_conv_kernel_size": 4}},
       "vision_config": {"patch_size": 2, "vt_hidden_size": 16, "vt_intermediate_size": 32, "vt_num_hidden_layers": 2,
                         "qkv_hidden_size": 16, "mm_hidden_size": 16, "text_hidden_size": 64, "init_pos_emb_height": 4,
                         "init_pos_emb_width": 4, "merge_kernel_size": [2, 2]}}


def _dims():
    return layout.K3Dims.from_json(CFG)


def test_partition_check_names_a_zero_based_reading():
    bad = json.loads(json.dumps(CFG))
    bad["text_config"]["linear_attn_config"].update(kda_layers=[0, 1, 2], full_attn_layers=[3])
    with pytest.raises(ValueError, match=r"missing \[4\].*out of range \[0\]"):
        layout.K3Dims.from_json(bad)


def test_two_directions_agree_on_every_slot():
    d = _dims()
    seen = set()
    n = 0
    for slot, name, shape, dtype in layout.slots(d):
        assert layout.parse(name) == slot, name
        assert name not in seen
        seen.add(name)
        n += 1
    # 3 sparse layers x 4 experts x 3 matrices x 2 halves
    assert sum(1 for s in seen if ".experts." in s) == 3 * 4 * 3 * 2
    assert "language_model.model.layers.0.mlp.gate_proj.weight" in seen                 # the dense layer
    assert "language_model.model.layers.3.self_attn.kv_a_proj_with_mqa.weight" in seen   # one-based list: layer 4 is index 3
    assert "language_model.model.layers.2.self_attn.A_log" in seen
    assert "language_model.model.layers.3.self_attn.A_log" not in seen
    assert n == len(seen)


def test_parse_is_strict_and_describe_decides_legality():
    d = _dims()
    assert layout.parse("language_model.model.layers.1.self_attn.A_log.weight") is None
    assert layout.parse("language_model.model.layers.1.self_attn.q_proj") is None
    assert layout.parse("language_model.model.layers.01.input_layernorm.weight") is None
    assert layout.parse("language_model.model.layers.1.block_sparse_moe.experts.0.w4.weight_packed") is None
    assert layout.parse("language_model.model.layers.1.mlp.gate_proj.bias") is None
    mla_on_kda = layout.parse("language_model.model.layers.0.self_attn.q_a_proj.weight")
    assert mla_on_kda == ("layer", 0, "attn", "q_a_proj") and layout.describe(d, mla_on_kda) is None
    assert layout.describe(d, ("layer", 9, "input_ln")) is None
    assert layout.describe(d, ("layer", 1, "mlp", "gate_proj")) is None                  # dense MLP on a sparse layer
    assert layout.describe(d, ("layer", 1, "moe", "expert", 4, "w1", "packed")) is None
    assert layout.describe(d, ("layer", 1, "moe", "expert", 0, "w2", "scale")) == ((32, 2), "U8")
    assert layout.describe(d, ("layer", 1, "moe", "expert", 0, "w1", "packed")) == ((64, 16), "U8")
    assert layout.describe(d, ("layer", 0, "attn", "A_log")) == ((8,), "F32")
    assert layout.describe(d, ("layer", 0, "attn", "q_conv1d")) == ((32, 1, 4), "F32")
    assert layout.describe(d, ("mm", "proj0")) == ((64, 64), "BF16")


def _write_checkpoint(tmp, n_shards=3, seed=0):
    d = _dims()
    rng = np.random.default_rng(seed)
    shards = [dict() for _ in range(n_shards)]
    bf = [set() for _ in range(n_shards)]
    truth, wm = {}, {}
    for k, (slot, name, shape, dtype) in enumerate(layout.slots(d)):
        s = k % n_shards
        if dtype == "U8":
            continue                                      # experts are written as code/scale pairs below
        if dtype == "BF16":
            a = torch.from_numpy(rng.standard_normal(shape).astype(np.float32)).to(torch.bfloat16)
            truth[name] = a
            shards[s][name] = a.view(torch.int16).numpy().view(np.uint16)
            bf[s].add(name)
        else:
            a = rng.standard_normal(shape).astype(np.float32)
            if name.endswith("A_log"):
                a[d.linear.num_heads:] = 0.0
            truth[name] = torch.from_numpy(a)
            shards[s][name] = a
        wm[name] = f"model-{s + 1:05d}-of-{n_shards:05d}.safetensors"
    for i in range(d.num_hidden_layers):
        if not d.is_moe_layer(i):
            continue
        for e in range(d.num_experts):
            for mat in ("w1", "w2", "w3"):
                out, inp = (32, 64) if mat == "w2" else (64, 32)
                codes, sc = quantize_mxfp4(rng.standard_normal((out, inp)).astype(np.float32) * 0.1)
                pre = f"language_model.model.layers.{i}.block_sparse_moe.experts.{e}.{mat}"
                s = (i + e) % n_shards
                shards[s][pre + ".weight_packed"], shards[s][pre + ".weight_scale"] = codes, sc
                truth[pre] = torch.from_numpy(decode_mxfp4(codes, sc))
                wm[pre + ".weight_packed"] = wm[pre + ".weight_scale"] = f"model-{s + 1:05d}-of-{n_shards:05d}.safetensors"
    for s in range(n_shards):
        save_file(shards[s], os.path.join(tmp, f"model-{s + 1:05d}-of-{n_shards:05d}.safetensors"), bf16=bf[s])
    with open(os.path.join(tmp, "model.safetensors.index.json"), "w") as f:
        json.dump({"metadata": {}, "weight_map": wm}, f)
    with open(os.path.join(tmp, "config.json"), "w") as f:
        json.dump(CFG, f)
    return truth


def test_reader_gate_dtypes_and_experts(tmp_path):
    truth = _write_checkpoint(str(tmp_path))
    ck = K3Checkpoint(str(tmp_path))
    assert len(ck) == len(ck.headers())
    g = ck.gate()
    assert g == {"unfilled": [], "unmapped": [], "mismatched": [], "not_inverse": []}
    name = "language_model.model.layers.0.self_attn.q_proj.weight"
    assert torch.equal(ck.bf16(name), truth[name])
    assert torch.equal(ck.slot(("layer", 0, "attn", "q_proj")), truth[name])
    with pytest.raises(CheckpointError, match="is BF16, expected F32"):
        ck.f32(name)
    with pytest.raises(CheckpointError, match="is F32, expected BF16"):
        ck.bf16("language_model.model.layers.0.self_attn.A_log")
    with pytest.raises(CheckpointError, match="not in model.safetensors.index.json"):
        ck.raw("language_model.model.layers.0.self_attn.nope.weight")
    ex = ck.expert(2, 3)
    pre = "language_model.model.layers.2.block_sparse_moe.experts.3."
    for m in ("w1", "w2", "w3"):
        assert torch.equal(ex[m], truth[pre + m])
    nv = ck.expert_nvfp4(2, 3)
    for m in ("w1", "w2", "w3"):
        codes, s8, s2 = nv[m]
        assert np.array_equal(decode_nvfp4(codes, s8, s2), truth[pre + m].numpy())         # an exact relabel
    kda = ck.kda_weights(1)
    assert kda["A_log"].shape == (4,) and kda["q_conv"].shape == (32, 4) and kda["g_proj"].shape == (32, 64)
    mla = ck.mla_weights(3)
    assert mla["q_b_proj"].shape == (4 * 12, 24) and mla["kv_b_proj"].shape == (4 * 16, 16)
    moe = ck.moe_block_weights(1)
    assert moe["gate_bias"].dtype == torch.float32 and moe["latent_norm"].shape == (32,) and moe["shared"]["down_proj"].shape == (64, 64)
    norms = ck.layer_norms(2)
    assert norms["attn_res_q1"].shape == (64,)
    ck.close()


def test_stale_index_and_layout_findings_are_loud(tmp_path):
    _write_checkpoint(str(tmp_path))
    idx = os.path.join(str(tmp_path), "model.safetensors.index.json")
    wm = json.load(open(idx))["weight_map"]
    name = "language_model.model.layers.1.input_layernorm.weight"
    other = next(s for s in sorted(set(wm.values())) if s != wm[name])
    wm2 = dict(wm)
    wm2[name] = other
    json.dump({"weight_map": wm2}, open(idx, "w"))
    ck = K3Checkpoint(str(tmp_path))
    with pytest.raises(CheckpointError, match="absent from .* own header"):
        ck.raw(name)
    with pytest.raises(CheckpointError, match="header but the index says"):
        ck.headers()
    ck.close()
    # a checkpoint with one tensor missing and one stray: both are named
    wm3 = {k: v for k, v in wm.items() if k != name}
    json.dump({"weight_map": wm3}, open(idx, "w"))
    d = _dims()
    heads = {n: (dt, sh) for _, n, sh, dt in layout.slots(d) if n != name}
    heads["language_model.model.layers.1.input_layernorm.bias"] = ("BF16", (64,))
    heads["language_model.model.layers.0.self_attn.dt_bias"] = ("BF16", (32,))
    g = layout.check_headers(d, heads)
    assert g["unfilled"] == [name] and g["unmapped"] == ["language_model.model.layers.1.input_layernorm.bias"]
    assert g["mismatched"][0][0] == "language_model.model.layers.0.self_attn.dt_bias" and not g["not_inverse"]


def test_a_log_padding_must_be_zero(tmp_path):
    _write_checkpoint(str(tmp_path))
    ck = K3Checkpoint(str(tmp_path))
    ck.dims.linear.num_heads = 3                       # pretend fewer heads: entry 3 is live, not padding
    with pytest.raises(CheckpointError, match="not zero padding"):
        ck.kda_weights(0)
    ck.close()


def test_kda_runs_on_checkpoint_weights(tmp_path):
    from mary_b200.models.k3.ops import K3Config, kda_attention
    _write_checkpoint(str(tmp_path))
    ck = K3Checkpoint(str(tmp_path))
    p = {k: (v.float() if v.dtype == torch.bfloat16 else v) for k, v in ck.kda_weights(0).items()}
    cfg = K3Config(4, [1, 2, 3], [4], n_heads=4, kda_head_dim=8)
    x = torch.randn(6, 64) * 0.5
    full = kda_attention(x, p, cfg)
    cache = {}
    steps = torch.cat([kda_attention(x[t:t + 1], p, cfg, cache) for t in range(6)])
    assert full.shape == (6, 64) and torch.isfinite(full).all()
    assert torch.allclose(full, steps, atol=1e-4, rtol=1e-4)
    ck.close()


def test_cli_gate(tmp_path, capsys):
    from mary_b200.cli.mary import main
    _write_checkpoint(str(tmp_path))
    assert main(["k3-gate", str(tmp_path)]) == 0
    assert "unfilled 0, unmapped 0, mismatched 0, not_inverse 0" in capsys.readouterr().out


def test_expert_address_book_gate_single_reads_and_cli(tmp_path, capsys):
    from mary_b200.cli.mary import main
    from mary_b200.models.k3.ckpt import expert_index, fetch_sweep, read_expert_bytes
    truth = _write_checkpoint(str(tmp_path))
    ck = K3Checkpoint(str(tmp_path))
    ix = expert_index(ck)
    assert ix["ok"] and len(ix["book"]) == ix["expected"] == 3 * 4
    assert ix["expert_bytes"] == 3 * (32 * 64 // 2 + 32 * 64 // 32)
    # one read covers the expert; its bytes are the six members in name order
    entry = ix["book"][(2, 1)]
    blob = read_expert_bytes(ck, entry)
    pre = "language_model.model.layers.2.block_sparse_moe.experts.1."
    want = b"".join(bytes(ck.raw(pre + m)[2]) for m in ("w1.weight_packed", "w1.weight_scale", "w2.weight_packed", "w2.weight_scale",
                                                        "w3.weight_packed", "w3.weight_scale"))
    assert blob == want
    assert sum(ix["resident"].values()) == sum(ck.raw_info(n)[2][1] - ck.raw_info(n)[2][0] for n in ck.weight_map if ".experts." not in n)
    sweep = fetch_sweep(ck, ix["book"], levels=(1, 2), per_level=4)
    assert [(n, c) for n, c, _, _ in sweep] == [(1, 4), (2, 4)] and all(g > 0 for *_, g in sweep)
    ck.close()
    assert main(["k3-experts", str(tmp_path), "--sweep", "1,2", "--per-level", "3"]) == 0
    assert "GATE PASS" in capsys.readouterr().out
    # an index that lost one member of one expert fails the gate and prints no bandwidth
    idx = os.path.join(str(tmp_path), "model.safetensors.index.json")
    wm = json.load(open(idx))["weight_map"]
    del wm[pre + "w2.weight_scale"]
    json.dump({"weight_map": wm}, open(idx, "w"))
    assert main(["k3-experts", str(tmp_path)]) == 1
    out = capsys.readouterr().out
    assert "GATE FAIL" in out and "readers" not in out


def test_encode_writes_little_endian_i64_and_prints_the_round_trip(tmp_path, capsys, monkeypatch):
    import io
    import sys
    tokenizers = pytest.importorskip("tokenizers")
    from tokenizers import Tokenizer, models, pre_tokenizers, decoders
    from mary_b200.cli.mary import main
    vocab = {"[UNK]": 0, "ĠThe": 1, "Ġcapital": 2, "Ġof": 3, "ĠFrance": 4, "Ġis": 5}
    tok = Tokenizer(models.WordLevel(vocab, unk_token="[UNK]"))
    tok.pre_tokenizer = pre_tokenizers.ByteLevel(add_prefix_space=False, use_regex=True)
    tok.decoder = decoders.ByteLevel()
    tok.save(str(tmp_path / "tokenizer.json"))

    class In:
        buffer = io.BytesIO(" The capital of France is".encode())
    monkeypatch.setattr(sys, "stdin", In)
    assert main(["encode", str(tmp_path / "p.ids"), "--tokenizer-json", str(tmp_path / "tokenizer.json")]) == 0
    ids = np.fromfile(tmp_path / "p.ids", dtype="<i8")
    assert ids.tolist() == [1, 2, 3, 4, 5]
    assert "decode: ' The capital of France is'" in capsys.readouterr().out


def test_fit_reports_resident_slabs_per_gpu_count(capsys):
    from mary_b200.cli.mary import main
    assert main(["fit", "--model", "k3", "--gpus", "1,8"]) == 0
    out = capsys.readouterr().out.splitlines()
    assert "fits only with" in out[0] and "of 61 expert slabs" in out[0] and "8 GPU(s): fits, all 61 expert slabs resident" in out[1]
    assert main(["fit", "--model", "k3", "--gpus", "1", "--capacity-gib", "20"]) == 1
