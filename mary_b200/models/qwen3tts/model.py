"""Qwen3-TTS frame generator: the talker (a Qwen3-style decoder over summed text + codec embeddings that emits codebook 0
of every 12.5 Hz frame) and the code predictor (a 5-layer decoder that fills in codebooks 1..15 of the frame).

Reference: dimensions src/models/qwen3tts/config.rs:6-62; talker src/models/qwen3tts/talker.rs:28-136; predictor flow
src/models/qwen3tts/predictor.rs:1-22 (fresh cache per frame; prefill ``[proj(h_talker), proj(emb_0(code_0))] -> head_0 ->
code_1``; step ``i``: ``proj(emb_i(code_i)) -> head_i -> code_{i+1}``); logits processing and the frame loop
src/models/qwen3tts/pipeline.rs:190-420.  The reference runs the predictor's 15 sequential single-token steps on the CPU or
through a per-op "megakernel" lane (src/models/qwen3tts/megakernel.rs, predictor_gpu.rs) because op submission dominated;
here both decoders are the package's ordinary paged-cache decoders (``models.mistral`` with q/k norm), every sampling step
is the device Gumbel-max kernel, and nothing is read back per codebook — the host sees one frame of 16 codes at a time."""
from __future__ import annotations

from dataclasses import dataclass, field

import numpy as np
import torch
from torch import nn

from ... import ops
from ...ops import sampling
from ...runtime.batch import BatchMeta
from ...runtime.kv_cache import PagedKVCache
from ..mistral.model import MistralConfig, MistralModel


@dataclass
class Qwen3TTSConfig:
    talker_layers: int = 28
    talker_hidden: int = 2048
    talker_heads: int = 16
    talker_kv_heads: int = 8
    talker_ffn: int = 6144
    head_dim: int = 128
    codec_vocab: int = 3072
    text_vocab: int = 151936
    text_hidden: int = 2048
    pred_layers: int = 5
    pred_hidden: int = 1024
    pred_heads: int = 16
    pred_kv_heads: int = 8
    pred_ffn: int = 3072
    pred_vocab: int = 2048
    num_code_groups: int = 16
    rope_theta: float = 1e6
    eps: float = 1e-6
    codec_pad: int = 2148
    codec_bos: int = 2149
    codec_eos: int = 2150

    @staticmethod
    def tiny():
        return Qwen3TTSConfig(talker_layers=2, talker_hidden=64, talker_heads=4, talker_kv_heads=2, talker_ffn=128, head_dim=16,
                              codec_vocab=96, text_vocab=50, text_hidden=48, pred_layers=2, pred_hidden=32, pred_heads=4, pred_kv_heads=2,
                              pred_ffn=64, pred_vocab=64, num_code_groups=4, codec_pad=70, codec_bos=71, codec_eos=72)

    def talker_cfg(self):
        return MistralConfig(self.talker_layers, self.talker_hidden, self.talker_ffn, self.talker_heads, self.talker_kv_heads,
                             self.head_dim, self.codec_vocab, self.rope_theta, self.eps, 8192, tie_word_embeddings=False, qk_norm=True,
                             name="qwen3tts-talker")

    def pred_cfg(self):
        return MistralConfig(self.pred_layers, self.pred_hidden, self.pred_ffn, self.pred_heads, self.pred_kv_heads, self.head_dim,
                             1, self.rope_theta, self.eps, 64, tie_word_embeddings=True, qk_norm=True, name="qwen3tts-predictor")


@dataclass
class SamplingParams:
    do_sample: bool = True
    top_k: int = 50
    temperature: float = 0.9
    repetition_penalty: float = 1.05
    subtalker_do_sample: bool = True
    subtalker_temperature: float = 0.9
    max_frames: int = 1024
    seed: int = 0


def _P(*shape, dtype, device):
    return nn.Parameter(torch.empty(*shape, dtype=dtype, device=device), requires_grad=False)


class Talker(nn.Module):
    """``stack.embed`` is the codec embedding ``[3072, H]`` (codebook 0 + control tokens), ``stack.lm_head`` the codebook-0 head."""

    def __init__(self, cfg: Qwen3TTSConfig, dtype=torch.float32, device="cpu"):
        super().__init__()
        self.cfg = cfg
        self.stack = MistralModel(cfg.talker_cfg(), dtype=dtype, device=device)
        kw = dict(dtype=dtype, device=device)
        self.text_embedding = _P(cfg.text_vocab, cfg.text_hidden, **kw)
        self.fc1_w, self.fc1_b = _P(cfg.text_hidden, cfg.text_hidden, **kw), _P(cfg.text_hidden, **kw)
        self.fc2_w, self.fc2_b = _P(cfg.talker_hidden, cfg.text_hidden, **kw), _P(cfg.talker_hidden, **kw)

    def embed_text(self, ids):
        """Text ids -> talker-space embeddings: text embedding, then the biased ResizeMLP ``fc2(silu(fc1(e)))``."""
        e = ops.embed(ids, self.text_embedding)
        h = torch.nn.functional.silu(ops.linear(e, self.fc1_w).float() + self.fc1_b.float()).to(e.dtype)
        return (ops.linear(h, self.fc2_w).float() + self.fc2_b.float()).to(e.dtype)

    def embed_codec(self, ids):
        return ops.embed(ids, self.stack.embed)

    def kv_spec(self):
        return self.stack.kv_spec()

    def forward(self, embeds, meta, cache):
        """Normed hidden states of every fed row."""
        return self.stack.hidden_from_embeds(embeds, meta, cache)

    def logits(self, hidden):
        return ops.linear(hidden, self.stack.lm_head).float()


class CodePredictor(nn.Module):
    def __init__(self, cfg: Qwen3TTSConfig, dtype=torch.float32, device="cpu"):
        super().__init__()
        self.cfg = cfg
        self.stack = MistralModel(cfg.pred_cfg(), dtype=dtype, device=device)
        kw = dict(dtype=dtype, device=device)
        n = cfg.num_code_groups - 1
        self.embeddings = nn.ParameterList([_P(cfg.pred_vocab, cfg.talker_hidden, **kw) for _ in range(n)])      # talker width
        self.heads = nn.ParameterList([_P(cfg.pred_vocab, cfg.pred_hidden, **kw) for _ in range(n)])
        self.has_proj = cfg.talker_hidden != cfg.pred_hidden
        if self.has_proj:
            self.proj_w, self.proj_b = _P(cfg.pred_hidden, cfg.talker_hidden, **kw), _P(cfg.pred_hidden, **kw)
        dev = torch.device(device)
        spec = self.stack.kv_spec()
        # one sequence of at most num_code_groups + 1 positions, restarted every frame: one page per layer is enough
        self.pages = (cfg.num_code_groups + 1 + 15) // 16
        self.cache = PagedKVCache(spec["num_layers"], self.pages + 1, 16, spec["kv_heads"], spec["head_dim"], dtype=dtype, device=dev)
        self.cache.alloc.extend(0, self.pages * 16)
        self.table, _ = self.cache.alloc.page_table([0])
        self.dev = dev

    def project(self, x):
        if not self.has_proj:
            return x
        if x.is_cuda and x.shape[0] == 1 and x.dtype == torch.bfloat16 and self.proj_w.shape[1] <= 8192:
            from ...ops import cuda as K                # one token: product and bias in one matrix-vector launch
            return K.step_matvec(x, self.proj_w, res=self.proj_b, mode="residual")
        return (ops.linear(x, self.proj_w).float() + self.proj_b.float()).to(x.dtype)

    def _meta(self, q, kv):
        return BatchMeta.build([q], [kv], self.table, 16, self.dev)

    def predict_frame(self, h_talker, code0_embed, temperature: float = 0.0, seed: int = 0, frame: int = 0):
        """``h_talker [H]``, ``code0_embed [H]`` (the talker's codec embedding row of the sampled codebook-0 id).  Returns
        ``(codes int64 [num_code_groups - 1], embed_sum [H])`` where ``embed_sum`` is the sum of the predictor's talker-width
        embeddings of those codes — the codec side of the talker's next input.

        The 15 steps are strictly sequential and tiny, so on the GPU their cost is launch submission, not math (the reason the
        reference moved this stage to the CPU, src/models/qwen3tts/cpu.rs:1-8, and wrote a persistent chain kernel,
        megakernel.rs:70-722).  Here the whole greedy frame (every decoder layer of every step, the heads, the arg-max and the
        embedding gathers) is captured ONCE as a CUDA graph over static buffers and replayed per frame: positions are the same
        in every frame, so the batch descriptors are built once."""
        if h_talker.is_cuda and temperature <= 0 and self.use_graph:
            if self._graph is None:
                self._capture(h_talker.dtype)
            self._g_in[0].copy_(h_talker), self._g_in[1].copy_(code0_embed)
            self._graph.replay()
            return self._g_codes.clone(), self._g_sum.clone()
        return self._frame(torch.stack([h_talker, code0_embed]), self._metas(), temperature, seed, frame)

    use_graph = True
    _graph = None

    def _metas(self):
        n = self.cfg.num_code_groups - 1
        if getattr(self, "_meta_list", None) is None:
            self._meta_list = [self._meta(2 if i == 0 else 1, i + 2) for i in range(n)]
        return self._meta_list

    def _frame(self, x2, metas, temperature, seed, frame):
        n = self.cfg.num_code_groups - 1
        x = self.project(x2)
        codes, rows = [], []
        for i in range(n):
            hid = self.stack.hidden_from_embeds(x, metas[i], self.cache)[-1:]
            lg = ops.linear(hid, self.heads[i]).float()
            tok = sampling.sample(lg, temperature, seed=seed, step=frame * 64 + i)
            codes.append(tok.reshape(1))
            e = ops.embed(tok.reshape(1).to(torch.int32), self.embeddings[i])
            rows.append(e[0])
            x = self.project(e)
        return torch.cat(codes), torch.stack(rows).float().sum(0)          # one sum over the frame's rows instead of a cast and an add per step

    def _capture(self, dtype):
        metas = self._metas()
        self._g_in = torch.zeros(2, self.cfg.talker_hidden, dtype=dtype, device=self.dev)
        side = torch.cuda.Stream(device=self.dev)
        side.wait_stream(torch.cuda.current_stream(self.dev))
        with torch.cuda.stream(side):                                    # one eager pass first: lazy initialisation stays out of the graph
            self._frame(self._g_in, metas, 0.0, 0, 0)
        torch.cuda.current_stream(self.dev).wait_stream(side)
        g = torch.cuda.CUDAGraph()
        with torch.cuda.graph(g):
            self._g_codes, self._g_sum = self._frame(self._g_in, metas, 0.0, 0, 0)
        self._graph = g

    def accumulate_frame(self, codes):
        """Sum of the talker-width embeddings of codebooks 1.. of one known frame (reference prompts)."""
        out = 0
        for i, c in enumerate(codes):
            out = out + ops.embed(torch.as_tensor([int(c)], dtype=torch.int32, device=self.dev), self.embeddings[i])[0].float()
        return out


def process_talker_logits(logits, generated, step: int, penalty: float, cfg: Qwen3TTSConfig):
    """Repetition penalty over the codebook-0 ids generated so far, no end-of-speech in the first two frames, and the
    control range ``[pred_vocab, codec_vocab)`` suppressed except end-of-speech (src/models/qwen3tts/pipeline.rs:190-210)."""
    lg = logits.clone()
    if len(generated):
        idx = torch.as_tensor(sorted(set(int(g) for g in generated)), device=lg.device)
        v = lg[idx]
        lg[idx] = torch.where(v > 0, v / penalty, v * penalty)
    if step < 2:
        lg[cfg.codec_eos] = float("-inf")
    keep = lg[cfg.codec_eos].clone()
    lg[cfg.pred_vocab:] = float("-inf")
    lg[cfg.codec_eos] = keep
    return lg


def generate_frames(talker: Talker, predictor: CodePredictor, prefill, trailing, tts_pad, params: SamplingParams, on_frame=None):
    """The frame loop: ``prefill [L, H]`` assembled input embeddings, ``trailing [n, H]`` text-side embeddings still to be fed
    (one per generated frame, then ``tts_pad [H]``).  Returns the frames ``[T, num_code_groups]`` (codebook 0 first);
    ``on_frame(codes) -> bool`` is a streaming sink that may stop the loop."""
    cfg = talker.cfg
    dev = prefill.device
    spec = talker.kv_spec()
    max_len = prefill.shape[0] + params.max_frames + 1
    pages = (max_len + 15) // 16
    cache = PagedKVCache(spec["num_layers"], pages + 1, 16, spec["kv_heads"], spec["head_dim"], dtype=prefill.dtype, device=dev)
    cache.alloc.extend(0, pages * 16)
    table, _ = cache.alloc.page_table([0])
    kv = prefill.shape[0]
    with torch.no_grad():
        hidden = talker(prefill, BatchMeta.build([kv], [kv], table, 16, dev), cache)[-1]
        generated, frames = [], []
        for step in range(params.max_frames):
            lg = process_talker_logits(talker.logits(hidden[None])[0], generated, step, params.repetition_penalty, cfg)
            t = params.temperature if params.do_sample else 0.0
            code0 = int(sampling.sample(lg[None], t, top_k=params.top_k if params.do_sample else 0, seed=params.seed, step=step)[0])
            generated.append(code0)
            if code0 == cfg.codec_eos:
                break
            e0 = talker.embed_codec(torch.as_tensor([code0], dtype=torch.int32, device=dev))[0]
            rest, esum = predictor.predict_frame(hidden, e0, params.subtalker_temperature if params.subtalker_do_sample else 0.0,
                                                 params.seed + 1, step)
            frame = [code0] + [int(c) for c in rest]
            frames.append(frame)
            if on_frame is not None and not on_frame(frame):
                frames.pop()
                break
            text_side = trailing[step] if step < trailing.shape[0] else tts_pad
            nxt = (e0.float() + esum + text_side.float()).to(prefill.dtype)
            kv += 1
            hidden = talker(nxt[None], BatchMeta.build([1], [kv], table, 16, dev), cache)[-1]
    return np.asarray(frames, dtype=np.int64).reshape(-1, cfg.num_code_groups)


def init_random_(talker: Talker, predictor: CodePredictor, seed: int = 0, std: float = 0.05):
    g = torch.Generator(device=talker.text_embedding.device).manual_seed(seed)
    for m in (talker, predictor):
        for n, p in m.named_parameters():
            if p.dim() == 1 and not n.endswith("_b"):
                p.data.fill_(1.0)
            else:
                p.data.normal_(0.0, std, generator=g)


def load_into(talker: Talker, predictor: CodePredictor, loader) -> None:
    """Checkpoint names: ``talker.model.*`` (codec/text embeddings, layers, norm), ``talker.text_projection.linear_fc{1,2}``,
    ``talker.codec_head``, ``talker.code_predictor.{model.layers.*, model.norm, model.codec_embedding.N, lm_head.N,
    small_to_mtp_projection}``."""
    dt = talker.stack.dtype

    def put(p, name):
        p.data.copy_(loader.load_tensor(name, dt).to(p.device))

    def stack(m, prefix):
        c = m.cfg
        for i, L in enumerate(m.layers):
            p = f"{prefix}.layers.{i}."
            q, k, v = (loader.load_tensor(p + f"self_attn.{n}_proj.weight", dt) for n in "qkv")
            L.w_qkv.data.copy_(torch.cat([q, k, v], 0))
            put(L.w_o, p + "self_attn.o_proj.weight")
            L.w_gu.data.copy_(torch.cat([loader.load_tensor(p + "mlp.gate_proj.weight", dt), loader.load_tensor(p + "mlp.up_proj.weight", dt)], 0))
            put(L.w_down, p + "mlp.down_proj.weight")
            put(L.ln_attn, p + "input_layernorm.weight")
            put(L.ln_ffn, p + "post_attention_layernorm.weight")
            if c.qk_norm:
                put(L.q_norm, p + "self_attn.q_norm.weight")
                put(L.k_norm, p + "self_attn.k_norm.weight")
        put(m.norm, prefix + ".norm.weight")
    stack(talker.stack, "talker.model")
    put(talker.stack.embed, "talker.model.codec_embedding.weight")
    put(talker.stack.lm_head, "talker.codec_head.weight")
    put(talker.text_embedding, "talker.model.text_embedding.weight")
    for n, (w, b) in (("linear_fc1", (talker.fc1_w, talker.fc1_b)), ("linear_fc2", (talker.fc2_w, talker.fc2_b))):
        put(w, f"talker.text_projection.{n}.weight")
        put(b, f"talker.text_projection.{n}.bias")
    cp = "talker.code_predictor"
    stack(predictor.stack, cp + ".model")
    for i in range(talker.cfg.num_code_groups - 1):
        put(predictor.embeddings[i], f"{cp}.model.codec_embedding.{i}.weight")
        put(predictor.heads[i], f"{cp}.lm_head.{i}.weight")
    if predictor.has_proj:
        put(predictor.proj_w, cp + ".small_to_mtp_projection.weight")
        put(predictor.proj_b, cp + ".small_to_mtp_projection.bias")
