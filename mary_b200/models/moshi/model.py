"""Full-duplex speech LM of the Moshi family: a temporal transformer over frames (one position = one 12.5 Hz frame of
17 token streams: text, 8 agent audio codebooks, 8 user audio codebooks), a depth transformer that emits the audio
codebooks of a frame one after the other, and the delay machine that staggers the streams.

Reference: dimensions and conventions src/models/personaplex/config.rs:17-80 (temporal 32 x 4096 full MHA, gated SiLU FFN
11264, RMSNorm eps 1e-8, interleaved RoPE; depformer 6 x 1024, 16 heads, FFN 2816, PER-STEP weights for 16 steps); the
stream bookkeeping src/models/personaplex/lmgen.rs:1-26,75-190 (ring of ``max_delay + 3`` positions per stream, caller
tokens written at ``offset + delay`` and flagged provided, initial tokens seeded while ``offset <= delay``, the model fed
position ``offset - 1``, sampled tokens written at ``offset`` where nothing was provided, the undelayed frame emitted once
``offset > max_delay``).  The reference runs the temporal step through per-op kernels (q8 / f16 matvec, fused add+RMSNorm,
RoPE + cache write, split-KV attention: src/models/personaplex/temporal_metal.rs:133-454) and the depformer through another
set (src/models/personaplex/depth_gpu.rs:111-308); here the temporal transformer is the package's paged-cache decoder
(``models.mistral``; interleaved RoPE is converted to split-half by permuting the q / k weight rows at load) and the depformer
steps are GEMMs of its per-step weight slices with a 16-position cache."""
from __future__ import annotations

from dataclasses import dataclass

import torch
from torch import nn

from ... import ops
from ...ops import reference as ref
from ...runtime.batch import BatchMeta
from ...runtime.kv_cache import PagedKVCache
from ..mistral.model import MistralConfig, MistralModel

UNGENERATED = -2


@dataclass
class MoshiConfig:
    dim: int = 4096
    layers: int = 32
    heads: int = 32
    ffn: int = 11264
    context: int = 3000
    eps: float = 1e-8
    rope_theta: float = 10000.0
    text_card: int = 32000
    card: int = 2048
    dep_dim: int = 1024
    dep_layers: int = 6
    dep_heads: int = 16
    dep_ffn: int = 2816
    dep_q: int = 16                               # audio codebooks the depformer emits (agent 8 + user 8)
    codebooks_per_stream: int = 8

    @property
    def num_streams(self) -> int:
        return 1 + self.dep_q

    @property
    def delays(self) -> list[int]:
        """Text and the semantic codebook of each audio stream are undelayed, the acoustic codebooks lag one frame."""
        per = [0] + [1] * (self.codebooks_per_stream - 1)
        return [0] + per * (self.dep_q // self.codebooks_per_stream)

    @property
    def max_delay(self) -> int:
        return max(self.delays)

    def initial(self, k: int) -> int:
        return self.text_card if k == 0 else self.card

    @staticmethod
    def tiny():
        return MoshiConfig(dim=64, layers=2, heads=4, ffn=96, context=64, text_card=50, card=24, dep_dim=32, dep_layers=2, dep_heads=4,
                           dep_ffn=48, dep_q=4, codebooks_per_stream=2)

    def temporal_cfg(self):
        return MistralConfig(self.layers, self.dim, self.ffn, self.heads, self.heads, self.dim // self.heads, 1, self.rope_theta, self.eps,
                             self.context, tie_word_embeddings=True, qk_norm=False, name="moshi-temporal")


class StreamCache:
    """The token bookkeeping of one conversation: pure integers, no tensors."""

    def __init__(self, c: MoshiConfig):
        self.c = c
        self.ct = c.max_delay + 3
        self.reset()

    def reset(self):
        n = self.c.num_streams
        self.cache = [[UNGENERATED] * self.ct for _ in range(n)]
        self.provided = [[False] * self.ct for _ in range(n)]
        self.offset = 0

    def prepare(self, user_audio=None, agent_audio=None, text=None):
        """Write the caller's tokens of this frame, seed initial tokens, and return the step to run: ``None`` for the very first
        call (offset 0 only seeds), else ``dict(input, target, provided, input_pos, target_pos)``."""
        c, ct, o = self.c, self.ct, self.offset
        d = c.delays
        per = c.codebooks_per_stream

        def put(k, t):
            wp = (o + d[k]) % ct
            self.cache[k][wp] = int(t)
            self.provided[k][wp] = True
        if user_audio is not None:
            for q, t in enumerate(user_audio):
                put(1 + per + q, t)
        if agent_audio is not None:
            for q, t in enumerate(agent_audio):
                put(1 + q, t)
        if text is not None:
            put(0, text)
        for k in range(c.num_streams):
            if o <= d[k]:
                self.cache[k][o % ct] = c.initial(k)
                self.provided[k][o % ct] = True
        if o == 0:
            for k in range(c.num_streams):
                self.cache[k][0] = c.initial(k)
            self.offset += 1
            return None
        ip, tp = (o - 1) % ct, o % ct
        return dict(input=[self.cache[k][ip] for k in range(c.num_streams)], target=[self.cache[k][tp] for k in range(c.num_streams)],
                    provided=[self.provided[k][tp] for k in range(c.num_streams)], input_pos=ip, target_pos=tp)

    def commit(self, p, sampled_text: int, sampled_audio):
        """Clear the consumed flags, keep the sampled tokens where nothing was provided, emit the undelayed frame (all streams)
        once past the delay horizon."""
        c, ct = self.c, self.ct
        for k in range(c.num_streams):
            self.provided[k][p["input_pos"]] = False
        if not self.provided[0][p["target_pos"]]:
            self.cache[0][p["target_pos"]] = int(sampled_text)
        for s, t in enumerate(sampled_audio):
            if not self.provided[1 + s][p["target_pos"]]:
                self.cache[1 + s][p["target_pos"]] = int(t)
        out = None
        if self.offset > c.max_delay:
            out = [self.cache[k][(self.offset - c.max_delay + c.delays[k]) % ct] for k in range(c.num_streams)]
        self.offset += 1
        return out

    def overwrite(self, snapshot) -> None:
        """Replace the token ring wholesale with a packaged snapshot ``[streams, ring]``; the ``provided`` flags and the offset are
        deliberately untouched (src/models/personaplex/lmgen.rs:188-201)."""
        rows = [[int(v) for v in row] for row in snapshot]
        if len(rows) != self.c.num_streams or any(len(r) != self.ct for r in rows):
            raise ValueError(f"cache snapshot must be [{self.c.num_streams}, {self.ct}]")
        self.cache = rows


def _P(*shape, dtype=torch.float32, device="cpu"):
    return nn.Parameter(torch.empty(*shape, dtype=dtype, device=device), requires_grad=False)


class Depformer(nn.Module):
    """Depth transformer with per-step weights: step ``t`` emits audio codebook ``t`` of the frame from the temporal hidden state
    and the token chosen at step ``t - 1`` (the text token for ``t = 0``), attending to the earlier steps of the same frame."""

    def __init__(self, c: MoshiConfig, dtype=torch.float32, device="cpu"):
        super().__init__()
        self.c = c
        S, D, F = c.dep_q, c.dep_dim, c.dep_ffn
        kw = dict(dtype=dtype, device=device)
        self.w_in = _P(S, D, c.dim, **kw)                          # depformer_in.{t}
        self.text_emb = _P(c.text_card + 1, D, **kw)               # step 0 is conditioned on the text token
        self.audio_emb = _P(S - 1, c.card + 1, D, **kw)            # depformer_emb.{t-1}
        self.norm1, self.norm2 = _P(c.dep_layers, D, **kw), _P(c.dep_layers, D, **kw)
        self.w_qkv = _P(c.dep_layers, S, 3 * D, D, **kw)           # per-step slices of the fused in_proj
        self.w_o = _P(c.dep_layers, S, D, D, **kw)
        self.w_gu = _P(c.dep_layers, S, 2 * F, D, **kw)
        self.w_down = _P(c.dep_layers, S, D, F, **kw)
        self.heads = _P(S, c.card, D, **kw)                        # linears.{t}

    def step(self, t: int, h_temporal, prev_token, cache):
        """One codebook step for a batch of frames: ``h_temporal [B, dim]``, ``prev_token [B]``, ``cache`` = list per layer of
        ``(k, v)`` buffers over all steps of the frame, rows ``0 .. t - 1`` filled (``None`` at ``t = 0``: they are created).  Returns ``(logits [B, card], cache)``."""
        c = self.c
        B = h_temporal.shape[0]
        nh, hd = c.dep_heads, c.dep_dim // c.dep_heads
        emb = ops.embed(prev_token.to(torch.int32), self.text_emb if t == 0 else self.audio_emb[t - 1])
        if B == 1 and emb.is_cuda and emb.dtype == torch.bfloat16 and c.dim <= 8192:
            from ...ops import cuda as K
            x = K.step_matvec(h_temporal, self.w_in[t], res=emb, mode="residual")        # input projection + embedding in one launch
        else:
            x = ops.linear(h_temporal, self.w_in[t]) + emb
        if cache is None:                                                              # one [B, steps, heads, dim] pair per layer, filled step by step
            cache = [(x.new_empty(B, c.dep_q, nh, hd), x.new_empty(B, c.dep_q, nh, hd)) for _ in range(c.dep_layers)]
        new_cache = cache
        # one frame on the GPU: every product is one token times a small matrix, so the norms and the residual adds ride in the
        # matrix-vector launches (rms folded into the product that follows it, the residual into the one before it)
        fused = B == 1 and x.is_cuda and x.dtype == torch.bfloat16 and max(c.dep_dim, c.dep_ffn) <= 8192
        if fused:
            from ...ops import cuda as K
        for li in range(c.dep_layers):
            if fused:
                qkv = K.step_matvec(x, self.w_qkv[li, t], self.norm1[li], c.eps)
            else:
                qkv = ops.linear(ops.rmsnorm(x, self.norm1[li], c.eps), self.w_qkv[li, t])
            q, k, v = qkv.view(B, 3, nh, hd).unbind(1)
            kc, vc = cache[li]
            kc[:, t], vc[:, t] = k, v
            a = torch.nn.functional.scaled_dot_product_attention(q[:, :, None], kc[:, :t + 1].transpose(1, 2), vc[:, :t + 1].transpose(1, 2))
            if fused:
                x = K.step_matvec(a.reshape(B, c.dep_dim), self.w_o[li, t], res=x, mode="residual")
                m = K.step_matvec(x, self.w_gu[li, t], self.norm2[li], c.eps, mode="swiglu")
                x = K.step_matvec(m, self.w_down[li, t], res=x, mode="residual")
            else:
                x = x + ops.linear(a.reshape(B, c.dep_dim), self.w_o[li, t])
                h = ops.rmsnorm(x, self.norm2[li], c.eps)
                x = x + ops.linear(ops.linear_glu(h, self.w_gu[li, t], "swiglu"), self.w_down[li, t])
        return ops.linear(x, self.heads[t]).float(), new_cache

    def generate(self, h_temporal, text_token, forced=None, sample=None):
        """All ``dep_q`` codebooks of a frame.  ``forced[s]`` (or ``None``) teacher-forces step ``s``'s token into the chain;
        ``sample(logits, s)`` picks a token (greedy when absent).  Returns tokens ``[B, dep_q]``.

        On the GPU the greedy chain (``dep_q`` steps x ``dep_layers`` layers of tiny GEMMs, no position dependence) is captured
        once per batch size as a CUDA graph and replayed per frame; forced tokens enter through a device mask / value pair."""
        if h_temporal.is_cuda and sample is None and self.use_graph:
            return self._replay(h_temporal, text_token, forced)
        prev, cache, out = text_token, None, []
        for t in range(self.c.dep_q):
            logits, cache = self.step(t, h_temporal, prev, cache)
            tok = sample(logits, t) if sample is not None else ref.argmax_first(logits)
            out.append(tok)
            prev = tok
            if forced is not None and forced[t] is not None:
                prev = torch.full_like(tok, int(forced[t]))
        return torch.stack(out, 1)

    use_graph = True

    def _chain(self, h, text_token, fmask, fval):
        prev, cache, out = text_token, None, []
        for t in range(self.c.dep_q):
            logits, cache = self.step(t, h, prev, cache)
            tok = ref.argmax_first(logits)
            out.append(tok)
            prev = torch.where(fmask[t], fval[t], tok)
        return torch.stack(out, 1)

    def _replay(self, h, text_token, forced):
        B, S = h.shape[0], self.c.dep_q
        graphs = self.__dict__.setdefault("_graphs", {})
        if B not in graphs:
            st = {"h": torch.zeros_like(h), "text": torch.zeros(B, dtype=torch.long, device=h.device),
                  "mask": torch.zeros(S, 1, dtype=torch.bool, device=h.device), "val": torch.zeros(S, 1, dtype=torch.long, device=h.device)}
            side = torch.cuda.Stream(device=h.device)
            side.wait_stream(torch.cuda.current_stream(h.device))
            with torch.cuda.stream(side):
                self._chain(st["h"], st["text"], st["mask"], st["val"])
            torch.cuda.current_stream(h.device).wait_stream(side)
            g = torch.cuda.CUDAGraph()
            with torch.cuda.graph(g):
                st["out"] = self._chain(st["h"], st["text"], st["mask"], st["val"])
            st["graph"] = g
            graphs[B] = st
        st = graphs[B]
        st["h"].copy_(h), st["text"].copy_(text_token)
        m = [f is not None for f in (forced or [None] * S)]
        v = [int(f) if f is not None else 0 for f in (forced or [None] * S)]
        st["mask"].copy_(torch.tensor(m, dtype=torch.bool).view(S, 1), non_blocking=True)
        st["val"].copy_(torch.tensor(v, dtype=torch.long).view(S, 1), non_blocking=True)
        st["graph"].replay()
        return st["out"].clone()


class LmGen(nn.Module):
    """Temporal transformer + depformer + stream bookkeeping for one conversation (batch 1)."""

    def __init__(self, c: MoshiConfig, dtype=torch.float32, device="cpu"):
        super().__init__()
        self.c = c
        dev = torch.device(device)
        self.temporal = MistralModel(c.temporal_cfg(), dtype=dtype, device=device)
        kw = dict(dtype=dtype, device=device)
        self.text_emb = _P(c.text_card + 1, c.dim, **kw)
        self.audio_emb = _P(c.dep_q, c.card + 1, c.dim, **kw)
        self.text_head = _P(c.text_card, c.dim, **kw)
        self.depformer = Depformer(c, dtype, device)
        self.stream = StreamCache(c)
        spec = self.temporal.kv_spec()
        pages = (c.context + 15) // 16
        self.cache = PagedKVCache(spec["num_layers"], pages + 1, 16, spec["kv_heads"], spec["head_dim"], dtype=dtype, device=dev)
        self.cache.alloc.extend(0, pages * 16)
        self.table, _ = self.cache.alloc.page_table([0])
        self.pos, self.dev = 0, dev

    def reset_session(self):
        self.stream.reset()
        self.pos = 0

    def embed_frame(self, tokens):
        """Sum of the stream embeddings of one frame (``tokens``: one id per stream)."""
        t = torch.as_tensor(tokens, dtype=torch.int32, device=self.dev)
        e = ops.embed(t[:1], self.text_emb).float()
        for s in range(self.c.dep_q):
            e = e + ops.embed(t[1 + s:2 + s], self.audio_emb[s]).float()
        return e.to(self.text_emb.dtype)

    def step(self, user_audio=None, agent_audio=None, text=None, sample=None):
        """One frame: returns the undelayed output frame (a list of ``num_streams`` token ids) once past the delay horizon,
        else ``None``."""
        p = self.stream.prepare(user_audio, agent_audio, text)
        if p is None:
            return None
        if self.pos >= self.c.context:
            raise RuntimeError("conversation longer than the attention context: start a new session")
        if self.dev.type == "cuda" and sample is None and self.use_graph:
            text_tok, audio = self._graph_frame(p)
            return self.stream.commit(p, text_tok, audio)
        return self._frame(self.embed_frame(p["input"]), p, sample)

    def _frame(self, x, p, sample=None):
        with torch.no_grad():
            self.pos += 1
            meta = BatchMeta.build([1], [self.pos], self.table, 16, self.dev)
            h = self.temporal.hidden_from_embeds(x, meta, self.cache)                    # [1, dim], final-normed
            text_logits = ops.linear(h, self.text_head).float()
            text_tok = sample(text_logits, -1) if sample is not None else ref.argmax_first(text_logits)
            next_text = torch.full_like(text_tok, int(p["target"][0])) if p["provided"][0] else text_tok
            forced = [p["target"][1 + s] if p["provided"][1 + s] else None for s in range(self.c.dep_q)]
            audio = self.depformer.generate(h, next_text, forced, sample)[0]
        return self.stream.commit(p, int(text_tok[0]), [int(a) for a in audio])

    # ------------------------------------------------------------------ system prompt (src/models/personaplex/pipeline.rs:117-160)
    def step_embeddings(self, x, sample=None):
        """Voice-prompt replay step: the stream cache still advances with dummy initial audio tokens and PAD text, but the temporal
        stack consumes the pre-recorded input embedding ``x [dim]`` instead of the embedding tables (lmgen.rs:287-302)."""
        from .voice_prompt import TEXT_PAD_TOKEN
        dummy = [self.c.card] * self.c.codebooks_per_stream
        p = None
        while p is None:
            p = self.stream.prepare(dummy, dummy, TEXT_PAD_TOKEN)
        if self.pos >= self.c.context:
            raise RuntimeError("voice prompt longer than the attention context")
        x = torch.as_tensor(x, device=self.dev).reshape(1, self.c.dim).to(self.text_emb.dtype)
        return self._frame(x, p, sample)

    def prompt_voice(self, voice) -> None:
        for row in voice.embeddings:
            self.step_embeddings(row)
        self.stream.overwrite(voice.cache.tolist())

    def _spacer(self, sine, silence):
        from .voice_prompt import SILENCE_TOKENS, SINE_TOKENS
        n = self.c.codebooks_per_stream
        sine, silence = list(sine or SINE_TOKENS[:n]), list(silence or SILENCE_TOKENS[:n])
        if len(sine) != n or len(silence) != n or max(sine + silence) >= self.c.card:
            raise ValueError(f"spacer frames need {n} codec tokens below {self.c.card} per stream")
        return sine, silence

    def prompt_silence(self, frames: int, sine=None, silence=None) -> None:
        """``frames`` steps of agent silence, the user's reference sine and PAD text (``sine`` / ``silence``: one frame of codec
        tokens each; default the 12.5 Hz codec's)."""
        from .voice_prompt import TEXT_PAD_TOKEN
        sine, silence = self._spacer(sine, silence)
        for _ in range(frames):
            self.step(sine, silence, TEXT_PAD_TOKEN)

    def prompt_text(self, tokens, sine=None, silence=None) -> None:
        sine, silence = self._spacer(sine, silence)
        for t in tokens:
            self.step(sine, silence, int(t))

    def run_prompt(self, prompt, sine=None, silence=None) -> None:
        """voice replay -> silence -> text -> silence (moshi ``step_system_prompts``)."""
        self.prompt_voice(prompt.voice)
        self.prompt_silence(prompt.silence_frames, sine, silence)
        self.prompt_text(prompt.text_tokens, sine, silence)
        self.prompt_silence(prompt.silence_frames, sine, silence)

    use_graph = True
    _gs = None

    def _frame_device(self, st):
        """The device side of one greedy frame over static buffers: batch descriptor from the device-resident frame counter,
        stream embeddings, temporal step, text head, forced-or-sampled text token, depth chain; the counter advances at the end."""
        n, meta, ps = st["n"], st["meta"], 16
        meta.positions.copy_(n.to(torch.int32))
        meta.kv_len.copy_((n + 1).to(torch.int32))
        page = st["table"][0].index_select(0, n // ps)
        meta.slot_mapping.copy_(page.long() * ps + n % ps)
        t = st["tokens"]
        e = ops.embed(t[:1], self.text_emb).float()
        for s in range(self.c.dep_q):
            e = e + ops.embed(t[1 + s:2 + s], self.audio_emb[s]).float()
        h = self.temporal.hidden_from_embeds(e.to(self.text_emb.dtype), meta, self.cache)
        text_tok = ref.argmax_first(ops.linear(h, self.text_head).float())
        next_text = torch.where(st["fmask"][0], st["fval"][0], text_tok)
        audio = self.depformer._chain(h, next_text, st["fmask"][1:], st["fval"][1:])
        st["out"] = torch.cat([text_tok, audio[0]])
        n.add_(1)

    def _graph_frame(self, p):
        """One frame as ONE graph replay: 17 token ids and the forced-token mask go up, 17 token ids come back."""
        S = self.c.num_streams
        if self._gs is None:
            dev = self.dev
            st = {"n": torch.zeros(1, dtype=torch.long, device=dev), "tokens": torch.zeros(S, dtype=torch.int32, device=dev),
                  "fmask": torch.zeros(S, 1, dtype=torch.bool, device=dev), "fval": torch.zeros(S, 1, dtype=torch.long, device=dev),
                  "table": torch.from_numpy(self.table).to(dev), "meta": BatchMeta.build([1], [self.c.context], self.table, 16, dev),
                  "host": torch.zeros(3, S, dtype=torch.long).pin_memory()}
            # the warm-up pass below writes the cache row of the current position; the first real frame overwrites it
            side = torch.cuda.Stream(device=dev)
            side.wait_stream(torch.cuda.current_stream(dev))
            with torch.cuda.stream(side), torch.no_grad():
                st["n"].fill_(self.pos)
                self._frame_device(st)
            torch.cuda.current_stream(dev).wait_stream(side)
            g = torch.cuda.CUDAGraph()
            with torch.cuda.graph(g), torch.no_grad():
                self._frame_device(st)
            st["graph"], st["n_host"] = g, -1
            self._gs = st
        st = self._gs
        if st["n_host"] != self.pos:                                          # a new session, or frames taken by the eager path
            st["n"].fill_(self.pos)
        host = st["host"]
        host[0] = torch.tensor(p["input"], dtype=torch.long)
        host[1] = torch.tensor([1 if f else 0 for f in p["provided"]], dtype=torch.long)
        host[2] = torch.tensor([int(v) if f else 0 for v, f in zip(p["target"], p["provided"])], dtype=torch.long)
        st["tokens"].copy_(host[0], non_blocking=True)
        st["fmask"].copy_(host[1].view(S, 1), non_blocking=True)
        st["fval"].copy_(host[2].view(S, 1), non_blocking=True)
        st["graph"].replay()
        self.pos += 1
        st["n_host"] = self.pos
        out = st["out"].tolist()
        return out[0], out[1:]


def init_random_(m: LmGen, seed: int = 0, std: float = 0.08):
    g = torch.Generator(device=m.text_emb.device).manual_seed(seed)
    for n, p in m.named_parameters():
        if p.dim() == 1 or n.endswith(("norm1", "norm2")):
            p.data.fill_(1.0)
        else:
            p.data.normal_(0.0, std, generator=g)


def load_into(m: LmGen, loader, prefix: str = "") -> None:
    """Fill the whole speech LM from the Hugging Face Moshi layout: ``decoder.model.*`` (temporal transformer: ``self_attn.{q,k,v,o}
    _proj.linear.weight``, the gated MLP's ``fc1`` = [gate; up] and ``fc2``, two RMSNorm gains per layer, the final norm),
    ``decoder.model.embed_tokens`` (text, one padding row past the vocabulary), ``decoder.lm_head`` (text logits), top-level
    ``embed_tokens.<s>`` (audio streams: the agent's codebooks first, then the user's) and ``depth_decoder.*`` (per-codebook
    "flexible" linears stored as one ``[codebooks, out, in]`` tensor each).  That layout's rotary embedding is already split-half,
    so the q / k rows are copied as they are."""
    c = m.c
    dt = m.text_emb.dtype

    def get(n):
        return loader.load_tensor(prefix + n, dt)

    def put(p, t):
        if tuple(p.shape) != tuple(t.shape):
            raise ValueError(f"shape {tuple(t.shape)} does not fit {tuple(p.shape)}")
        p.data.copy_(t.to(p.device, dt))
    put(m.text_emb, get("decoder.model.embed_tokens.weight"))
    put(m.text_head, get("decoder.lm_head.weight"))
    for s in range(c.dep_q):
        put(m.audio_emb[s], get(f"embed_tokens.{s}.weight"))
    t = m.temporal
    put(t.norm, get("decoder.model.norm.weight"))
    for i, L in enumerate(t.layers):
        p = f"decoder.model.layers.{i}."
        put(L.w_qkv, torch.cat([get(p + f"self_attn.{x}_proj.linear.weight") for x in "qkv"], 0))
        put(L.w_o, get(p + "self_attn.o_proj.linear.weight"))
        put(L.w_gu, get(p + "mlp.fc1.weight"))
        put(L.w_down, get(p + "mlp.fc2.weight"))
        put(L.ln_attn, get(p + "input_layernorm.weight"))
        put(L.ln_ffn, get(p + "post_attention_layernorm.weight"))
    d = m.depformer
    put(d.w_in, get("depth_decoder.input_projections.weight"))
    put(d.text_emb, get("depth_decoder.text_embed_tokens.weight"))
    put(d.heads, get("depth_decoder.lm_heads.weight"))
    for s in range(c.dep_q - 1):
        put(d.audio_emb[s], get(f"depth_decoder.embed_tokens.{s}.weight"))
    for li in range(c.dep_layers):
        p = f"depth_decoder.layers.{li}."
        put(d.w_qkv[li], torch.cat([get(p + f"self_attn.{x}_proj.linear.weight") for x in "qkv"], 1))
        put(d.w_o[li], get(p + "self_attn.o_proj.linear.weight"))
        put(d.w_gu[li], get(p + "mlp.fc1.weight"))
        put(d.w_down[li], get(p + "mlp.fc2.weight"))
        put(d.norm1[li], get(p + "input_layernorm.weight"))
        put(d.norm2[li], get(p + "post_attention_layernorm.weight"))
