"""CUDA arm of the streaming codec: the weights of a ``MimiCodec`` re-laid for the tensor-core GEMM, activations kept
time-major ``[L, C]`` in f32 between layers and gathered to bf16 GEMM rows by ``csrc/kernels/codec.cu``.

A convolution ``[C_out, C_in, k]`` becomes the GEMM weight ``[C_out, k * C_in]`` (tap-major, the order the im2col gather
writes); a transposed convolution ``[C_in, C_out, k]`` becomes ``[k * C_out, C_in]`` so that one GEMM yields every tap's
contribution and the overlap-add kernel sums the (at most ``k / stride``) taps that land on each output sample.  The
codebook search is the GEMM ``r . c^T`` with bias ``-|c|^2 / 2`` followed by the device arg-max.  The transformer uses the
package's paged attention with a sliding window."""
from __future__ import annotations

import torch
import torch.nn.functional as F

from ...ops import cuda as K
from ...ops.cuda import _p, _stream, check, declare, lib
from ...runtime.batch import BatchMeta
from ...runtime.kv_cache import PagedKVCache
from .mimi import MimiCodec

declare("mary_im2col_causal", "ppppiiiiiiis")
declare("mary_overlap_add", "pppppiiiis")
declare("mary_dw_transconv", "pppppiiiis")
declare("mary_layernorm", "ppppiifs")
declare("mary_act_bf16", "pplis")


def _pad8(n):
    """GEMM rows are TMA loads: 16-byte row pitch (8 bf16) and at least one 64-element K tile."""
    return max((n + 7) // 8 * 8, 64)


class _Conv:
    def __init__(self, m, dev):
        w = m.weight.detach().float()
        self.cout, self.cin, self.k = w.shape
        self.stride, self.replicate = m.stride, m.replicate
        self.kc = self.k * self.cin
        self.ld = _pad8(self.kc)
        self.npad = (self.cout + 7) // 8 * 8
        wg = torch.zeros(self.npad, self.ld)
        wg[:self.cout, :self.kc] = w.permute(0, 2, 1).reshape(self.cout, self.kc)
        self.w = wg.to(dev, torch.bfloat16)
        self.b = None
        if m.bias is not None:
            self.b = torch.zeros(self.npad, device=dev)
            self.b[:self.cout] = m.bias.detach().float().to(dev)

    def __call__(self, x, state, act=0):
        """``x [L, Cin]`` f32 -> ``([L / stride, Cout] f32, new state)``; ``act`` is applied to the input on the way."""
        L = x.shape[0]
        T = L // self.stride
        col = torch.zeros(T, self.ld, dtype=torch.bfloat16, device=x.device) if self.ld != self.kc else \
            torch.empty(T, self.ld, dtype=torch.bfloat16, device=x.device)
        ctx = self.k - self.stride
        new_state = torch.empty(max(ctx, 1), self.cin, dtype=torch.float32, device=x.device)
        check(lib().mary_im2col_causal(_p(x), _p(state), _p(new_state), _p(col), self.ld, L, self.cin, self.k, self.stride, act,
                                       int(self.replicate), _stream()), "im2col_causal")
        y = K.gemm(col, self.w, bias=self.b, epi="f32")
        return (y if self.npad == self.cout else y[:, :self.cout].contiguous()), new_state


class _TransConv:
    def __init__(self, m, dev):
        w = m.weight.detach().float()                     # [Cin, Cout / groups, k]
        self.k, self.stride, self.depthwise = m.k, m.stride, m.groups > 1
        self.cin = w.shape[0]
        if self.depthwise:
            self.cout = self.cin
            self.w = w[:, 0, :].contiguous().to(dev)      # [C, k]
            self.b = None
        else:
            self.cout = w.shape[1]
            self.w = w.permute(2, 1, 0).reshape(self.k * self.cout, self.cin).contiguous().to(dev, torch.bfloat16)
            self.b = m.bias.detach().float().to(dev)

    def __call__(self, x, tail, act=0):
        T = x.shape[0]
        y = torch.empty(T * self.stride, self.cout, dtype=torch.float32, device=x.device)
        new_tail = torch.empty(max(self.k - self.stride, 1), self.cout, dtype=torch.float32, device=x.device)
        if self.depthwise:
            check(lib().mary_dw_transconv(_p(x), _p(self.w), _p(tail), _p(new_tail), _p(y), T, self.cin, self.k, self.stride, _stream()),
                  "dw_transconv")
            return y, new_tail
        xa = torch.empty(T, self.cin, dtype=torch.bfloat16, device=x.device)
        check(lib().mary_act_bf16(_p(x), _p(xa), x.numel(), act, _stream()), "act_bf16")
        z = K.gemm(xa, self.w, epi="f32")                 # [T, k * Cout]
        check(lib().mary_overlap_add(_p(z), _p(tail), _p(new_tail), _p(self.b), _p(y), T, self.cout, self.k, self.stride, _stream()),
              "overlap_add")
        return y, new_tail


class _Res:
    def __init__(self, m, dev):
        self.c1, self.c2 = _Conv(m.c1, dev), _Conv(m.c2, dev)

    def __call__(self, x, state):
        s = state or [None, None]
        h, s0 = self.c1(x, s[0], act=1)
        h, s1 = self.c2(h, s[1], act=1)
        return x + h, [s0, s1]


class _Transformer:
    def __init__(self, m, c, dev, max_frames: int):
        self.c, self.dev = c, dev
        f32 = lambda t: t.detach().float().to(dev)          # noqa: E731
        bf = lambda t: t.detach().to(dev, torch.bfloat16)   # noqa: E731
        self.layers = [dict(ln1=(f32(L.ln1_w), f32(L.ln1_b)), ln2=(f32(L.ln2_w), f32(L.ln2_b)), qkv=bf(L.w_qkv), o=bf(L.w_o),
                            fc1=bf(L.w_fc1), fc2=bf(L.w_fc2), s1=f32(L.scale1), s2=f32(L.scale2)) for L in m.layers]
        self.nh, self.hd = c.tr_heads, c.hidden // c.tr_heads
        self.max_frames = max_frames
        self.inv = (c.rope_theta ** (-torch.arange(0, self.hd, 2, dtype=torch.float32) / self.hd)).to(dev)

    def new_state(self):
        pages = (self.max_frames + 15) // 16
        cache = PagedKVCache(len(self.layers), pages + 1, 16, self.nh, self.hd, dtype=torch.bfloat16, device=self.dev)
        cache.alloc.extend(0, pages * 16)
        table, _ = cache.alloc.page_table([0])
        return {"pos": 0, "cache": cache, "table": table}

    def _ln(self, x, wb):
        out = torch.empty(x.shape, dtype=torch.bfloat16, device=x.device)
        check(lib().mary_layernorm(_p(x), _p(wb[0]), _p(wb[1]), _p(out), x.shape[0], x.shape[1], self.c.tr_eps, _stream()), "layernorm")
        return out

    def __call__(self, x, st):
        """``x [T, H]`` f32 -> same; the KV cache of ``st`` grows by ``T`` positions."""
        st = st or self.new_state()
        T, H = x.shape
        pos0 = st["pos"]
        if pos0 + T > self.max_frames:
            raise ValueError("codec transformer cache exhausted: raise max_frames")
        meta = BatchMeta.build([T], [pos0 + T], st["table"], 16, self.dev)
        ang = meta.positions[:, None].float() * self.inv[None]
        cos, sin = ang.cos()[:, None, :], ang.sin()[:, None, :]

        def rot(t):
            a, b = t[..., 0::2].float(), t[..., 1::2].float()
            return torch.stack([a * cos - b * sin, a * sin + b * cos], -1).reshape(t.shape).to(torch.bfloat16)
        cache = st["cache"]
        for li, L in enumerate(self.layers):
            qkv = K.gemm(self._ln(x, L["ln1"]), L["qkv"]).view(T, 3, self.nh, self.hd)
            q, k, v = rot(qkv[:, 0]), rot(qkv[:, 1]), qkv[:, 2]
            cache.k[li].view(-1, self.nh, self.hd)[meta.slot_mapping] = k
            cache.v[li].view(-1, self.nh, self.hd)[meta.slot_mapping] = v
            a = K.paged_attention(q.contiguous(), cache.k[li], cache.v[li], meta, self.hd ** -0.5, self.c.tr_window, kernel="general")
            x = torch.addcmul(x, L["s1"], K.gemm(a.reshape(T, H), L["o"], epi="f32"))
            h = K.gemm(self._ln(x, L["ln2"]), L["fc1"], epi="f32")
            g = torch.empty(h.shape, dtype=torch.bfloat16, device=h.device)
            check(lib().mary_act_bf16(_p(h), _p(g), h.numel(), 2, _stream()), "act_bf16")
            x = torch.addcmul(x, L["s2"], K.gemm(g, L["fc2"], epi="f32"))
        st["pos"] = pos0 + T
        return x, st


class _RVQ:
    def __init__(self, m, dev):
        self.inp = m.input_proj.detach().to(dev, torch.bfloat16)
        self.out = m.output_proj.detach().to(dev, torch.bfloat16)
        cw = [b.codewords().detach().float() for b in m.books]
        self.cw32 = [c.to(dev) for c in cw]
        self.cw = [c.to(dev, torch.bfloat16) for c in cw]
        self.bias = [(-0.5 * (c.to(torch.bfloat16).float() ** 2).sum(-1)).to(dev) for c in cw]

    def encode(self, x):
        r = K.gemm(x.to(torch.bfloat16), self.inp, epi="f32")
        codes = []
        for cw, cw32, b in zip(self.cw, self.cw32, self.bias):
            score = K.gemm(r.to(torch.bfloat16), cw, bias=b, epi="f32")
            i, _ = K.argmax(score)
            r = r - cw32[i]
            codes.append(i)
        return torch.stack(codes, -1)

    def decode(self, codes):
        q = sum(cw[codes[:, j]] for j, cw in enumerate(self.cw32))
        return K.gemm(q.to(torch.bfloat16), self.out, epi="f32")


class MimiCuda:
    """``MimiCodec`` weights on a CUDA device with the kernels above.  ``max_frames`` bounds a streaming session (transformer
    positions); ``encode_step`` / ``decode_step`` mirror the CPU arm."""

    def __init__(self, codec: MimiCodec, device="cuda", max_frames: int = 4096):
        c = self.c = codec.c
        dev = self.dev = torch.device(device)
        self.enc_stem = _Conv(codec.enc_stem, dev)
        self.enc_res = [_Res(m, dev) for m in codec.enc_res]
        self.enc_down = [_Conv(m, dev) for m in codec.enc_down]
        self.enc_last = _Conv(codec.enc_last, dev)
        self.enc_tr = _Transformer(codec.enc_tr, c, dev, 2 * max_frames)
        self.downsample = _Conv(codec.downsample, dev)
        self.rvq_first, self.rvq_rest = _RVQ(codec.rvq_first, dev), _RVQ(codec.rvq_rest, dev)
        self.upsample = _TransConv(codec.upsample, dev)
        self.dec_tr = _Transformer(codec.dec_tr, c, dev, 2 * max_frames)
        self.dec_stem = _Conv(codec.dec_stem, dev)
        self.dec_up = [_TransConv(m, dev) for m in codec.dec_up]
        self.dec_res = [_Res(m, dev) for m in codec.dec_res]
        self.dec_last = _Conv(codec.dec_last, dev)

    def encode_step(self, pcm, state=None):
        assert pcm.shape[0] % self.c.samples_per_frame == 0, "feed whole frames"
        st = dict(state or {})
        x = pcm.to(self.dev, torch.float32).reshape(-1, 1)
        x, st["stem"] = self.enc_stem(x, st.get("stem"))
        for i, (res, down) in enumerate(zip(self.enc_res, self.enc_down)):
            x, st[f"res{i}"] = res(x, st.get(f"res{i}"))
            x, st[f"down{i}"] = down(x, st.get(f"down{i}"), act=1)
        x, st["last"] = self.enc_last(x, st.get("last"), act=1)
        x, st["tr"] = self.enc_tr(x, st.get("tr"))
        x, st["ds"] = self.downsample(x, st.get("ds"))
        return torch.cat([self.rvq_first.encode(x), self.rvq_rest.encode(x)], -1), st

    def decode_step(self, codes, state=None):
        st = dict(state or {})
        codes = codes.to(self.dev)
        x = self.rvq_first.decode(codes[:, :1]) + self.rvq_rest.decode(codes[:, 1:])
        x, st["up"] = self.upsample(x, st.get("up"))
        x, st["tr"] = self.dec_tr(x, st.get("tr"))
        x, st["stem"] = self.dec_stem(x, st.get("stem"))
        for i, (up, res) in enumerate(zip(self.dec_up, self.dec_res)):
            x, st[f"up{i}"] = up(x, st.get(f"up{i}"), act=1)
            x, st[f"res{i}"] = res(x, st.get(f"res{i}"))
        x, st["last"] = self.dec_last(x, st.get("last"), act=1)
        return x[:, 0], st

    def encode(self, pcm):
        pad = (-pcm.shape[0]) % self.c.samples_per_frame
        return self.encode_step(F.pad(pcm, (0, pad)))[0]

    def decode(self, codes):
        return self.decode_step(codes)[0]
