// Training-path kernels of the LoRA fine-tuning step (forward AND backward of the element-wise pieces, and the adapter weight
// gradients), all bf16 in memory and f32 in registers.  The reference trains with burn's autodiff over its own ops
// (src/bin/gemma_train_lora.rs:259-319, adapter math src/models/gemma/lora.rs:413-428); here every piece is one launch:
//
//   rmsnorm_train_fwd / _bwd   out = (res + x * rstd(x) * w) * alpha        (w, res optional; frozen w: no weight gradient)
//   geglu_train_fwd / _bwd     out = gelu_tanh(g) * u over gu = [g | u]
//   qkv_norm_rope_fwd / _bwd   per-head RMS norm (q, k with gains, v without) followed by the split-half rotation of q and k
//   lora_wgrad                 out[r, c] = sum_m small[m, r] * big[m, c]    (dA = (dL/du)^T x and dB^T = (s u)^T dy, r <= 48)
//
// Every pointer comes with its row pitch, so that producers write straight into the widened buffers of the adapter GEMMs
// ([x | s u] and [dy | dL/du]) and no concatenation copy exists.
#include "common.cuh"
#include "host_utils.h"

namespace {
using namespace mary;

__device__ __forceinline__ void ld8(const __nv_bfloat16* p, float* f) {
  const uint4 v = *(const uint4*)p;
  const __nv_bfloat162* h = (const __nv_bfloat162*)&v;
#pragma unroll
  for (int j = 0; j < 4; ++j) { const float2 a = __bfloat1622float2(h[j]); f[2 * j] = a.x; f[2 * j + 1] = a.y; }
}
__device__ __forceinline__ void st8(__nv_bfloat16* p, const float* f) {
  uint4 v;
  __nv_bfloat162* h = (__nv_bfloat162*)&v;
#pragma unroll
  for (int j = 0; j < 4; ++j) h[j] = __floats2bfloat162_rn(f[2 * j], f[2 * j + 1]);
  *(uint4*)p = v;
}

// N consecutive bf16 values (N = 1, 2, 4 or 8; the address is a multiple of 2 N bytes)
template <int N>
__device__ __forceinline__ void ldn(const __nv_bfloat16* p, float* f) {
  if (N == 1) { f[0] = __bfloat162float(*p); return; }
  if (N == 8) { ld8(p, f); return; }
  if (N == 4) {
    const uint2 v = *(const uint2*)p;
    const __nv_bfloat162* h = (const __nv_bfloat162*)&v;
    const float2 a = __bfloat1622float2(h[0]), b = __bfloat1622float2(h[1]);
    f[0] = a.x; f[1] = a.y; f[2] = b.x; f[3] = b.y;
    return;
  }
  const float2 a = __bfloat1622float2(*(const __nv_bfloat162*)p);
  f[0] = a.x; f[1] = a.y;
}
template <int N>
__device__ __forceinline__ void stn(__nv_bfloat16* p, const float* f) {
  if (N == 1) { *p = __float2bfloat16(f[0]); return; }
  if (N == 8) { st8(p, f); return; }
  if (N == 4) {
    uint2 v;
    __nv_bfloat162* h = (__nv_bfloat162*)&v;
    h[0] = __floats2bfloat162_rn(f[0], f[1]); h[1] = __floats2bfloat162_rn(f[2], f[3]);
    *(uint2*)p = v;
    return;
  }
  *(__nv_bfloat162*)p = __floats2bfloat162_rn(f[0], f[1]);
}

// two sums over the CTA at once (one round of barriers instead of two)
__device__ __forceinline__ float2 block_sum2(float a, float b, float2* red) {
  a = warp_sum(a);
  b = warp_sum(b);
  const int w = threadIdx.x >> 5, nw = blockDim.x >> 5;
  if ((threadIdx.x & 31) == 0) red[w] = make_float2(a, b);
  __syncthreads();
  float2 t = make_float2(0.f, 0.f);
  for (int i = 0; i < nw; ++i) { t.x += red[i].x; t.y += red[i].y; }      // every thread sums the few warp totals itself
  return t;
}

// ----------------------------------------------------------------------------- RMS norm over rows of width H (H % 8 == 0)
// one CTA per row; the row stays in registers between the reduction and the write (H <= 8 * 8 * blockDim.x)
constexpr int RN_MAX = 4;   // 8-element chunks per thread

__global__ void rmsnorm_train_fwd_kernel(const __nv_bfloat16* __restrict__ x, int64_t ldx, const __nv_bfloat16* __restrict__ w,
                                         const __nv_bfloat16* __restrict__ res, int64_t ldr, float alpha, float eps,
                                         __nv_bfloat16* __restrict__ out, int64_t ldo, int H) {
  __shared__ float2 red[32];
  const int64_t row = blockIdx.x;
  const __nv_bfloat16* xr = x + row * ldx;
  float v[RN_MAX][8];
  float ss = 0.f;
#pragma unroll
  for (int i = 0; i < RN_MAX; ++i) {
    const int c = (i * blockDim.x + threadIdx.x) * 8;
    if (c < H) {
      ld8(xr + c, v[i]);
#pragma unroll
      for (int j = 0; j < 8; ++j) ss = fmaf(v[i][j], v[i][j], ss);
    }
  }
  const float rstd = rsqrtf(block_sum2(ss, 0.f, red).x / (float)H + eps);
#pragma unroll
  for (int i = 0; i < RN_MAX; ++i) {
    const int c = (i * blockDim.x + threadIdx.x) * 8;
    if (c < H) {
      float g[8], r[8], o[8];
      if (w) ld8(w + c, g);
      if (res) ld8(res + row * ldr + c, r);
#pragma unroll
      for (int j = 0; j < 8; ++j) {
        float y = v[i][j] * rstd;
        if (w) y *= g[j];
        if (res) y += r[j];
        o[j] = y * alpha;
      }
      st8(out + row * ldo + c, o);
    }
  }
}

// dx = alpha * rstd * (g - xhat * mean(g * xhat)),  g = dy * w,  xhat = x * rstd  (rstd recomputed from x)
// d_res (optional) = alpha * dy
__global__ void rmsnorm_train_bwd_kernel(const __nv_bfloat16* __restrict__ dy, int64_t ldy, const __nv_bfloat16* __restrict__ x, int64_t ldx,
                                         const __nv_bfloat16* __restrict__ w, float alpha, float eps, __nv_bfloat16* __restrict__ dx,
                                         int64_t lddx, __nv_bfloat16* __restrict__ dres, int64_t lddr, int H) {
  __shared__ float2 red[32];
  const int64_t row = blockIdx.x;
  float xv[RN_MAX][8], gv[RN_MAX][8];
  float ss = 0.f, sg = 0.f;
#pragma unroll
  for (int i = 0; i < RN_MAX; ++i) {
    const int c = (i * blockDim.x + threadIdx.x) * 8;
    if (c < H) {
      float g[8];
      ld8(x + row * ldx + c, xv[i]);
      ld8(dy + row * ldy + c, gv[i]);
      if (dres) {
        float o[8];
#pragma unroll
        for (int j = 0; j < 8; ++j) o[j] = gv[i][j] * alpha;
        st8(dres + row * lddr + c, o);
      }
      if (w) ld8(w + c, g);
#pragma unroll
      for (int j = 0; j < 8; ++j) {
        if (w) gv[i][j] *= g[j];
        ss = fmaf(xv[i][j], xv[i][j], ss);
        sg = fmaf(gv[i][j], xv[i][j], sg);
      }
    }
  }
  const float2 tot = block_sum2(ss, sg, red);
  ss = tot.x;
  sg = tot.y;
  const float rstd = rsqrtf(ss / (float)H + eps);
  const float k = sg * rstd * rstd / (float)H;        // mean(g * xhat) * rstd
#pragma unroll
  for (int i = 0; i < RN_MAX; ++i) {
    const int c = (i * blockDim.x + threadIdx.x) * 8;
    if (c < H) {
      float o[8];
#pragma unroll
      for (int j = 0; j < 8; ++j) o[j] = alpha * rstd * (gv[i][j] - xv[i][j] * k);
      st8(dx + row * lddx + c, o);
    }
  }
}

// ----------------------------------------------------------------------------- GeGLU (tanh form)
__device__ __forceinline__ void gelu_tanh_and_grad(float x, float* val, float* grad) {
  const float k0 = 0.7978845608028654f, k1 = 0.044715f;
  const float t = tanhf(k0 * (x + k1 * x * x * x));
  *val = 0.5f * x * (1.0f + t);
  *grad = 0.5f * (1.0f + t) + 0.5f * x * (1.0f - t * t) * k0 * (1.0f + 3.0f * k1 * x * x);
}

__global__ void geglu_train_fwd_kernel(const __nv_bfloat16* __restrict__ gu, int64_t ldg, __nv_bfloat16* __restrict__ out, int64_t ldo, int F,
                                       int64_t rows) {
  const int c = (blockIdx.x * blockDim.x + threadIdx.x) * 8;
  if (c >= F) return;
  for (int64_t row = blockIdx.y; row < rows; row += gridDim.y) {
    float g[8], u[8], o[8];
    ld8(gu + row * ldg + c, g);
    ld8(gu + row * ldg + F + c, u);
#pragma unroll
    for (int j = 0; j < 8; ++j) o[j] = gelu_tanh_f(g[j]) * u[j];
    st8(out + row * ldo + c, o);
  }
}

__global__ void geglu_train_bwd_kernel(const __nv_bfloat16* __restrict__ dout, int64_t ldd, const __nv_bfloat16* __restrict__ gu, int64_t ldg,
                                       __nv_bfloat16* __restrict__ dgu, int64_t lddg, int F, int64_t rows) {
  const int c = (blockIdx.x * blockDim.x + threadIdx.x) * 8;
  if (c >= F) return;
  for (int64_t row = blockIdx.y; row < rows; row += gridDim.y) {
    float g[8], u[8], d[8], dg[8], du[8];
    ld8(gu + row * ldg + c, g);
    ld8(gu + row * ldg + F + c, u);
    ld8(dout + row * ldd + c, d);
#pragma unroll
    for (int j = 0; j < 8; ++j) {
      float val, grad;
      gelu_tanh_and_grad(g[j], &val, &grad);
      dg[j] = d[j] * u[j] * grad;
      du[j] = d[j] * val;
    }
    st8(dgu + row * lddg + c, dg);
    st8(dgu + row * lddg + F + c, du);
  }
}

// ----------------------------------------------------------------------------- per-head norm + rotation of a fused q | k | v row
// one warp per (token, head); head dim D = 8 * 32 * CH / ... : every lane holds D / 32 values as pairs (i, i + D / 2) so that the
// rotation needs no exchange: lane l holds elements [l * D/64, (l + 1) * D/64) of each half.
template <int D, bool BWD>
__global__ void qkv_norm_rope_kernel(const __nv_bfloat16* __restrict__ in, int64_t ldi, const __nv_bfloat16* __restrict__ x, int64_t ldx,
                                     const int* __restrict__ pos, const float* __restrict__ inv_freq, const __nv_bfloat16* __restrict__ qw,
                                     const __nv_bfloat16* __restrict__ kw, float eps, __nv_bfloat16* __restrict__ out, int64_t ldo, int n_q,
                                     int n_kv, int64_t n_rows) {
  constexpr int PER = D / 64;                     // values per lane and half
  const int heads = n_q + 2 * n_kv;
  const int64_t wid = (int64_t)blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5);
  if (wid >= n_rows * heads) return;
  const int lane = threadIdx.x & 31;
  const int64_t t = wid / heads;
  const int h = (int)(wid % heads);
  const bool is_v = h >= n_q + n_kv;
  const __nv_bfloat16* gain = h < n_q ? qw : (is_v ? nullptr : kw);
  const int c0 = h * D + lane * PER;
  float a[PER], b[PER], ga[PER], gb[PER], cs[PER], sn[PER];
  if (gain) { ldn<PER>(gain + lane * PER, ga); ldn<PER>(gain + D / 2 + lane * PER, gb); }
#pragma unroll
  for (int j = 0; j < PER; ++j) {
    if (!gain) { ga[j] = 1.f; gb[j] = 1.f; }
    if (!is_v) {
      const float ang = (float)pos[t] * inv_freq[lane * PER + j];
      sincosf(ang, &sn[j], &cs[j]);
    } else { cs[j] = 1.f; sn[j] = 0.f; }
  }
  if (!BWD) {
    // forward: in = raw projection row; out = rope(norm(in))
    float ss = 0.f;
    ldn<PER>(in + t * ldi + c0, a);
    ldn<PER>(in + t * ldi + c0 + D / 2, b);
#pragma unroll
    for (int j = 0; j < PER; ++j) ss = fmaf(a[j], a[j], fmaf(b[j], b[j], ss));
    const float rstd = rsqrtf(warp_sum(ss) / (float)D + eps);
    float o1[PER], o2[PER];
#pragma unroll
    for (int j = 0; j < PER; ++j) {
      // the normed value is rounded to the storage type before it is rotated (two ops in the reference)
      const float na = __bfloat162float(__float2bfloat16(a[j] * rstd * ga[j])), nb = __bfloat162float(__float2bfloat16(b[j] * rstd * gb[j]));
      o1[j] = na * cs[j] - nb * sn[j];
      o2[j] = na * sn[j] + nb * cs[j];
    }
    stn<PER>(out + t * ldo + c0, o1);
    stn<PER>(out + t * ldo + c0 + D / 2, o2);
  } else {
    // backward: in = gradient of the rotated row, x = raw projection row; out = gradient of the raw row
    float xa[PER], xb[PER], d1[PER], d2[PER];
    float ss = 0.f, sg = 0.f;
    ldn<PER>(in + t * ldi + c0, d1);
    ldn<PER>(in + t * ldi + c0 + D / 2, d2);
    ldn<PER>(x + t * ldx + c0, xa);
    ldn<PER>(x + t * ldx + c0 + D / 2, xb);
#pragma unroll
    for (int j = 0; j < PER; ++j) {
      a[j] = (d1[j] * cs[j] + d2[j] * sn[j]) * ga[j];            // transpose of the rotation, then the gain
      b[j] = (-d1[j] * sn[j] + d2[j] * cs[j]) * gb[j];
      ss = fmaf(xa[j], xa[j], fmaf(xb[j], xb[j], ss));
      sg = fmaf(a[j], xa[j], fmaf(b[j], xb[j], sg));
    }
    ss = warp_sum(ss);
    sg = warp_sum(sg);
    const float rstd = rsqrtf(ss / (float)D + eps);
    const float k = sg * rstd * rstd / (float)D;
    float o1[PER], o2[PER];
#pragma unroll
    for (int j = 0; j < PER; ++j) {
      o1[j] = rstd * (a[j] - xa[j] * k);
      o2[j] = rstd * (b[j] - xb[j] * k);
    }
    stn<PER>(out + t * ldo + c0, o1);
    stn<PER>(out + t * ldo + c0 + D / 2, o2);
  }
}

// ----------------------------------------------------------------------------- adapter weight gradients
// ws[split, r, c] = sum over the split's rows m of small[m, r] * big[m, c], r < Rv <= R; 128 threads x CPT columns per CTA
template <int R, int CPT>
__global__ void __launch_bounds__(128) lora_wgrad_kernel(const __nv_bfloat16* __restrict__ small, int64_t lds, const __nv_bfloat16* __restrict__ big,
                                                         int64_t ldb, int M, int C, int rows_per_split, float* __restrict__ ws, int Rv) {
  __shared__ __align__(16) float sm[32][R];
  const int c0 = (blockIdx.x * 128 + threadIdx.x) * CPT;
  const int m_lo = blockIdx.y * rows_per_split, m_hi = min(M, m_lo + rows_per_split);
  float acc[R][CPT];
#pragma unroll
  for (int r = 0; r < R; ++r)
#pragma unroll
    for (int j = 0; j < CPT; ++j) acc[r][j] = 0.f;
  for (int m0 = m_lo; m0 < m_hi; m0 += 32) {
    __syncthreads();
    for (int i = threadIdx.x; i < 32 * R; i += 128) {
      const int mi = i / R, r = i % R;
      sm[mi][r] = (m0 + mi < m_hi && r < Rv) ? __bfloat162float(small[(int64_t)(m0 + mi) * lds + r]) : 0.f;
    }
    __syncthreads();
    if (c0 < C) {
      const int n = min(32, m_hi - m0);
#pragma unroll 2
      for (int mi = 0; mi < n; ++mi) {
        float v[CPT];
        const __nv_bfloat16* bp = big + (int64_t)(m0 + mi) * ldb + c0;
        if (CPT == 8) ld8(bp, v);
        else {
#pragma unroll
          for (int j = 0; j < CPT; j += 2) { const float2 f = __bfloat1622float2(*(const __nv_bfloat162*)(bp + j)); v[j] = f.x; v[j + 1] = f.y; }
        }
#pragma unroll
        for (int r4 = 0; r4 < R; r4 += 4) {
          const float4 s = *(const float4*)&sm[mi][r4];
#pragma unroll
          for (int j = 0; j < CPT; ++j) {
            acc[r4][j] = fmaf(s.x, v[j], acc[r4][j]);
            acc[r4 + 1][j] = fmaf(s.y, v[j], acc[r4 + 1][j]);
            acc[r4 + 2][j] = fmaf(s.z, v[j], acc[r4 + 2][j]);
            acc[r4 + 3][j] = fmaf(s.w, v[j], acc[r4 + 3][j]);
          }
        }
      }
    }
  }
  if (c0 < C) {
#pragma unroll
    for (int r = 0; r < R; ++r)
      if (r < Rv) {
#pragma unroll
        for (int j = 0; j < CPT; ++j) ws[((int64_t)blockIdx.y * Rv + r) * C + c0 + j] = acc[r][j];
      }
  }
}

// The same product on the tensor cores (mma.sync m16n8k16, bf16 in, f32 out): the contraction runs over the TOKENS, which is
// the strided dimension of both operands, so both fragments are read with ldmatrix.trans from row-major shared tiles.  The
// kernel is bound by streaming `big` once; tcgen05 would need both operands MN-major and brings nothing at 16-48 output rows.
//   CTA: 128 threads, 256 columns (64 per warp = 8 n-tiles), rows of its split in chunks of 32 (two k-steps)
//   RT: 16-row tiles of the output (Rv <= 16 RT, Rv % 8 == 0)
constexpr int WG_COLS = 256, WG_KT = 32;
constexpr int WG_BPITCH = WG_COLS * 2 + 16;     // bytes; the 16 spreads the 8 rows of an ldmatrix over the banks
constexpr int WG_SPITCH = 48 * 2 + 16;

__device__ __forceinline__ void ldsm_x4_trans(uint32_t addr, uint32_t& r0, uint32_t& r1, uint32_t& r2, uint32_t& r3) {
  asm volatile("ldmatrix.sync.aligned.m8n8.x4.trans.shared.b16 {%0, %1, %2, %3}, [%4];" : "=r"(r0), "=r"(r1), "=r"(r2), "=r"(r3) : "r"(addr));
}
__device__ __forceinline__ void mma_bf16_16816(float* c, const uint32_t* a, uint32_t b0, uint32_t b1) {
  asm volatile("mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0, %1, %2, %3}, {%4, %5, %6, %7}, {%8, %9}, {%0, %1, %2, %3};"
               : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3]) : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1));
}

template <int RT>
__global__ void __launch_bounds__(128) lora_wgrad_tc_kernel(const __nv_bfloat16* __restrict__ small, int64_t lds,
                                                            const __nv_bfloat16* __restrict__ big, int64_t ldb, int M, int C,
                                                            int rows_per_split, float* __restrict__ ws, int Rv) {
  __shared__ __align__(16) uint8_t sb[WG_KT * WG_BPITCH];
  __shared__ __align__(16) uint8_t ss[WG_KT * WG_SPITCH];
  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  const int col0 = blockIdx.x * WG_COLS;
  const int m_lo = blockIdx.y * rows_per_split, m_hi = min(M, m_lo + rows_per_split);
  float acc[RT][8][4];
#pragma unroll
  for (int a = 0; a < RT; ++a)
#pragma unroll
    for (int n = 0; n < 8; ++n)
#pragma unroll
      for (int j = 0; j < 4; ++j) acc[a][n][j] = 0.f;
  uint4 pb[8], ps[2];
  const uint4 zero = make_uint4(0, 0, 0, 0);
  auto fetch = [&](int m0) {
#pragma unroll
    for (int i = 0; i < 8; ++i) {
      const int id = i * 128 + tid, row = id >> 5, ch = id & 31;
      const int m = m0 + row, c = col0 + ch * 8;
      pb[i] = (m < m_hi && c < C) ? *(const uint4*)(big + (int64_t)m * ldb + c) : zero;
    }
#pragma unroll
    for (int i = 0; i < 2; ++i) {
      const int id = i * 128 + tid, row = id / (2 * RT), ch = id % (2 * RT);
      const int m = m0 + row;
      ps[i] = (id < WG_KT * 2 * RT && m < m_hi && ch * 8 < Rv) ? *(const uint4*)(small + (int64_t)m * lds + ch * 8) : zero;
    }
  };
  fetch(m_lo);
  const uint32_t sb_u = smem_u32(sb), ss_u = smem_u32(ss);
  for (int m0 = m_lo; m0 < m_hi; m0 += WG_KT) {
    __syncthreads();                                   // the previous chunk's fragments have been read
#pragma unroll
    for (int i = 0; i < 8; ++i) {
      const int id = i * 128 + tid, row = id >> 5, ch = id & 31;
      *(uint4*)(sb + row * WG_BPITCH + ch * 16) = pb[i];
    }
#pragma unroll
    for (int i = 0; i < 2; ++i) {
      const int id = i * 128 + tid, row = id / (2 * RT), ch = id % (2 * RT);
      if (id < WG_KT * 2 * RT) *(uint4*)(ss + row * WG_SPITCH + ch * 16) = ps[i];
    }
    __syncthreads();
    if (m0 + WG_KT < m_hi) fetch(m0 + WG_KT);          // the next chunk travels while this one is multiplied
#pragma unroll
    for (int ks = 0; ks < WG_KT / 16; ++ks) {
      uint32_t a[RT][4];
#pragma unroll
      for (int rt = 0; rt < RT; ++rt) {
        // matrices: (r0, k0) (r0 + 8, k0) (r0, k0 + 8) (r0 + 8, k0 + 8), each the transpose of ss[k .. k + 8][r .. r + 8]
        const int mrow = ks * 16 + (lane >> 4) * 8 + (lane & 7), rcol = rt * 16 + ((lane >> 3) & 1) * 8;
        ldsm_x4_trans(ss_u + mrow * WG_SPITCH + rcol * 2, a[rt][0], a[rt][1], a[rt][2], a[rt][3]);
      }
#pragma unroll
      for (int np = 0; np < 4; ++np) {
        // matrices: (k0, c0) (k0 + 8, c0) (k0, c0 + 8) (k0 + 8, c0 + 8): b0, b1 of two neighbouring n-tiles
        const int mrow = ks * 16 + ((lane >> 3) & 1) * 8 + (lane & 7), ccol = warp * 64 + np * 16 + (lane >> 4) * 8;
        uint32_t b0, b1, b2, b3;
        ldsm_x4_trans(sb_u + mrow * WG_BPITCH + ccol * 2, b0, b1, b2, b3);
#pragma unroll
        for (int rt = 0; rt < RT; ++rt) {
          mma_bf16_16816(acc[rt][2 * np], a[rt], b0, b1);
          mma_bf16_16816(acc[rt][2 * np + 1], a[rt], b2, b3);
        }
      }
    }
  }
  const int g = lane >> 2, t = lane & 3;
#pragma unroll
  for (int rt = 0; rt < RT; ++rt)
#pragma unroll
    for (int n = 0; n < 8; ++n) {
      const int c = col0 + warp * 64 + n * 8 + 2 * t;
      if (c < C) {
        const int r0 = rt * 16 + g, r1 = r0 + 8;
        if (r0 < Rv) *(float2*)(ws + ((int64_t)blockIdx.y * Rv + r0) * C + c) = make_float2(acc[rt][n][0], acc[rt][n][1]);
        if (r1 < Rv) *(float2*)(ws + ((int64_t)blockIdx.y * Rv + r1) * C + c) = make_float2(acc[rt][n][2], acc[rt][n][3]);
      }
    }
}

// ----------------------------------------------------------------------------- soft-capped cross-entropy, loss and gradient
// One CTA per row of logits [rows, V] (bf16): z = cap * tanh(l / cap) (cap <= 0: z = l); loss = logsumexp(z) - z[label];
// the row is OVERWRITTEN with d loss / d l * scale = scale * (softmax(z) - onehot) * (1 - tanh^2).  Two passes over the row:
// an online (max, sum) pass and the write pass, which finds the row in L2 (a row is 2 V bytes, the concurrently processed rows
// of all SMs stay below the L2 size for vocabularies up to 400k).
// tanh through exp: the fast-math tanh approximation (relative error near 1e-3) would move a soft-capped logit by 0.01 and more
__device__ __forceinline__ float tanh_exp(float x) { return 1.f - __fdividef(2.f, __expf(2.f * x) + 1.f); }

__device__ __forceinline__ void ms_merge(float& m, float& s, float m2, float s2) {
  const float mn = fmaxf(m, m2);
  if (mn == -INFINITY) return;                       // two empty partials: (-inf) - (-inf) would be NaN
  s = s * __expf(m - mn) + s2 * __expf(m2 - mn);
  m = mn;
}

__global__ void __launch_bounds__(1024) softcap_ce_kernel(__nv_bfloat16* __restrict__ logits, int64_t ld, const int64_t* __restrict__ labels,
                                                          int V, float cap, float scale, float* __restrict__ loss) {
  __shared__ float red_m[32], red_s[32];
  __shared__ float sh_lse, sh_zy;
  const int64_t row = blockIdx.x;
  __nv_bfloat16* lr = logits + row * ld;
  const float inv_cap = cap > 0.f ? 1.f / cap : 0.f;
  const int label = (int)labels[row];
  float m = -INFINITY, sum = 0.f;
  for (int c = threadIdx.x * 8; c < V; c += blockDim.x * 8) {
    float v[8];
    ld8(lr + c, v);
#pragma unroll
    for (int j = 0; j < 8; ++j) {
      const float z = cap > 0.f ? cap * tanh_exp(v[j] * inv_cap) : v[j];
      if (c + j == label) sh_zy = z;
      if (z > m) { sum = sum * __expf(m - z) + 1.f; m = z; } else sum += __expf(z - m);
    }
  }
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) {
    const float m2 = __shfl_xor_sync(0xffffffffu, m, o), s2 = __shfl_xor_sync(0xffffffffu, sum, o);
    ms_merge(m, sum, m2, s2);
  }
  const int w = threadIdx.x >> 5, nw = blockDim.x >> 5;
  if ((threadIdx.x & 31) == 0) { red_m[w] = m; red_s[w] = sum; }
  __syncthreads();
  if (w == 0) {
    m = (int)threadIdx.x < nw ? red_m[threadIdx.x] : -INFINITY;
    sum = (int)threadIdx.x < nw ? red_s[threadIdx.x] : 0.f;
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) {
      const float m2 = __shfl_xor_sync(0xffffffffu, m, o), s2 = __shfl_xor_sync(0xffffffffu, sum, o);
      ms_merge(m, sum, m2, s2);
    }
    if (threadIdx.x == 0) {
      sh_lse = m + __logf(sum);
      loss[row] = (label >= 0 && label < V) ? sh_lse - sh_zy : 0.f;
    }
  }
  __syncthreads();
  const float lse = sh_lse;
  const float on = (label >= 0 && label < V) ? scale : 0.f;      // a label outside the vocabulary: the row is ignored
  for (int c = threadIdx.x * 8; c < V; c += blockDim.x * 8) {
    float v[8], o[8];
    ld8(lr + c, v);
#pragma unroll
    for (int j = 0; j < 8; ++j) {
      float t = 0.f, z = v[j];
      if (cap > 0.f) { t = tanh_exp(v[j] * inv_cap); z = cap * t; }
      const float p = __expf(z - lse);
      o[j] = on * (p - (c + j == label ? 1.f : 0.f)) * (1.f - t * t);
    }
    st8(lr + c, o);
  }
}

// out[r, c] = sum over splits of ws[split, r, c]
__global__ void lora_wgrad_reduce_kernel(const float* __restrict__ ws, int splits, int64_t n, float* __restrict__ out) {
  const int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
  if (i >= n) return;
  float s = 0.f;
  for (int k = 0; k < splits; ++k) s += ws[(int64_t)k * n + i];
  out[i] = s;
}
}  // namespace

static inline int rn_threads(int H) {
  int t = (H / 8 + RN_MAX - 1) / RN_MAX;
  t = (t + 31) / 32 * 32;
  return t < 32 ? 32 : t;
}

MARY_API int mary_rmsnorm_train_fwd(const void* x, int64_t ldx, const void* w, const void* res, int64_t ldr, float alpha, float eps, void* out,
                                    int64_t ldo, int64_t rows, int H, cudaStream_t s) {
  if (rows <= 0) return MARY_OK;
  if ((H & 7) || (ldx & 7) || (ldo & 7) || (res && (ldr & 7)) || H > 8 * RN_MAX * 1024) return MARY_ERR_BAD_ARG;
  rmsnorm_train_fwd_kernel<<<(unsigned)rows, rn_threads(H), 0, s>>>((const __nv_bfloat16*)x, ldx, (const __nv_bfloat16*)w, (const __nv_bfloat16*)res,
                                                                   ldr, alpha, eps, (__nv_bfloat16*)out, ldo, H);
  MARY_CHECK_LAUNCH();
  return MARY_OK;
}

MARY_API int mary_rmsnorm_train_bwd(const void* dy, int64_t ldy, const void* x, int64_t ldx, const void* w, float alpha, float eps, void* dx,
                                    int64_t lddx, void* dres, int64_t lddr, int64_t rows, int H, cudaStream_t s) {
  if (rows <= 0) return MARY_OK;
  if ((H & 7) || (ldx & 7) || (ldy & 7) || (lddx & 7) || (dres && (lddr & 7)) || H > 8 * RN_MAX * 1024) return MARY_ERR_BAD_ARG;
  rmsnorm_train_bwd_kernel<<<(unsigned)rows, rn_threads(H), 0, s>>>((const __nv_bfloat16*)dy, ldy, (const __nv_bfloat16*)x, ldx,
                                                                   (const __nv_bfloat16*)w, alpha, eps, (__nv_bfloat16*)dx, lddx,
                                                                   (__nv_bfloat16*)dres, lddr, H);
  MARY_CHECK_LAUNCH();
  return MARY_OK;
}

MARY_API int mary_geglu_train_fwd(const void* gu, int64_t ldg, void* out, int64_t ldo, int64_t rows, int F, cudaStream_t s) {
  if (rows <= 0) return MARY_OK;
  if ((F & 7) || (ldg & 7) || (ldo & 7)) return MARY_ERR_BAD_ARG;
  const dim3 grid((F / 8 + 255) / 256, (unsigned)(rows < 65535 ? rows : 65535));
  geglu_train_fwd_kernel<<<grid, 256, 0, s>>>((const __nv_bfloat16*)gu, ldg, (__nv_bfloat16*)out, ldo, F, rows);
  MARY_CHECK_LAUNCH();
  return MARY_OK;
}

MARY_API int mary_geglu_train_bwd(const void* dout, int64_t ldd, const void* gu, int64_t ldg, void* dgu, int64_t lddg, int64_t rows, int F,
                                  cudaStream_t s) {
  if (rows <= 0) return MARY_OK;
  if ((F & 7) || (ldg & 7) || (ldd & 7) || (lddg & 7)) return MARY_ERR_BAD_ARG;
  const dim3 grid((F / 8 + 255) / 256, (unsigned)(rows < 65535 ? rows : 65535));
  geglu_train_bwd_kernel<<<grid, 256, 0, s>>>((const __nv_bfloat16*)dout, ldd, (const __nv_bfloat16*)gu, ldg, (__nv_bfloat16*)dgu, lddg, F, rows);
  MARY_CHECK_LAUNCH();
  return MARY_OK;
}

// bwd == 0: out = rope(norm(in)); bwd != 0: in = gradient of the output, x = the forward's input, out = gradient of that input
MARY_API int mary_qkv_norm_rope_train(const void* in, int64_t ldi, const void* x, int64_t ldx, const int* pos, const float* inv_freq,
                                      const void* qw, const void* kw, float eps, void* out, int64_t ldo, int n_q, int n_kv, int D,
                                      int64_t rows, int bwd, cudaStream_t s) {
  if (rows <= 0) return MARY_OK;
  if ((D != 64 && D != 128 && D != 256 && D != 512) || n_q < 1 || n_kv < 1 || (bwd && !x) || (ldi & 7) || (ldo & 7) || (bwd && (ldx & 7))) return MARY_ERR_BAD_ARG;
  const int64_t warps = rows * (n_q + 2 * n_kv);
  const unsigned grid = (unsigned)((warps + 7) / 8);
#define QNR(D_)                                                                                                                             \
  if (bwd) qkv_norm_rope_kernel<D_, true><<<grid, 256, 0, s>>>((const __nv_bfloat16*)in, ldi, (const __nv_bfloat16*)x, ldx, pos, inv_freq,   \
                                                               (const __nv_bfloat16*)qw, (const __nv_bfloat16*)kw, eps, (__nv_bfloat16*)out, \
                                                               ldo, n_q, n_kv, rows);                                                       \
  else qkv_norm_rope_kernel<D_, false><<<grid, 256, 0, s>>>((const __nv_bfloat16*)in, ldi, (const __nv_bfloat16*)x, ldx, pos, inv_freq,      \
                                                            (const __nv_bfloat16*)qw, (const __nv_bfloat16*)kw, eps, (__nv_bfloat16*)out,    \
                                                            ldo, n_q, n_kv, rows)
  if (D == 64) { QNR(64); } else if (D == 128) { QNR(128); } else if (D == 256) { QNR(256); } else { QNR(512); }
#undef QNR
  MARY_CHECK_LAUNCH();
  return MARY_OK;
}

// out[R, C] (f32) = small[M, R]^T big[M, C], 1 <= R <= 48; ws: scratch of mary_lora_wgrad_splits(M, C, R) * R * C floats.
// R % 8 == 0 with 16-byte aligned operands takes the tensor-core kernel, anything else the SIMT one.
static inline bool wgrad_tc_ok(const void* small, int64_t lds, const void* big, int R) {
  return (R & 7) == 0 && (lds & 7) == 0 && ((uintptr_t)small & 15) == 0 && ((uintptr_t)big & 15) == 0;
}

MARY_API int mary_lora_wgrad_splits(int M, int C, int R) {
  const int cpt = R <= 16 ? 8 : (R <= 32 ? 4 : 2);
  const int per_cta = (R & 7) == 0 ? WG_COLS : 128 * cpt;
  const int slabs = (C + per_cta - 1) / per_cta;
  int splits = (((R & 7) == 0 ? 4 : 2) * mary_num_sms() + slabs - 1) / slabs;
  const int max_splits = (M + 31) / 32;
  if (splits > max_splits) splits = max_splits;
  if (splits > 64) splits = 64;
  return splits < 1 ? 1 : splits;
}

MARY_API int mary_lora_wgrad(const void* small, int64_t lds, const void* big, int64_t ldb, int M, int R, int C, float* ws, float* out,
                             cudaStream_t s) {
  if (M <= 0 || C <= 0) return MARY_OK;
  if (R < 1 || R > 48 || (C & 7) || (ldb & 7)) return MARY_ERR_BAD_ARG;
  const int splits = mary_lora_wgrad_splits(M, C, R);
  int rps = (M + splits - 1) / splits;
  rps = (rps + 31) / 32 * 32;
  if (wgrad_tc_ok(small, lds, big, R)) {
    const dim3 grid((C + WG_COLS - 1) / WG_COLS, splits);
    if (R <= 16) lora_wgrad_tc_kernel<1><<<grid, 128, 0, s>>>((const __nv_bfloat16*)small, lds, (const __nv_bfloat16*)big, ldb, M, C, rps, ws, R);
    else if (R <= 32) lora_wgrad_tc_kernel<2><<<grid, 128, 0, s>>>((const __nv_bfloat16*)small, lds, (const __nv_bfloat16*)big, ldb, M, C, rps, ws, R);
    else lora_wgrad_tc_kernel<3><<<grid, 128, 0, s>>>((const __nv_bfloat16*)small, lds, (const __nv_bfloat16*)big, ldb, M, C, rps, ws, R);
  } else {
    const int cpt = R <= 16 ? 8 : (R <= 32 ? 4 : 2);
    const dim3 grid((C + 128 * cpt - 1) / (128 * cpt), splits);
    if (R <= 16) lora_wgrad_kernel<16, 8><<<grid, 128, 0, s>>>((const __nv_bfloat16*)small, lds, (const __nv_bfloat16*)big, ldb, M, C, rps, ws, R);
    else if (R <= 32) lora_wgrad_kernel<32, 4><<<grid, 128, 0, s>>>((const __nv_bfloat16*)small, lds, (const __nv_bfloat16*)big, ldb, M, C, rps, ws, R);
    else lora_wgrad_kernel<48, 2><<<grid, 128, 0, s>>>((const __nv_bfloat16*)small, lds, (const __nv_bfloat16*)big, ldb, M, C, rps, ws, R);
  }
  MARY_CHECK_LAUNCH();
  const int64_t n = (int64_t)R * C;
  lora_wgrad_reduce_kernel<<<(unsigned)((n + 255) / 256), 256, 0, s>>>(ws, splits, n, out);
  MARY_CHECK_LAUNCH();
  return MARY_OK;
}

// Soft-capped cross-entropy of rows of logits: loss[row] and, in place of the logits, scale * d loss / d logits.
MARY_API int mary_softcap_ce(void* logits, int64_t ld, const int64_t* labels, int64_t rows, int V, float cap, float scale, float* loss,
                             cudaStream_t s) {
  if (rows <= 0) return MARY_OK;
  if ((V & 7) || (ld & 7)) return MARY_ERR_BAD_ARG;
  const int threads = V >= 8192 ? 1024 : (V >= 2048 ? 256 : 64);
  softcap_ce_kernel<<<(unsigned)rows, threads, 0, s>>>((__nv_bfloat16*)logits, ld, labels, V, cap, scale, loss);
  MARY_CHECK_LAUNCH();
  return MARY_OK;
}
