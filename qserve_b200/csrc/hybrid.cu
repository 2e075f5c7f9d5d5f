// qserve_b200 -- kernels of the unquantised hybrid decoders (attention layers and recurrent layers in one stack, fp32 residual stream).
//
// Everything here works on a FLAT batch of tokens: a step of the engine brings, for every live sequence, a run of consecutive
// tokens (a portion of a prompt or one decoded token).  Per-token tables (`tok_slot`, `tok_pos`, `tok_entry`) and per-entry tables
// (`entry_start`, `entry_len`, `entry_slot`, `entry_pos0`) say where a token belongs; the paged key/value cache is addressed through a
// block table indexed by the sequence's slot.  The same kernels therefore serve whole prompts, portions and single decoded tokens, and a
// position's result does not depend on what else is in the batch.
//
// Storage type ST is bfloat16 or float (the engine's activation / cache type); scores, softmax weights, norms, rotary angles, decays,
// gates of the recurrence, the recurrent state and the residual stream are fp32 in both.
#include <cuda_bf16.h>
#include <math.h>

#include "../../include/qserve_b200.h"
#include "common.cuh"
#include "launch.h"

namespace qs {
namespace {

template <typename ST> __device__ __forceinline__ float ldf(const ST* p);
template <> __device__ __forceinline__ float ldf<float>(const float* p) { return *p; }
template <> __device__ __forceinline__ float ldf<__nv_bfloat16>(const __nv_bfloat16* p) { return __bfloat162float(*p); }
template <typename ST> __device__ __forceinline__ void stf(ST* p, float v);
template <> __device__ __forceinline__ void stf<float>(float* p, float v) { *p = v; }
template <> __device__ __forceinline__ void stf<__nv_bfloat16>(__nv_bfloat16* p, float v) { *p = __float2bfloat16_rn(v); }

__device__ __forceinline__ float warp_sum(float v) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
  return v;
}
__device__ __forceinline__ float warp_max(float v) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v = fmaxf(v, __shfl_xor_sync(0xffffffffu, v, o));
  return v;
}
// block-wide sum / max over up to 32 warps; `red` holds 33 floats; every thread gets the result
__device__ __forceinline__ float block_sum(float v, float* red) {
  v = warp_sum(v);
  const int w = threadIdx.x >> 5, nw = (blockDim.x + 31) >> 5;
  __syncthreads();
  if ((threadIdx.x & 31) == 0) red[w] = v;
  __syncthreads();
  float t = (threadIdx.x & 31) < nw ? red[threadIdx.x & 31] : 0.f;
  return warp_sum(t);
}
__device__ __forceinline__ float block_max(float v, float* red) {
  v = warp_max(v);
  const int w = threadIdx.x >> 5, nw = (blockDim.x + 31) >> 5;
  __syncthreads();
  if ((threadIdx.x & 31) == 0) red[w] = v;
  __syncthreads();
  float t = (threadIdx.x & 31) < nw ? red[threadIdx.x & 31] : -INFINITY;
  return warp_max(t);
}

__device__ __forceinline__ float silu_f(float z) { return z / (1.f + expf(-z)); }

// ---------------------------------------------------------------------------------------------------------------------------------
// embedding: token row (+ hashed (previous, current) pair row) -> fp32 residual stream
// ---------------------------------------------------------------------------------------------------------------------------------
template <typename ST>
__global__ void embed_pair_kernel(float* __restrict__ out, const int* __restrict__ tokens, const int* __restrict__ prev, const ST* __restrict__ table,
                                  const ST* __restrict__ pair, int W, int buckets, long long mul_prev, long long mul_cur) {
  const int t = blockIdx.x;
  const long long tok = tokens[t];
  const ST* e = table + tok * W;
  const ST* b = nullptr;
  if (pair != nullptr) {
    const long long p = prev[t];
    const long long row = p < 0 ? buckets : (p * mul_prev + tok * mul_cur) % buckets;
    b = pair + row * W;
  }
  for (int i = threadIdx.x; i < W; i += blockDim.x) out[(size_t)t * W + i] = ldf(e + i) + (b ? ldf(b + i) : 0.f);
}

// ---------------------------------------------------------------------------------------------------------------------------------
// RMS norm of the fp32 stream with one or two gains (the two branches of a parallel layer read the same normalised row):
//   out_k = x * rsqrt(mean(x^2) + eps) * (offset + w_k)
// ---------------------------------------------------------------------------------------------------------------------------------
template <typename ST>
__global__ void rms_norm2_kernel(ST* __restrict__ out1, ST* __restrict__ out2, const float* __restrict__ x, const float* __restrict__ w1,
                                 const float* __restrict__ w2, float offset, float eps, int W) {
  __shared__ float red[33];
  const float* row = x + (size_t)blockIdx.x * W;
  float ss = 0.f;
  for (int i = threadIdx.x; i < W; i += blockDim.x) {
    const float v = row[i];
    ss += v * v;
  }
  ss = block_sum(ss, red);
  const float r = 1.f / sqrtf(ss / (float)W + eps);
  for (int i = threadIdx.x; i < W; i += blockDim.x) {
    const float v = row[i] * r;
    stf(out1 + (size_t)blockIdx.x * W + i, v * (offset + w1[i]));
    if (out2 != nullptr) stf(out2 + (size_t)blockIdx.x * W + i, v * (offset + w2[i]));
  }
}

// x += y  (fp32 stream, y in the storage type)
template <typename ST>
__global__ void residual_add_kernel(float* __restrict__ x, const ST* __restrict__ y, size_t n) {
  const size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
  if (i < n) x[i] += ldf(y + i);
}

// out[t, i] = gelu_tanh(in[t, i]) * in[t, ff + i]
template <typename ST>
__global__ void gelu_tanh_mul_kernel(ST* __restrict__ out, long long out_stride, const ST* __restrict__ in, int ff) {
  const int t = blockIdx.x;
  const int i = blockIdx.y * blockDim.x + threadIdx.x;
  if (i >= ff) return;
  const float z = ldf(in + (size_t)t * 2 * ff + i), u = ldf(in + (size_t)t * 2 * ff + ff + i);
  const float g = 0.5f * z * (1.f + tanhf(0.7978845608028654f * (z + 0.044715f * z * z * z)));
  stf(out + (size_t)t * out_stride + i, g * u);
}

// ---------------------------------------------------------------------------------------------------------------------------------
// rotary embedding (interleaved pairs, per-pair frequency table, amplitude factor) on the q and k parts of the projection row, and the
// append of the rotated key row and the value row to the paged cache.
//   row layout: [H * maps * D queries | G * maps * D keys | G * Dv values]
//   K page: [page_size][G][maps * D], V page: [page_size][G][Dv]
// grid (tokens, H + G); the first H blocks rotate a query head in place, the others rotate + store a key head and copy its value head.
// ---------------------------------------------------------------------------------------------------------------------------------
template <typename ST>
__global__ void rope_append_kernel(ST* __restrict__ proj, long long stride, const int* __restrict__ tok_slot, const int* __restrict__ tok_pos,
                                   const int* __restrict__ block_table, int max_blocks, ST* __restrict__ kpool, ST* __restrict__ vpool,
                                   const float* __restrict__ inv_freq, float amp, int H, int G, int maps, int D, int Dv, int rot_dims, int page) {
  const int t = blockIdx.x, u = blockIdx.y;
  const int pos = tok_pos[t];
  const int half = rot_dims >> 1;
  ST* row = proj + (size_t)t * stride;
  if (u < H) {
    ST* q = row + (size_t)u * maps * D;
    for (int i = threadIdx.x; i < maps * half; i += blockDim.x) {
      const int m = i / half, p = i - m * half;
      float s, c;
      sincosf((float)pos * inv_freq[p], &s, &c);
      s *= amp; c *= amp;
      ST* a = q + m * D + 2 * p;
      const float x0 = ldf(a), x1 = ldf(a + 1);
      stf(a, x0 * c - x1 * s);
      stf(a + 1, x1 * c + x0 * s);
    }
    return;
  }
  const int g = u - H;
  const int slot = tok_slot[t];
  const int pg = block_table[(size_t)slot * max_blocks + pos / page];
  const size_t cell = (size_t)pg * page + (pos % page);
  const ST* k = row + (size_t)H * maps * D + (size_t)g * maps * D;
  ST* kd = kpool + (cell * G + g) * (size_t)(maps * D);
  for (int i = threadIdx.x; i < maps * D; i += blockDim.x) {
    const int d = i % D;
    float v;
    if (d < rot_dims) {
      const int p = d >> 1;
      float s, c;
      sincosf((float)pos * inv_freq[p], &s, &c);
      s *= amp; c *= amp;
      const int b0 = i - d;
      const float x0 = ldf(k + b0 + (d & ~1)), x1 = ldf(k + b0 + (d | 1));
      v = (d & 1) ? (x1 * c + x0 * s) : (x0 * c - x1 * s);
    } else {
      v = ldf(k + i);
    }
    stf(kd + i, v);
  }
  const ST* vs = row + (size_t)(H + G) * maps * D + (size_t)g * Dv;
  ST* vd = vpool + (cell * G + g) * (size_t)Dv;
  for (int i = threadIdx.x; i < Dv; i += blockDim.x) vd[i] = vs[i];
}

// ---------------------------------------------------------------------------------------------------------------------------------
// causal attention over the paged cache with `MAPS` softmax maps per head that share the values (MAPS = 2: differential attention).
// One block per (token, query head).  Keys are walked in tiles of KT; a warp scores one key at a time with coalesced loads of the
// key row (fp32 dot products), the block keeps an online softmax per map (fp32 weights), and thread d accumulates output dimension(s)
// d, d + blockDim, ... for every map.  Epilogue:
//   MAPS == 2: o = a1 - lambda a2;   then (head_norm) o <- o * rsqrt(mean(o^2) + eps);   o <- o * out_scale
// ---------------------------------------------------------------------------------------------------------------------------------
constexpr int kAttnThreads = 128;
constexpr int kAttnKT = 128;
constexpr int kAttnMaxV = 4;  // value dims per thread: Dv <= 512

template <typename ST, int MAPS>
__global__ void __launch_bounds__(kAttnThreads) paged_multimap_attention_kernel(
    ST* __restrict__ out, long long out_stride, const ST* __restrict__ q, long long q_stride, const ST* __restrict__ kpool,
    const ST* __restrict__ vpool, const int* __restrict__ tok_slot, const int* __restrict__ tok_pos, const int* __restrict__ block_table,
    int max_blocks, int H, int G, int D, int Dv, float scale, float lambda, float out_scale, float eps, int head_norm, int page) {
  extern __shared__ float sm[];
  float* qs = sm;                      // [MAPS * D]
  float* ps = qs + MAPS * D;           // [MAPS][KT]
  float* red = ps + MAPS * kAttnKT;    // [33]
  __shared__ int pages[kAttnKT];       // page of every key of the tile (KT keys span at most KT pages)

  const int t = blockIdx.x, h = blockIdx.y, g = h / (H / G);
  const int pos = tok_pos[t], slot = tok_slot[t];
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  const int* bt = block_table + (size_t)slot * max_blocks;

  const ST* qrow = q + (size_t)t * q_stride + (size_t)h * MAPS * D;
  for (int i = threadIdx.x; i < MAPS * D; i += blockDim.x) qs[i] = ldf(qrow + i);

  float m_run[MAPS], l_run[MAPS], acc[MAPS][kAttnMaxV];
#pragma unroll
  for (int m = 0; m < MAPS; ++m) {
    m_run[m] = -INFINITY;
    l_run[m] = 0.f;
#pragma unroll
    for (int j = 0; j < kAttnMaxV; ++j) acc[m][j] = 0.f;
  }
  const int n_keys = pos + 1;
  for (int base = 0; base < n_keys; base += kAttnKT) {
    const int nk = min(kAttnKT, n_keys - base);
    __syncthreads();  // previous tile's ps / pages fully consumed (and qs written, first time)
    for (int j = threadIdx.x; j < nk; j += blockDim.x) pages[j] = bt[(base + j) / page];
    __syncthreads();
    // scores: warp per key
    for (int j = warp; j < nk; j += kAttnThreads / 32) {
      const int kj = base + j;
      const ST* kr = kpool + (((size_t)pages[j] * page + (kj % page)) * G + g) * (size_t)(MAPS * D);
#pragma unroll
      for (int m = 0; m < MAPS; ++m) {
        float d = 0.f;
        for (int i = lane; i < D; i += 32) d += qs[m * D + i] * ldf(kr + m * D + i);
        d = warp_sum(d);
        if (lane == 0) ps[m * kAttnKT + j] = d * scale;
      }
    }
    __syncthreads();
    // online softmax per map
    float corr[MAPS];
#pragma unroll
    for (int m = 0; m < MAPS; ++m) {
      float mx = -INFINITY;
      for (int j = threadIdx.x; j < nk; j += blockDim.x) mx = fmaxf(mx, ps[m * kAttnKT + j]);
      mx = block_max(mx, red);
      const float m_new = fmaxf(m_run[m], mx);
      float s = 0.f;
      for (int j = threadIdx.x; j < nk; j += blockDim.x) {
        const float p = expf(ps[m * kAttnKT + j] - m_new);
        ps[m * kAttnKT + j] = p;
        s += p;
      }
      s = block_sum(s, red);
      corr[m] = expf(m_run[m] - m_new);  // 0 on the first tile (m_run = -inf)
      l_run[m] = l_run[m] * corr[m] + s;
      m_run[m] = m_new;
    }
    __syncthreads();
    // weighted values: thread owns output dims
#pragma unroll
    for (int j = 0; j < kAttnMaxV; ++j) {
      const int d = threadIdx.x + j * kAttnThreads;
      if (d < Dv) {
        float a[MAPS];
#pragma unroll
        for (int m = 0; m < MAPS; ++m) a[m] = acc[m][j] * corr[m];
        for (int kk = 0; kk < nk; ++kk) {
          const int kj = base + kk;
          const float v = ldf(vpool + (((size_t)pages[kk] * page + (kj % page)) * G + g) * (size_t)Dv + d);
#pragma unroll
          for (int m = 0; m < MAPS; ++m) a[m] += ps[m * kAttnKT + kk] * v;
        }
#pragma unroll
        for (int m = 0; m < MAPS; ++m) acc[m][j] = a[m];
      }
    }
  }
  // epilogue
  float o[kAttnMaxV];
  float ss = 0.f;
#pragma unroll
  for (int j = 0; j < kAttnMaxV; ++j) {
    const int d = threadIdx.x + j * kAttnThreads;
    o[j] = 0.f;
    if (d < Dv) {
      float v = acc[0][j] / l_run[0];
      if (MAPS == 2) v -= lambda * (acc[MAPS - 1][j] / l_run[MAPS - 1]);
      o[j] = v;
      ss += v * v;
    }
  }
  float r = out_scale;
  if (head_norm) {
    ss = block_sum(ss, red);
    r *= 1.f / sqrtf(ss / (float)Dv + eps);
  }
  ST* orow = out + (size_t)t * out_stride + (size_t)h * Dv;
#pragma unroll
  for (int j = 0; j < kAttnMaxV; ++j) {
    const int d = threadIdx.x + j * kAttnThreads;
    if (d < Dv) stf(orow + d, o[j] * r);
  }
}

// ---------------------------------------------------------------------------------------------------------------------------------
// gated delta rule, step 1: per token, short causal convolution + silu over the q | k | v channels (taps before the portion come from
// the sequence's convolution state, taps before the sequence's start are zero), unit-length q (times D^-1/2) and k per head, the write
// strength beta = sigmoid(b) and the decay exp(-exp(A_log) softplus(a + dt_bias)) per head.  All fp32 from the projections on.
//   projection row: [G*D q | G*D k | H*Dv v | H*Dv output gate | H b | H a]
//   prepared row (fp32): [G*D q | G*D k | H*Dv v | H beta | H decay]
//   convolution state (fp32): [slots][taps - 1][C], oldest first, C = 2 G D + H Dv
// ---------------------------------------------------------------------------------------------------------------------------------
template <typename ST>
__global__ void delta_prepare_kernel(float* __restrict__ prep, const ST* __restrict__ proj, long long stride, const float* __restrict__ conv_w,
                                     const float* __restrict__ conv_state, const float* __restrict__ a_log, const float* __restrict__ dt_bias,
                                     const int* __restrict__ tok_entry, const int* __restrict__ tok_pos, const int* __restrict__ entry_start,
                                     const int* __restrict__ entry_slot, int H, int G, int D, int Dv, int taps, float unit_eps) {
  extern __shared__ float y[];  // [C]
  const int t = blockIdx.x;
  const int C = 2 * G * D + H * Dv;
  const int P = C + 2 * H;
  const int e = tok_entry[t], pos = tok_pos[t];
  const int local = t - entry_start[e];
  const float* st = conv_state + (size_t)entry_slot[e] * (taps - 1) * C;
  for (int c = threadIdx.x; c < C; c += blockDim.x) {
    float a = 0.f;
    for (int j = 0; j < taps; ++j) {
      const int back = taps - 1 - j;
      if (pos - back < 0) continue;
      float x;
      if (local - back >= 0) x = ldf(proj + (size_t)(t - back) * stride + c);
      else x = st[(size_t)(taps - 1 + local - back) * C + c];
      a += conv_w[(size_t)c * taps + j] * x;
    }
    y[c] = silu_f(a);
  }
  __syncthreads();
  float* o = prep + (size_t)t * P;
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, nw = blockDim.x >> 5;
  for (int u = warp; u < 2 * G; u += nw) {  // q heads then k heads
    const float* v = y + (size_t)u * D;
    float ss = 0.f;
    for (int i = lane; i < D; i += 32) ss += v[i] * v[i];
    ss = warp_sum(ss);
    float r = 1.f / sqrtf(ss + unit_eps);
    if (u < G) r *= 1.f / sqrtf((float)D);
    for (int i = lane; i < D; i += 32) o[(size_t)u * D + i] = v[i] * r;
  }
  for (int c = 2 * G * D + threadIdx.x; c < C; c += blockDim.x) o[c] = y[c];
  const ST* row = proj + (size_t)t * stride;
  for (int hh = threadIdx.x; hh < H; hh += blockDim.x) {
    const float b = ldf(row + C + H * Dv + hh);
    const float a = ldf(row + C + H * Dv + H + hh) + dt_bias[hh];
    const float sp = a > 20.f ? a : log1pf(expf(a));
    o[C + hh] = 1.f / (1.f + expf(-b));
    o[C + H + hh] = expf(-expf(a_log[hh]) * sp);
  }
}

// step 1b: the sequence's convolution state after the portion = its last taps-1 inputs (older ones shift out)
template <typename ST>
__global__ void delta_conv_state_kernel(float* __restrict__ conv_state, const ST* __restrict__ proj, long long stride,
                                        const int* __restrict__ entry_start, const int* __restrict__ entry_len, const int* __restrict__ entry_slot,
                                        const int* __restrict__ entry_pos0, int C, int taps) {
  const int e = blockIdx.y;
  const int c = blockIdx.x * blockDim.x + threadIdx.x;
  if (c >= C) return;
  const int n = entry_len[e], s0 = entry_start[e], keep = taps - 1;
  float* st = conv_state + (size_t)entry_slot[e] * keep * C;
  const bool fresh = entry_pos0[e] == 0;
  float tmp[16];
  for (int i = 0; i < keep; ++i) {
    const int src = n - keep + i;  // index in the portion, negative: older than the portion
    if (src >= 0) tmp[i] = ldf(proj + (size_t)(s0 + src) * stride + c);
    else tmp[i] = fresh ? 0.f : st[(size_t)(keep + src) * C + c];
  }
  for (int i = 0; i < keep; ++i) st[(size_t)i * C + c] = tmp[i];
}

// step 2: the recurrence.  One block per (entry, head); thread d owns column d of the head's [D, Dv] state in registers (D <= DP).
// Per token, in this order:  S <- decay S;  u = beta (v - S^T k);  S <- S + k u^T;  o = S^T q.
template <int DP>
__global__ void delta_scan_kernel(float* __restrict__ o_raw, const float* __restrict__ prep, float* __restrict__ state,
                                  const int* __restrict__ entry_start, const int* __restrict__ entry_len, const int* __restrict__ entry_slot,
                                  const int* __restrict__ entry_pos0, int H, int G, int D, int Dv) {
  __shared__ float qk[2][2 * DP];
  const int e = blockIdx.x, h = blockIdx.y, g = h / (H / G);
  const int d = threadIdx.x;
  const int C = 2 * G * D + H * Dv, P = C + 2 * H;
  const int n = entry_len[e], s0 = entry_start[e];
  float* Sg = state + ((size_t)entry_slot[e] * H + h) * (size_t)D * Dv;
  float S[DP];
  const bool live = d < Dv;
  const bool fresh = entry_pos0[e] == 0;
#pragma unroll
  for (int i = 0; i < DP; ++i) S[i] = (live && !fresh && i < D) ? Sg[(size_t)i * Dv + d] : 0.f;
  for (int i = threadIdx.x; i < 2 * DP; i += blockDim.x) {
    const int which = i / DP, j = i - which * DP;
    qk[0][i] = j < D ? prep[(size_t)s0 * P + (size_t)which * G * D + (size_t)g * D + j] : 0.f;
  }
  __syncthreads();
  for (int t = 0; t < n; ++t) {
    const float* row = prep + (size_t)(s0 + t) * P;
    const float* cur = qk[t & 1];
    if (t + 1 < n) {  // stage the next token's q | k while this one is processed
      float* nxt = qk[(t + 1) & 1];
      for (int i = threadIdx.x; i < 2 * DP; i += blockDim.x) {
        const int which = i / DP, j = i - which * DP;
        nxt[i] = j < D ? row[P + (size_t)which * G * D + (size_t)g * D + j] : 0.f;
      }
    }
    if (live) {
      const float decay = row[C + H + h], beta = row[C + h], v = row[2 * G * D + (size_t)h * Dv + d];
      float kS = 0.f;
#pragma unroll
      for (int i = 0; i < DP; ++i) {
        S[i] *= decay;
        kS += S[i] * cur[DP + i];
      }
      const float u = beta * (v - kS);
      float o = 0.f;
#pragma unroll
      for (int i = 0; i < DP; ++i) {
        S[i] += cur[DP + i] * u;
        o += S[i] * cur[i];
      }
      o_raw[(size_t)(s0 + t) * H * Dv + (size_t)h * Dv + d] = o;
    }
    __syncthreads();
  }
  if (live) {
#pragma unroll
    for (int i = 0; i < DP; ++i)
      if (i < D) Sg[(size_t)i * Dv + d] = S[i];
  }
}

// step 3: per (token, head) unit-RMS read-out times a shared per-dimension weight times silu(output gate); one warp each
template <typename ST>
__global__ void delta_gate_out_kernel(ST* __restrict__ out, long long out_stride, const float* __restrict__ o_raw, const ST* __restrict__ proj,
                                      long long stride, const float* __restrict__ norm_w, int T, int H, int G, int D, int Dv, float eps) {
  const int w = (blockIdx.x * blockDim.x + threadIdx.x) >> 5, lane = threadIdx.x & 31;
  if (w >= T * H) return;
  const int t = w / H, h = w - t * H;
  const float* o = o_raw + (size_t)t * H * Dv + (size_t)h * Dv;
  const ST* gate = proj + (size_t)t * stride + 2 * G * D + H * Dv + (size_t)h * Dv;
  float ss = 0.f;
  for (int i = lane; i < Dv; i += 32) ss += o[i] * o[i];
  ss = warp_sum(ss);
  const float r = 1.f / sqrtf(ss / (float)Dv + eps);
  ST* dst = out + (size_t)t * out_stride + (size_t)h * Dv;
  for (int i = lane; i < Dv; i += 32) stf(dst + i, o[i] * r * norm_w[i] * silu_f(ldf(gate + i)));
}

template <typename ST>
int launch_attention(void* out, long long out_stride, const void* q, long long q_stride, const void* kpool, const void* vpool, const int* tok_slot,
                     const int* tok_pos, const int* block_table, int max_blocks, int T, int H, int G, int maps, int D, int Dv, float scale,
                     float lambda, float out_scale, float eps, int head_norm, int page, cudaStream_t s) {
  const size_t smem = (size_t)(maps * D + maps * kAttnKT + 33) * sizeof(float);
  dim3 grid(T, H);
  if (maps == 2) {
    if (smem > 48 * 1024) cudaFuncSetAttribute(paged_multimap_attention_kernel<ST, 2>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
    paged_multimap_attention_kernel<ST, 2><<<grid, kAttnThreads, smem, s>>>((ST*)out, out_stride, (const ST*)q, q_stride, (const ST*)kpool,
        (const ST*)vpool, tok_slot, tok_pos, block_table, max_blocks, H, G, D, Dv, scale, lambda, out_scale, eps, head_norm, page);
  } else {
    if (smem > 48 * 1024) cudaFuncSetAttribute(paged_multimap_attention_kernel<ST, 1>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
    paged_multimap_attention_kernel<ST, 1><<<grid, kAttnThreads, smem, s>>>((ST*)out, out_stride, (const ST*)q, q_stride, (const ST*)kpool,
        (const ST*)vpool, tok_slot, tok_pos, block_table, max_blocks, H, G, D, Dv, scale, lambda, out_scale, eps, head_norm, page);
  }
  return check_cuda(cudaGetLastError(), "hyb_attention");
}

template <typename ST>
int launch_delta(void* out, long long out_stride, float* prep, float* o_raw, const void* proj, long long stride, const float* conv_w,
                 float* conv_state, float* state, const float* a_log, const float* dt_bias, const float* norm_w, const int* tok_entry,
                 const int* tok_pos, const int* entry_start, const int* entry_len, const int* entry_slot, const int* entry_pos0, int T, int E,
                 int H, int G, int D, int Dv, int taps, float unit_eps, float eps, cudaStream_t s) {
  const int C = 2 * G * D + H * Dv;
  const size_t smem = (size_t)C * sizeof(float);
  if (smem > 48 * 1024) cudaFuncSetAttribute(delta_prepare_kernel<ST>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
  delta_prepare_kernel<ST><<<T, 256, smem, s>>>(prep, (const ST*)proj, stride, conv_w, conv_state, a_log, dt_bias, tok_entry, tok_pos, entry_start,
                                                 entry_slot, H, G, D, Dv, taps, unit_eps);
  if (taps > 1)
    delta_conv_state_kernel<ST><<<dim3((C + 127) / 128, E), 128, 0, s>>>(conv_state, (const ST*)proj, stride, entry_start, entry_len, entry_slot,
                                                                          entry_pos0, C, taps);
  const int threads = ((Dv + 31) / 32) * 32;
  dim3 grid(E, H);
#define QS_SCAN(DP) delta_scan_kernel<DP><<<grid, threads, 0, s>>>(o_raw, prep, state, entry_start, entry_len, entry_slot, entry_pos0, H, G, D, Dv)
  if (D <= 16) QS_SCAN(16);
  else if (D <= 32) QS_SCAN(32);
  else if (D <= 64) QS_SCAN(64);
  else if (D <= 128) QS_SCAN(128);
  else QS_SCAN(256);
#undef QS_SCAN
  const int warps = T * H;
  delta_gate_out_kernel<ST><<<(warps + 3) / 4, 128, 0, s>>>((ST*)out, out_stride, o_raw, (const ST*)proj, stride, norm_w, T, H, G, D, Dv, eps);
  return check_cuda(cudaGetLastError(), "hyb_gated_delta");
}

}  // namespace
}  // namespace qs

using namespace qs;

#define QS_DT(dtype, CALL_BF16, CALL_F32)                                               \
  do {                                                                                  \
    if ((dtype) == QS_DTYPE_BF16) { CALL_BF16; }                                        \
    else if ((dtype) == QS_DTYPE_F32) { CALL_F32; }                                     \
    else return set_error(qs::QS_ERR_INVALID, "dtype must be QS_DTYPE_BF16 or QS_DTYPE_F32"); \
  } while (0)

extern "C" {

int qs_hyb_embed(float* out, const int32_t* tokens, const int32_t* prev, const void* table, const void* pair_table, int tokens_n, int width,
                 int buckets, int64_t mul_prev, int64_t mul_cur, int dtype, void* stream) {
  QS_REQUIRE(out && tokens && table, "hyb_embed: null tensor");
  QS_REQUIRE(pair_table == nullptr || (prev != nullptr && buckets > 0), "hyb_embed: the pair table needs previous tokens and buckets > 0");
  if (tokens_n == 0) return qs::QS_OK;
  cudaStream_t s = (cudaStream_t)stream;
  QS_DT(dtype,
        (embed_pair_kernel<__nv_bfloat16><<<tokens_n, 128, 0, s>>>(out, tokens, prev, (const __nv_bfloat16*)table, (const __nv_bfloat16*)pair_table,
                                                                    width, buckets, mul_prev, mul_cur)),
        (embed_pair_kernel<float><<<tokens_n, 128, 0, s>>>(out, tokens, prev, (const float*)table, (const float*)pair_table, width, buckets,
                                                           mul_prev, mul_cur)));
  return check_cuda(cudaGetLastError(), "hyb_embed");
}

int qs_hyb_rms_norm(void* out1, void* out2, const float* x, const float* w1, const float* w2, float offset, float eps, int tokens_n, int width,
                    int dtype, void* stream) {
  QS_REQUIRE(out1 && x && w1 && (out2 == nullptr || w2 != nullptr), "hyb_rms_norm: null tensor");
  if (tokens_n == 0) return qs::QS_OK;
  cudaStream_t s = (cudaStream_t)stream;
  const int threads = width >= 1024 ? 256 : 128;
  QS_DT(dtype,
        (rms_norm2_kernel<__nv_bfloat16><<<tokens_n, threads, 0, s>>>((__nv_bfloat16*)out1, (__nv_bfloat16*)out2, x, w1, w2, offset, eps, width)),
        (rms_norm2_kernel<float><<<tokens_n, threads, 0, s>>>((float*)out1, (float*)out2, x, w1, w2, offset, eps, width)));
  return check_cuda(cudaGetLastError(), "hyb_rms_norm");
}

int qs_hyb_residual_add(float* x, const void* y, int64_t n, int dtype, void* stream) {
  QS_REQUIRE(x && y, "hyb_residual_add: null tensor");
  if (n == 0) return qs::QS_OK;
  cudaStream_t s = (cudaStream_t)stream;
  const unsigned blocks = (unsigned)((n + 255) / 256);
  QS_DT(dtype, (residual_add_kernel<__nv_bfloat16><<<blocks, 256, 0, s>>>(x, (const __nv_bfloat16*)y, (size_t)n)),
        (residual_add_kernel<float><<<blocks, 256, 0, s>>>(x, (const float*)y, (size_t)n)));
  return check_cuda(cudaGetLastError(), "hyb_residual_add");
}

int qs_hyb_gelu_tanh_mul(void* out, int64_t out_stride, const void* in, int tokens_n, int ff, int dtype, void* stream) {
  QS_REQUIRE(out && in, "hyb_gelu_tanh_mul: null tensor");
  if (tokens_n == 0) return qs::QS_OK;
  cudaStream_t s = (cudaStream_t)stream;
  dim3 grid(tokens_n, (ff + 255) / 256);
  QS_DT(dtype, (gelu_tanh_mul_kernel<__nv_bfloat16><<<grid, 256, 0, s>>>((__nv_bfloat16*)out, out_stride, (const __nv_bfloat16*)in, ff)),
        (gelu_tanh_mul_kernel<float><<<grid, 256, 0, s>>>((float*)out, out_stride, (const float*)in, ff)));
  return check_cuda(cudaGetLastError(), "hyb_gelu_tanh_mul");
}

int qs_hyb_rope_append(void* proj, int64_t stride, const int32_t* tok_slot, const int32_t* tok_pos, const int32_t* block_table, int max_blocks,
                       void* kpool, void* vpool, const float* inv_freq, float amplitude, int tokens_n, int heads, int kv_heads, int maps,
                       int dim, int vdim, int rot_dims, int page_size, int dtype, void* stream) {
  QS_REQUIRE(proj && tok_slot && tok_pos && block_table && kpool && vpool && inv_freq, "hyb_rope_append: null tensor");
  QS_REQUIRE(rot_dims % 2 == 0 && rot_dims <= dim && heads % kv_heads == 0 && page_size > 0, "hyb_rope_append: bad head geometry");
  if (tokens_n == 0) return qs::QS_OK;
  cudaStream_t s = (cudaStream_t)stream;
  dim3 grid(tokens_n, heads + kv_heads);
  QS_DT(dtype,
        (rope_append_kernel<__nv_bfloat16><<<grid, 64, 0, s>>>((__nv_bfloat16*)proj, stride, tok_slot, tok_pos, block_table, max_blocks,
                                                                (__nv_bfloat16*)kpool, (__nv_bfloat16*)vpool, inv_freq, amplitude, heads, kv_heads,
                                                                maps, dim, vdim, rot_dims, page_size)),
        (rope_append_kernel<float><<<grid, 64, 0, s>>>((float*)proj, stride, tok_slot, tok_pos, block_table, max_blocks, (float*)kpool,
                                                        (float*)vpool, inv_freq, amplitude, heads, kv_heads, maps, dim, vdim, rot_dims, page_size)));
  return check_cuda(cudaGetLastError(), "hyb_rope_append");
}

int qs_hyb_attention(void* out, int64_t out_stride, const void* q, int64_t q_stride, const void* kpool, const void* vpool,
                     const int32_t* tok_slot, const int32_t* tok_pos, const int32_t* block_table, int max_blocks, int tokens_n, int heads,
                     int kv_heads, int maps, int dim, int vdim, float scale, float lambda, float out_scale, float eps, int head_norm,
                     int page_size, int dtype, void* stream) {
  QS_REQUIRE(out && q && kpool && vpool && tok_slot && tok_pos && block_table, "hyb_attention: null tensor");
  QS_REQUIRE(maps == 1 || maps == 2, "hyb_attention: 1 or 2 softmax maps per head");
  QS_REQUIRE(heads % kv_heads == 0 && vdim <= kAttnThreads * kAttnMaxV && page_size > 0, "hyb_attention: bad head geometry (vdim <= 512)");
  if (tokens_n == 0) return qs::QS_OK;
  cudaStream_t s = (cudaStream_t)stream;
  QS_DT(dtype,
        return launch_attention<__nv_bfloat16>(out, out_stride, q, q_stride, kpool, vpool, tok_slot, tok_pos, block_table, max_blocks, tokens_n,
                                               heads, kv_heads, maps, dim, vdim, scale, lambda, out_scale, eps, head_norm, page_size, s),
        return launch_attention<float>(out, out_stride, q, q_stride, kpool, vpool, tok_slot, tok_pos, block_table, max_blocks, tokens_n, heads,
                                       kv_heads, maps, dim, vdim, scale, lambda, out_scale, eps, head_norm, page_size, s));
}

int qs_hyb_gated_delta(void* out, int64_t out_stride, float* prep, float* o_raw, const void* proj, int64_t stride, const float* conv_w,
                       float* conv_state, float* state, const float* a_log, const float* dt_bias, const float* norm_w,
                       const int32_t* tok_entry, const int32_t* tok_pos, const int32_t* entry_start, const int32_t* entry_len,
                       const int32_t* entry_slot, const int32_t* entry_pos0, int tokens_n, int entries, int heads, int kv_heads, int dim,
                       int vdim, int taps, float unit_eps, float eps, int dtype, void* stream) {
  QS_REQUIRE(out && prep && o_raw && proj && conv_w && state && a_log && dt_bias && norm_w, "hyb_gated_delta: null tensor");
  QS_REQUIRE(tok_entry && tok_pos && entry_start && entry_len && entry_slot && entry_pos0, "hyb_gated_delta: null batch table");
  QS_REQUIRE(taps >= 1 && taps <= 17 && (taps == 1 || conv_state != nullptr), "hyb_gated_delta: 1..17 convolution taps");
  QS_REQUIRE(heads % kv_heads == 0 && dim <= 256 && vdim <= 1024, "hyb_gated_delta: dim <= 256, vdim <= 1024");
  if (tokens_n == 0) return qs::QS_OK;
  cudaStream_t s = (cudaStream_t)stream;
  QS_DT(dtype,
        return launch_delta<__nv_bfloat16>(out, out_stride, prep, o_raw, proj, stride, conv_w, conv_state, state, a_log, dt_bias, norm_w,
                                           tok_entry, tok_pos, entry_start, entry_len, entry_slot, entry_pos0, tokens_n, entries, heads,
                                           kv_heads, dim, vdim, taps, unit_eps, eps, s),
        return launch_delta<float>(out, out_stride, prep, o_raw, proj, stride, conv_w, conv_state, state, a_log, dt_bias, norm_w, tok_entry,
                                   tok_pos, entry_start, entry_len, entry_slot, entry_pos0, tokens_n, entries, heads, kv_heads, dim, vdim,
                                   taps, unit_eps, eps, s));
}

}  // extern "C"
