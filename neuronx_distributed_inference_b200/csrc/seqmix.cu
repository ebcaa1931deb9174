// Ragged sequence-mixer kernels: sum + RMS norm of an fp32 residual stream, short causal convolutions with carried inputs, the fused
// front half of a convolved-projection attention layer (convolution + row-wide q/k norm + partial interleaved rotation + paged cache
// write), soft-capped kept-prefix sliding-window attention over the paged cache, the Mamba-2 recurrence with a carried fp32 state,
// grouped RMS norm and the clamped gate product.  Norms, softmax, decays, step sizes and states are fp32; activations are bf16 or fp32
// (template parameter).  This file is compiled WITHOUT fast-math: tanh / exp / divisions are the accurate ones.
#include <cuda_bf16.h>
#include <math.h>

#include <algorithm>
#include <type_traits>

#include "common.cuh"
#include "seqmix.h"

namespace nxdi {
namespace {

template <typename T> __device__ __forceinline__ float ldf(const T* p);
template <> __device__ __forceinline__ float ldf<float>(const float* p) { return *p; }
template <> __device__ __forceinline__ float ldf<__nv_bfloat16>(const __nv_bfloat16* p) { return __bfloat162float(*p); }
template <typename T> __device__ __forceinline__ void stf(T* p, float v);
template <> __device__ __forceinline__ void stf<float>(float* p, float v) { *p = v; }
template <> __device__ __forceinline__ void stf<__nv_bfloat16>(__nv_bfloat16* p, float v) { *p = __float2bfloat16_rn(v); }

// sum over the block; every thread gets the result.  `red` holds 32 floats.
__device__ __forceinline__ float block_sum(float v, float* red) {
  v = warp_sum(v);
  const int lane = threadIdx.x & 31, w = threadIdx.x >> 5, nw = (blockDim.x + 31) >> 5;
  __syncthreads();
  if (lane == 0) red[w] = v;
  __syncthreads();
  float t = lane < nw ? red[lane] : 0.f;
  return warp_sum(t);
}

__device__ __forceinline__ float sigmoidf_acc(float x) { return 1.f / (1.f + expf(-x)); }

// ---- out = rms_unit(alpha * x + y) * (offset + w) ---------------------------------------------------------------------------
template <typename TY>
__global__ void __launch_bounds__(256) scaled_add_rmsnorm_kernel(const float* __restrict__ x, const TY* __restrict__ y,
                                                                 const float* __restrict__ w, float* __restrict__ out,
                                                                 __nv_bfloat16* __restrict__ out_lp, int W, float alpha, float eps,
                                                                 float offset) {
  __shared__ float red[32];
  const long long row = blockIdx.x;
  const float* xr = x + row * W;
  const TY* yr = y ? y + row * W : nullptr;
  float ss = 0.f;
  for (int c = threadIdx.x; c < W; c += blockDim.x) {
    float s = alpha * xr[c] + (yr ? ldf(yr + c) : 0.f);
    ss += s * s;
  }
  ss = block_sum(ss, red);
  const float r = 1.f / sqrtf(ss / (float)W + eps);
  for (int c = threadIdx.x; c < W; c += blockDim.x) {
    float s = alpha * xr[c] + (yr ? ldf(yr + c) : 0.f);
    float o = s * r * (w ? (w[c] + offset) : 1.f);
    out[row * W + c] = o;
    if (out_lp) out_lp[row * W + c] = __float2bfloat16_rn(o);
  }
}

// ---- short causal convolution with carried inputs ----------------------------------------------------------------------------
// input at window index i (i = t - K + 1 + j): i >= 0 -> u[b, i]; i < 0 -> carried row K - 1 + i of the line (zero when ctx == 0)
template <typename T>
__device__ __forceinline__ float conv_input(const T* u_row0, long long u_st, const T* st_line, int C, int K, int i, int c, bool has_ctx) {
  if (i >= 0) return ldf(u_row0 + (long long)i * u_st + c);
  return has_ctx ? ldf(st_line + (long long)(K - 1 + i) * C + c) : 0.f;
}

template <typename T>
__global__ void __launch_bounds__(256) short_conv_kernel(const T* __restrict__ u, long long u_sb, long long u_st,
                                                         const float* __restrict__ w, const float* __restrict__ bias,
                                                         const T* __restrict__ state, const int* __restrict__ lines,
                                                         const int* __restrict__ ctx_len, const int* __restrict__ q_len,
                                                         float* __restrict__ y, int T_, int C, int K, int silu) {
  const int b = blockIdx.z, t = blockIdx.x, c = blockIdx.y * blockDim.x + threadIdx.x;      // tokens on grid.x: no 65535 limit
  if (c >= C || t >= q_len[b]) return;
  const bool has_ctx = ctx_len[b] > 0;
  const T* u0 = u + (long long)b * u_sb;
  const T* sl = state + (long long)lines[b] * (K - 1) * C;
  float acc = bias ? bias[c] : 0.f;
  for (int j = 0; j < K; ++j) acc += w[(long long)c * K + j] * conv_input(u0, u_st, sl, C, K, t - K + 1 + j, c, has_ctx);
  if (silu) acc = acc * sigmoidf_acc(acc);
  y[((long long)b * T_ + t) * C + c] = acc;
}

template <typename T>
__global__ void __launch_bounds__(256) short_conv_update_kernel(const T* __restrict__ u, long long u_sb, long long u_st, T* __restrict__ state,
                                                                const int* __restrict__ lines, const int* __restrict__ ctx_len,
                                                                const int* __restrict__ q_len, int C, int K) {
  const int b = blockIdx.y, c = blockIdx.x * blockDim.x + threadIdx.x;
  const int n = q_len[b];
  if (c >= C || n <= 0) return;
  const bool has_ctx = ctx_len[b] > 0;
  const T* u0 = u + (long long)b * u_sb;
  T* sl = state + (long long)lines[b] * (K - 1) * C;
  float keep[SEQMIX_MAX_TAPS];
  // new row j = input at window index n - (K - 1) + j
#pragma unroll
  for (int j = 0; j < SEQMIX_MAX_TAPS - 1; ++j)
    if (j < K - 1) keep[j] = conv_input(u0, u_st, sl, C, K, n - (K - 1) + j, c, has_ctx);
#pragma unroll
  for (int j = 0; j < SEQMIX_MAX_TAPS - 1; ++j)
    if (j < K - 1) stf(sl + (long long)j * C + c, keep[j]);
}

// ---- convolution + row-wide q / k norm + partial interleaved rotation + paged cache write -------------------------------------
template <typename T>
__global__ void __launch_bounds__(256) conv_qknorm_rope_append_kernel(ConvQkParams p) {
  extern __shared__ float buf[];      // [Cq + Ck + Cv] convolved row
  __shared__ float red[32];
  const int b = blockIdx.y, t = blockIdx.x;
  if (t >= p.q_len[b]) return;
  const int Cq = p.n_q * p.D, Ck = p.n_kv * p.D, Cv = p.n_kv * p.Dv, C = Cq + Ck + Cv, K = p.K;
  const bool has_ctx = p.ctx_len[b] > 0;
  const T* u0 = (const T*)p.p + (long long)b * p.p_sb;
  const T* sl = (const T*)p.state + (long long)p.lines[b] * (K - 1) * C;
  float sq = 0.f, sk = 0.f;
  for (int c = threadIdx.x; c < C; c += blockDim.x) {
    float acc = 0.f;
    for (int j = 0; j < K; ++j) acc += p.conv_w[(long long)c * K + j] * conv_input(u0, p.p_st, sl, C, K, t - K + 1 + j, c, has_ctx);
    buf[c] = acc;
    if (c < Cq) sq += acc * acc;
    else if (c < Cq + Ck) sk += acc * acc;
  }
  sq = block_sum(sq, red);
  sk = block_sum(sk, red);
  // a null norm weight: that row is not normalised
  const float rq = p.q_norm_w ? 1.f / sqrtf(sq / (float)Cq + p.eps) : 1.f;
  const float rk = (Ck && p.k_norm_w) ? 1.f / sqrtf(sk / (float)Ck + p.eps) : 1.f;
  const long long tok = (long long)b * p.T + t;
  const float* cs = p.cos + tok * (p.R / 2);
  const float* sn = p.sin + tok * (p.R / 2);
  const int pos = p.ctx_len[b] + t;
  long long slot = 0;
  if (p.n_kv) slot = (long long)p.block_table[(long long)b * p.max_blocks + pos / p.page] * p.page + pos % p.page;
  T* qo = (T*)p.q_out + tok * Cq;
  T* ko = (T*)p.k_cache + slot * Ck;
  T* vo = (T*)p.v_cache + slot * Cv;
  for (int c = threadIdx.x; c < Cq + Ck; c += blockDim.x) {
    const bool isq = c < Cq;
    const int cc = isq ? c : c - Cq;
    const float r = isq ? rq : rk;
    const float* nw = isq ? p.q_norm_w : p.k_norm_w;
    const int d = cc % p.D;
    float self = buf[c] * r * (nw ? nw[cc] : 1.f);
    if (d < p.R) {
      const float other = buf[c ^ 1] * r * (nw ? nw[cc ^ 1] : 1.f);
      const float co = cs[d >> 1], si = sn[d >> 1];
      self = (d & 1) ? (self * co + other * si) : (self * co - other * si);
    }
    stf((isq ? qo : ko) + cc, self);
  }
  for (int c = threadIdx.x; c < Cv; c += blockDim.x) stf(vo + c, buf[Cq + Ck + c]);
}

// Two channels per thread (every rotation pair, 4- or 8-byte accesses): taken when value size and row strides are even.
template <typename T> __device__ __forceinline__ float2 ld2(const T* p);
template <> __device__ __forceinline__ float2 ld2<float>(const float* p) { return *reinterpret_cast<const float2*>(p); }
template <> __device__ __forceinline__ float2 ld2<__nv_bfloat16>(const __nv_bfloat16* p) {
  return __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(p));
}
template <typename T> __device__ __forceinline__ void st2(T* p, float a, float b);
template <> __device__ __forceinline__ void st2<float>(float* p, float a, float b) { *reinterpret_cast<float2*>(p) = make_float2(a, b); }
template <> __device__ __forceinline__ void st2<__nv_bfloat16>(__nv_bfloat16* p, float a, float b) {
  *reinterpret_cast<__nv_bfloat162*>(p) = __floats2bfloat162_rn(a, b);
}

template <typename T>
__global__ void __launch_bounds__(256) conv_qknorm_rope_append_pair_kernel(ConvQkParams p) {
  extern __shared__ float buf[];      // [Cq + Ck + Cv] convolved row
  __shared__ float red[32];
  const int b = blockIdx.y, t = blockIdx.x;
  if (t >= p.q_len[b]) return;
  const int Cq = p.n_q * p.D, Ck = p.n_kv * p.D, Cv = p.n_kv * p.Dv, C = Cq + Ck + Cv, K = p.K;
  const bool has_ctx = p.ctx_len[b] > 0;
  const T* u0 = (const T*)p.p + (long long)b * p.p_sb;
  const T* sl = (const T*)p.state + (long long)p.lines[b] * (K - 1) * C;
  float sq = 0.f, sk = 0.f;
  for (int c = 2 * threadIdx.x; c < C; c += 2 * blockDim.x) {
    float a0 = 0.f, a1 = 0.f;
    for (int j = 0; j < K; ++j) {
      const int i = t - K + 1 + j;
      float2 v = make_float2(0.f, 0.f);
      if (i >= 0) v = ld2(u0 + (long long)i * p.p_st + c);
      else if (has_ctx) v = ld2(sl + (long long)(K - 1 + i) * C + c);
      a0 += p.conv_w[(long long)c * K + j] * v.x;
      a1 += p.conv_w[(long long)(c + 1) * K + j] * v.y;
    }
    buf[c] = a0;
    buf[c + 1] = a1;
    const float ss = a0 * a0 + a1 * a1;
    if (c < Cq) sq += ss;
    else if (c < Cq + Ck) sk += ss;
  }
  sq = block_sum(sq, red);
  sk = block_sum(sk, red);
  // a null norm weight: that row is not normalised
  const float rq = p.q_norm_w ? 1.f / sqrtf(sq / (float)Cq + p.eps) : 1.f;
  const float rk = (Ck && p.k_norm_w) ? 1.f / sqrtf(sk / (float)Ck + p.eps) : 1.f;
  const long long tok = (long long)b * p.T + t;
  const float* cs = p.cos + tok * (p.R / 2);
  const float* sn = p.sin + tok * (p.R / 2);
  const int pos = p.ctx_len[b] + t;
  long long slot = 0;
  if (p.n_kv) slot = (long long)p.block_table[(long long)b * p.max_blocks + pos / p.page] * p.page + pos % p.page;
  T* qo = (T*)p.q_out + tok * Cq;
  T* ko = (T*)p.k_cache + slot * Ck;
  T* vo = (T*)p.v_cache + slot * Cv;
  for (int c = 2 * threadIdx.x; c < Cq + Ck; c += 2 * blockDim.x) {
    const bool isq = c < Cq;
    const int cc = isq ? c : c - Cq;
    const float r = isq ? rq : rk;
    const float* nw = isq ? p.q_norm_w : p.k_norm_w;
    const int d = cc % p.D;
    float a = buf[c] * r * (nw ? nw[cc] : 1.f), bb = buf[c + 1] * r * (nw ? nw[cc + 1] : 1.f);
    if (d < p.R) {
      const float co = cs[d >> 1], si = sn[d >> 1];
      const float ra = a * co - bb * si, rb = bb * co + a * si;
      a = ra;
      bb = rb;
    }
    st2((isq ? qo : ko) + cc, a, bb);
  }
  for (int c = 2 * threadIdx.x; c < Cv; c += 2 * blockDim.x) st2(vo + c, buf[Cq + Ck + c], buf[Cq + Ck + c + 1]);
}

// ---- soft-capped kept-prefix sliding-window attention over the paged cache ---------------------------------------------------
template <typename T> struct Vec;                     // 16-byte vectors of the activation type
template <> struct Vec<float> { static constexpr int N = 4; };
template <> struct Vec<__nv_bfloat16> { static constexpr int N = 8; };

template <typename T>
__device__ __forceinline__ float dot_row(const float* qs, const T* k, int D, bool vec_ok) {
  float s = 0.f;
  if (vec_ok) {
    constexpr int N = Vec<T>::N;
    for (int d = 0; d < D; d += N) {
      const uint4 raw = *reinterpret_cast<const uint4*>(k + d);
      if constexpr (N == 4) {
        s += qs[d] * __uint_as_float(raw.x) + qs[d + 1] * __uint_as_float(raw.y) + qs[d + 2] * __uint_as_float(raw.z) +
             qs[d + 3] * __uint_as_float(raw.w);
      } else {
        s += qs[d] * bf16lo(raw.x) + qs[d + 1] * bf16hi(raw.x) + qs[d + 2] * bf16lo(raw.y) + qs[d + 3] * bf16hi(raw.y) +
             qs[d + 4] * bf16lo(raw.z) + qs[d + 5] * bf16hi(raw.z) + qs[d + 6] * bf16lo(raw.w) + qs[d + 7] * bf16hi(raw.w);
      }
    }
  } else {
    for (int d = 0; d < D; ++d) s += qs[d] * ldf(k + d);
  }
  return s;
}

constexpr int ATT_WARPS = 4;
constexpr int ATT_VPL = SEQMIX_MAX_VDIM / 32;      // value channels per lane

// SPLIT = false: warp w of a block owns query blockIdx.x * 4 + w.  SPLIT = true: the four warps share query blockIdx.x, warp w takes
// key chunks w, w + 4, ... and the partial (max, sum, acc) are merged through shared memory (few queries, long ranges: decode).
template <typename T, bool SPLIT>
__global__ void __launch_bounds__(SPLIT ? 1024 : ATT_WARPS * 32) paged_window_attention_kernel(WindowAttnParams p) {
  extern __shared__ float smem[];      // [warps][D] scaled queries, then (SPLIT) [warps][Dv + 2] partials
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31, nwarps = blockDim.x >> 5;
  const long long nq = (long long)p.B * p.T * p.Hq;
  const long long qi = SPLIT ? (long long)blockIdx.x : (long long)blockIdx.x * nwarps + warp;
  const bool in_range = qi < nq;
  const int h = in_range ? (int)(qi % p.Hq) : 0;
  const long long tok = in_range ? qi / p.Hq : 0;
  const int b = (int)(tok / p.T), t = (int)(tok % p.T);
  const bool live = in_range && t < p.q_len[b];
  if (!SPLIT && !live) return;
  if (SPLIT && !live) return;          // uniform over the block: all warps share the query
  const int D = p.D, Dv = p.Dv, g = h / (p.Hq / p.G);
  float* qs = smem + warp * D;
  const T* qrow = (const T*)p.q + qi * D;
  const float qscale = p.head_scale ? p.scale * p.head_scale[h] : p.scale;
  for (int d = lane; d < D; d += 32) qs[d] = ldf(qrow + d) * qscale;
  __syncwarp();
  const int pos = p.ctx_len[b] + t;
  // visible keys: a window that ends at the query, or the query's chunk up to the query
  const int lo = p.chunk > 0 ? (pos / p.chunk) * p.chunk : (p.window > 0 ? max(pos - p.window + 1, 0) : 0);
  const int nA = p.window > 0 ? min(p.keep_first, lo) : 0;       // kept first tokens that the window no longer covers
  const int n = nA + (pos - lo + 1);
  const float slope = p.slopes ? p.slopes[h] : 0.f;
  const int* table = p.block_table + (long long)b * p.max_blocks;
  const bool kvec = ((D * (int)sizeof(T)) % 16) == 0;
  const T* kc = (const T*)p.k_cache;
  const T* vc = (const T*)p.v_cache;
  float m = -INFINITY, l = 0.f, acc[ATT_VPL];
#pragma unroll
  for (int i = 0; i < ATT_VPL; ++i) acc[i] = 0.f;
  // value rows whose byte size is 16 * 2^k (k <= 5) are read as 16-byte pieces, LPR lanes per row
  constexpr int VN = Vec<T>::N;
  const int LPR = Dv / VN;
  const bool vvec = Dv % VN == 0 && LPR >= 1 && LPR <= 32 && (LPR & (LPR - 1)) == 0 && (p.v_rs * (long long)sizeof(T)) % 16 == 0;
  const int sub = vvec ? lane / LPR : 0, piece = vvec ? lane % LPR : 0;
  float accv[VN];
#pragma unroll
  for (int e = 0; e < VN; ++e) accv[e] = 0.f;
  const int nchunks = (n + 31) / 32;
  for (int ch = SPLIT ? warp : 0; ch < nchunks; ch += SPLIT ? nwarps : 1) {
    const int idx = ch * 32 + lane;
    float s = -INFINITY;
    long long row = 0;
    if (idx < n) {
      const int j = idx < nA ? idx : lo + (idx - nA);
      row = ((long long)table[j / p.page] * p.page + j % p.page) * p.G + g;
      s = dot_row(qs, kc + row * D, D, kvec);
      if (p.softcap > 0.f) s = p.softcap * tanhf(s / p.softcap);
      s -= slope * (float)(pos - j);
    }
    const float m_new = fmaxf(m, warp_max(s));
    const float corr = expf(m - m_new);          // m = -inf on the first chunk: exp(-inf) = 0
    const float pj = idx < n ? expf(s - m_new) : 0.f;
    l = l * corr + warp_sum(pj);
#pragma unroll
    for (int i = 0; i < ATT_VPL; ++i) acc[i] *= corr;
    m = m_new;
    const int cnt = min(32, n - ch * 32);
    if (vvec) {
      // LPR lanes read one value row as 16-byte pieces: 32 / LPR keys per load instruction
#pragma unroll
      for (int e = 0; e < VN; ++e) accv[e] *= corr;
      for (int jj = 0; jj < cnt; jj += 32 / LPR) {
        const int src = jj + sub;
        const float pw = __shfl_sync(0xffffffffu, pj, src & 31);
        const long long r = __shfl_sync(0xffffffffu, row, src & 31);
        if (src < cnt) {
          const uint4 raw = *reinterpret_cast<const uint4*>(vc + r * p.v_rs + piece * VN);
          if constexpr (VN == 4) {
            accv[0] += pw * __uint_as_float(raw.x); accv[1] += pw * __uint_as_float(raw.y);
            accv[2] += pw * __uint_as_float(raw.z); accv[3] += pw * __uint_as_float(raw.w);
          } else {
            accv[0] += pw * bf16lo(raw.x); accv[1] += pw * bf16hi(raw.x); accv[2] += pw * bf16lo(raw.y); accv[3] += pw * bf16hi(raw.y);
            accv[4] += pw * bf16lo(raw.z); accv[5] += pw * bf16hi(raw.z); accv[6] += pw * bf16lo(raw.w); accv[7] += pw * bf16hi(raw.w);
          }
        }
      }
    } else {
      for (int jj = 0; jj < cnt; ++jj) {
        const float pw = __shfl_sync(0xffffffffu, pj, jj);
        const long long r = __shfl_sync(0xffffffffu, row, jj);
        const T* vrow = vc + r * p.v_rs;
#pragma unroll
        for (int i = 0; i < ATT_VPL; ++i) {
          const int dv = lane + 32 * i;
          if (dv < Dv) acc[i] += pw * ldf(vrow + dv);
        }
      }
    }
  }
  if (vvec) {
    // fold the lanes that shared a piece, then hand the row over in the (lane + 32 i) layout the epilogue uses
    for (int o = LPR; o < 32; o <<= 1)
#pragma unroll
      for (int e = 0; e < VN; ++e) accv[e] += __shfl_xor_sync(0xffffffffu, accv[e], o);
    float* mine = smem + nwarps * D + warp * (Dv + 2);
    if (sub == 0)
#pragma unroll
      for (int e = 0; e < VN; ++e) mine[piece * VN + e] = accv[e];
    __syncwarp();
#pragma unroll
    for (int i = 0; i < ATT_VPL; ++i) {
      const int dv = lane + 32 * i;
      acc[i] = dv < Dv ? mine[dv] : 0.f;
    }
    __syncwarp();
  }
  if (SPLIT) {
    float* part = smem + nwarps * D + warp * (Dv + 2);
#pragma unroll
    for (int i = 0; i < ATT_VPL; ++i) {
      const int dv = lane + 32 * i;
      if (dv < Dv) part[dv] = acc[i];
    }
    if (lane == 0) { part[Dv] = m; part[Dv + 1] = l; }
    __syncthreads();
    if (warp != 0) return;
    float M = -INFINITY;
    for (int w = 0; w < nwarps; ++w) M = fmaxf(M, smem[nwarps * D + w * (Dv + 2) + Dv]);
    l = 0.f;
#pragma unroll
    for (int i = 0; i < ATT_VPL; ++i) acc[i] = 0.f;
    for (int w = 0; w < nwarps; ++w) {
      const float* pw = smem + nwarps * D + w * (Dv + 2);
      const float f = pw[Dv] == -INFINITY ? 0.f : expf(pw[Dv] - M);
      l += pw[Dv + 1] * f;
#pragma unroll
      for (int i = 0; i < ATT_VPL; ++i) {
        const int dv = lane + 32 * i;
        if (dv < Dv) acc[i] += pw[dv] * f;
      }
    }
    m = M;
  }
  if (p.sinks) l += expf(p.sinks[h] - m);      // the sink: one more term of the denominator, no value (a live query sees itself: m is finite)
  const float inv = 1.f / l;
  T* orow = (T*)p.out + qi * Dv;
  const T* grow = p.gate ? (const T*)p.gate + (long long)b * p.g_sb + (long long)t * p.g_st + (p.gate_per_head ? (long long)h : (long long)h * Dv)
                         : nullptr;
  const float head_gate = (grow && p.gate_per_head) ? sigmoidf_acc(ldf(grow)) : 1.f;
#pragma unroll
  for (int i = 0; i < ATT_VPL; ++i) {
    const int dv = lane + 32 * i;
    if (dv < Dv) {
      float o = acc[i] * inv * head_gate;
      if (grow && !p.gate_per_head) o *= sigmoidf_acc(ldf(grow + dv));
      stf(orow + dv, o);
    }
  }
}

// ---- the same attention on tensor cores (bf16, head sizes 64 / 128): prompt portions ------------------------------------------
// Block = 64 queries of one (row, head), 4 warps x 16 query rows.  Keys and values come in tiles of 64 from the paged cache into
// shared memory; S = Q K^T and O += P V run on mma.sync m16n8k16 with fp32 accumulators; scale, soft cap, mask and the online
// softmax are fp32 on the accumulator fragments; P is rounded to bf16 for the second product.  Tiles cover the kept first tokens
// that the block's window no longer reaches, then the window itself; the per-element mask is the exact visibility rule.
constexpr int MMA_MT = 64, MMA_KT = 64;

__device__ __forceinline__ float tanh_fast(float x) { return 1.f - __fdividef(2.f, __expf(2.f * x) + 1.f); }

// VPREFIX: the value of a key is the first DV channels of its key row (latent caches): the key tile in shared memory serves both products.
template <int D, int DV, bool VPREFIX>
__global__ void __launch_bounds__(128, (D + DV <= 256) ? 3 : 2) paged_window_attention_mma_kernel(WindowAttnParams p) {
  constexpr int KS = D + 8, VS = VPREFIX ? KS : DV + 8, STAGE = MMA_KT * (VPREFIX ? KS : KS + VS);
  extern __shared__ __align__(16) unsigned char mma_smem[];       // two stages of [64][KS] keys + [64][VS] values
  __nv_bfloat16* stage0 = reinterpret_cast<__nv_bfloat16*>(mma_smem);
  const int h = blockIdx.y, b = blockIdx.z, t0 = blockIdx.x * MMA_MT;
  const int qn = p.q_len[b];
  if (t0 >= qn) return;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31, gid = lane >> 2, tig = lane & 3;
  const int g = h / (p.Hq / p.G), ctx = p.ctx_len[b];
  const int r0 = t0 + warp * 16 + gid, r1 = r0 + 8;            // this thread's two query rows (token index in the row of the batch)
  const int pos0 = ctx + r0, pos1 = ctx + r1;
  uint32_t qa[D / 16][4];
  {
    const __nv_bfloat16* qb = (const __nv_bfloat16*)p.q + ((long long)b * p.T * p.Hq + h) * D;
#pragma unroll
    for (int ks = 0; ks < D / 16; ++ks) {
      const int col = ks * 16 + tig * 2;
      qa[ks][0] = r0 < p.T ? *reinterpret_cast<const uint32_t*>(qb + (long long)r0 * p.Hq * D + col) : 0u;
      qa[ks][1] = r1 < p.T ? *reinterpret_cast<const uint32_t*>(qb + (long long)r1 * p.Hq * D + col) : 0u;
      qa[ks][2] = r0 < p.T ? *reinterpret_cast<const uint32_t*>(qb + (long long)r0 * p.Hq * D + col + 8) : 0u;
      qa[ks][3] = r1 < p.T ? *reinterpret_cast<const uint32_t*>(qb + (long long)r1 * p.Hq * D + col + 8) : 0u;
    }
  }
  float o[DV / 8][4];
#pragma unroll
  for (int i = 0; i < DV / 8; ++i) o[i][0] = o[i][1] = o[i][2] = o[i][3] = 0.f;
  float m0 = -INFINITY, m1 = -INFINITY, l0 = 0.f, l1 = 0.f;
  const int p_first = ctx + t0, p_last = ctx + min(t0 + MMA_MT, qn) - 1;
  const int lo = p.chunk > 0 ? (p_first / p.chunk) * p.chunk : (p.window > 0 ? max(p_first - p.window + 1, 0) : 0);
  const int nA = p.window > 0 ? min(p.keep_first, lo) : 0;
  const float slope = p.slopes ? p.slopes[h] : 0.f;
  const float hscale = p.head_scale ? p.scale * p.head_scale[h] : p.scale;
  const int* table = p.block_table + (long long)b * p.max_blocks;
  const __nv_bfloat16* kc = (const __nv_bfloat16*)p.k_cache;
  const __nv_bfloat16* vc = (const __nv_bfloat16*)p.v_cache;
  const int ntA = (nA + MMA_KT - 1) / MMA_KT, ntB = (p_last + 1 - lo + MMA_KT - 1) / MMA_KT, ntiles = ntA + ntB;
  const float inv_cap = p.softcap > 0.f ? 1.f / p.softcap : 0.f;
  const int page_shift = (p.page & (p.page - 1)) == 0 ? __ffs(p.page) - 1 : -1;
  const int warp_pos_lo = ctx + t0 + warp * 16, warp_pos_hi = warp_pos_lo + 15;
  // tile i covers keys [j0, min(j0 + 64, end)): first the kept tokens below the window, then the window
  auto tile_range = [&](int i, int& j0, int& end) {
    if (i < ntA) { j0 = i * MMA_KT; end = nA; }
    else { j0 = lo + (i - ntA) * MMA_KT; end = p_last + 1; }
  };
  // all copies of a tile are issued back to back (16-byte cp.async, zero fill past `end`), one commit group per tile
  auto load_tile = [&](int i) {
    int j0, end;
    tile_range(i, j0, end);
    __nv_bfloat16* Kd = stage0 + (i & 1) * STAGE;
    __nv_bfloat16* Vd = VPREFIX ? Kd : Kd + MMA_KT * KS;
    // every copy is independent of the others (addresses from the block table, no carried state), so all of them are in flight at
    // once; pages of 2^k tokens (the usual case) are located with a shift and a mask instead of a division
    auto copy_rows = [&](const __nv_bfloat16* cache, long long rs, __nv_bfloat16* dst0, auto Wc, auto LDc) {
      constexpr int W = decltype(Wc)::value, LD = decltype(LDc)::value, cpr = W / 8;
#pragma unroll
      for (int k = 0; k < MMA_KT * cpr / 128; ++k) {
        const int c = threadIdx.x + 128 * k, r = c / cpr, ch = c % cpr, j = j0 + r, jj = min(j, end - 1);
        const int pi = page_shift >= 0 ? (jj >> page_shift) : jj / p.page, po = jj - pi * p.page;
        const long long row = ((long long)table[pi] * p.page + po) * p.G + g;
        const uint32_t dst = (uint32_t)__cvta_generic_to_shared(dst0 + r * LD + ch * 8);
        const int nbytes = j < end ? 16 : 0;
        asm volatile("cp.async.cg.shared.global [%0], [%1], 16, %2;" ::"r"(dst), "l"(cache + row * rs + ch * 8), "r"(nbytes));
      }
    };
    copy_rows(kc, (long long)D, Kd, std::integral_constant<int, D>{}, std::integral_constant<int, KS>{});
    if constexpr (!VPREFIX) copy_rows(vc, p.v_rs, Vd, std::integral_constant<int, DV>{}, std::integral_constant<int, VS>{});
    asm volatile("cp.async.commit_group;");
  };
  load_tile(0);
  for (int i = 0; i < ntiles; ++i) {
    if (i + 1 < ntiles) {
      load_tile(i + 1);                   // lands while tile i is computed
      asm volatile("cp.async.wait_group 1;");
    } else {
      asm volatile("cp.async.wait_group 0;");
    }
    __syncthreads();
    int j0, end;
    tile_range(i, j0, end);
    const __nv_bfloat16* Ks = stage0 + (i & 1) * STAGE;
    const uint32_t vs_base = (uint32_t)__cvta_generic_to_shared(VPREFIX ? Ks : Ks + MMA_KT * KS);
    {
      float sc[MMA_KT / 8][4];
#pragma unroll
      for (int nt = 0; nt < MMA_KT / 8; ++nt) sc[nt][0] = sc[nt][1] = sc[nt][2] = sc[nt][3] = 0.f;
#pragma unroll
      for (int ks = 0; ks < D / 16; ++ks)
#pragma unroll
        for (int nt = 0; nt < MMA_KT / 8; ++nt) {
          const __nv_bfloat16* kp = Ks + (nt * 8 + gid) * KS + ks * 16 + tig * 2;
          const uint32_t bb[2] = {*reinterpret_cast<const uint32_t*>(kp), *reinterpret_cast<const uint32_t*>(kp + 8)};
          mma_bf16_16816(sc[nt], qa[ks], bb);
        }
      // a tile that every row of this warp sees completely needs no mask
      const bool full = j0 + MMA_KT <= end && j0 + MMA_KT - 1 <= warp_pos_lo &&
                        (p.window <= 0 || warp_pos_hi - j0 < p.window || j0 + MMA_KT <= p.keep_first) &&
                        (p.chunk <= 0 || j0 / p.chunk == warp_pos_hi / p.chunk);
      float mx0 = -INFINITY, mx1 = -INFINITY;
#pragma unroll
      for (int nt = 0; nt < MMA_KT / 8; ++nt)
#pragma unroll
        for (int e = 0; e < 4; ++e) {
          float v = sc[nt][e] * hscale;
          if (p.softcap > 0.f) v = p.softcap * tanh_fast(v * inv_cap);
          const int j = j0 + nt * 8 + tig * 2 + (e & 1);
          const int pos = (e < 2) ? pos0 : pos1;
          v -= slope * (float)(pos - j);
          if (!full) {
            const bool see = j < end && j <= pos && (p.window <= 0 || pos - j < p.window || j < p.keep_first) &&
                             (p.chunk <= 0 || j / p.chunk == pos / p.chunk);
            v = see ? v : -INFINITY;
          }
          sc[nt][e] = v;
          if (e < 2) mx0 = fmaxf(mx0, v); else mx1 = fmaxf(mx1, v);
        }
      mx0 = fmaxf(mx0, __shfl_xor_sync(0xffffffffu, mx0, 1));
      mx0 = fmaxf(mx0, __shfl_xor_sync(0xffffffffu, mx0, 2));
      mx1 = fmaxf(mx1, __shfl_xor_sync(0xffffffffu, mx1, 1));
      mx1 = fmaxf(mx1, __shfl_xor_sync(0xffffffffu, mx1, 2));
      const float n0 = fmaxf(m0, mx0), n1 = fmaxf(m1, mx1);
      const float base0 = n0 == -INFINITY ? 0.f : n0, base1 = n1 == -INFINITY ? 0.f : n1;
      const float c0 = m0 == -INFINITY ? 0.f : __expf(m0 - base0), c1 = m1 == -INFINITY ? 0.f : __expf(m1 - base1);
      m0 = n0; m1 = n1;
      float s0 = 0.f, s1 = 0.f;
      uint32_t pa[MMA_KT / 16][4];
#pragma unroll
      for (int nt = 0; nt < MMA_KT / 8; ++nt) {
        const float e0 = __expf(sc[nt][0] - base0), e1 = __expf(sc[nt][1] - base0);
        const float e2 = __expf(sc[nt][2] - base1), e3 = __expf(sc[nt][3] - base1);
        s0 += e0 + e1;
        s1 += e2 + e3;
        pa[nt >> 1][(nt & 1) * 2] = pack_bf16(e0, e1);
        pa[nt >> 1][(nt & 1) * 2 + 1] = pack_bf16(e2, e3);
      }
      l0 = l0 * c0 + s0;
      l1 = l1 * c1 + s1;
#pragma unroll
      for (int i2 = 0; i2 < DV / 8; ++i2) { o[i2][0] *= c0; o[i2][1] *= c0; o[i2][2] *= c1; o[i2][3] *= c1; }
#pragma unroll
      for (int kk = 0; kk < MMA_KT / 16; ++kk)
#pragma unroll
        for (int nv = 0; nv < DV / 8; nv += 2) {
          // four 8x8 blocks of V (keys kk*16 .. +15, value channels nv*8 .. +15), transposed on load: B fragments of two n-tiles
          const int row = kk * 16 + (lane & 7) + ((lane >> 3) & 1) * 8, col = (nv + (lane >> 4)) * 8;
          const uint32_t addr = vs_base + (uint32_t)((row * VS + col) * 2);
          uint32_t v0, v1, v2, v3;
          asm volatile("ldmatrix.sync.aligned.m8n8.x4.trans.shared.b16 {%0,%1,%2,%3}, [%4];" : "=r"(v0), "=r"(v1), "=r"(v2), "=r"(v3) : "r"(addr));
          const uint32_t ba[2] = {v0, v1}, bb[2] = {v2, v3};
          mma_bf16_16816(o[nv], pa[kk], ba);
          mma_bf16_16816(o[nv + 1], pa[kk], bb);
        }
    }
    __syncthreads();                      // the stage is free for tile i + 2
  }
  l0 += __shfl_xor_sync(0xffffffffu, l0, 1);
  l0 += __shfl_xor_sync(0xffffffffu, l0, 2);
  l1 += __shfl_xor_sync(0xffffffffu, l1, 1);
  l1 += __shfl_xor_sync(0xffffffffu, l1, 2);
  if (p.sinks) {                             // rows past q_len have m = -inf and are never stored
    const float sk = p.sinks[h];
    l0 += __expf(sk - m0);
    l1 += __expf(sk - m1);
  }
  float i0 = 1.f / l0, i1 = 1.f / l1;
  __nv_bfloat16* ob = (__nv_bfloat16*)p.out + ((long long)b * p.T * p.Hq + h) * DV;
  const __nv_bfloat16* gb = (p.gate && !p.gate_per_head) ? (const __nv_bfloat16*)p.gate + (long long)b * p.g_sb + (long long)h * DV : nullptr;
  if (p.gate && p.gate_per_head) {
    const __nv_bfloat16* gh = (const __nv_bfloat16*)p.gate + (long long)b * p.g_sb + h;
    if (r0 < qn) i0 *= sigmoidf_acc(__bfloat162float(gh[(long long)r0 * p.g_st]));
    if (r1 < qn) i1 *= sigmoidf_acc(__bfloat162float(gh[(long long)r1 * p.g_st]));
  }
#pragma unroll
  for (int nv = 0; nv < DV / 8; ++nv) {
    const int col = nv * 8 + tig * 2;
    if (r0 < qn) {
      float a = o[nv][0] * i0, c = o[nv][1] * i0;
      if (gb) {
        a *= sigmoidf_acc(__bfloat162float(gb[(long long)r0 * p.g_st + col]));
        c *= sigmoidf_acc(__bfloat162float(gb[(long long)r0 * p.g_st + col + 1]));
      }
      *reinterpret_cast<uint32_t*>(ob + (long long)r0 * p.Hq * DV + col) = pack_bf16(a, c);
    }
    if (r1 < qn) {
      float a = o[nv][2] * i1, c = o[nv][3] * i1;
      if (gb) {
        a *= sigmoidf_acc(__bfloat162float(gb[(long long)r1 * p.g_st + col]));
        c *= sigmoidf_acc(__bfloat162float(gb[(long long)r1 * p.g_st + col + 1]));
      }
      *reinterpret_cast<uint32_t*>(ob + (long long)r1 * p.Hq * DV + col) = pack_bf16(a, c);
    }
  }
}

// ---- Mamba-2 recurrence with a carried state ----------------------------------------------------------------------------------
// Block = one (row, head, 16 head channels); 8 lanes split the state axis of a channel and hold their share of S in registers.  Time
// runs in batches of 16 steps: the B / C / x / dt / z values of batch r + 1 are fetched into registers while batch r is computed out
// of shared memory, so the global-load latency is paid once per sequence instead of once per batch.
constexpr int SCAN_PT = 16;      // head channels per block
constexpr int SCAN_NS = 8;       // lanes that split the state axis for one channel
constexpr int SCAN_TT = 16;      // time steps staged per batch
constexpr int SCAN_THREADS = SCAN_PT * SCAN_NS;

// NB = ceil(N / 128): state values per lane = 16 * NB, staged B / C values per thread and batch = 16 * NB
template <typename T, int NB>
__global__ void __launch_bounds__(SCAN_THREADS, NB == 1 ? 4 : 2) ssd_scan_kernel(SsdScanParams p) {
  extern __shared__ float sm[];
  constexpr int NPT = 16 * NB;             // state values per lane: n = ns * NPT + i
  constexpr int NP = 160 * NB;             // padded row of staged B / C: 4 floats after every 16, so that the 8 lanes' float4 reads miss each other
  const int N = p.N, P = p.P;
  float* Bs = sm;                          // [TT][NP], zero past N
  float* Cs = Bs + SCAN_TT * NP;           // [TT][NP]
  float* xs = Cs + SCAN_TT * NP;           // [TT][PT]
  float* ys = xs + SCAN_TT * SCAN_PT;      // [TT][PT]
  float* zs = ys + SCAN_TT * SCAN_PT;      // [TT][PT]
  float* dts = zs + SCAN_TT * SCAN_PT;     // [TT]
  float* dAs = dts + SCAN_TT;              // [TT]
  const int b = blockIdx.z, h = blockIdx.y, p0 = blockIdx.x * SCAN_PT;
  const int n_tok = p.q_len[b];
  if (n_tok <= 0) return;
  const int tid = threadIdx.x, pl = tid / SCAN_NS, ns = tid % SCAN_NS;
  const int pc = p0 + pl;                  // this thread's head channel
  const bool pok = pc < P;
  const int g = h / (p.nh / p.G);
  const int inner = p.nh * P, Cd = inner + 2 * p.G * N;
  float* Sg = p.state + ((long long)p.lines[b] * p.nh + h) * N * P;
  float S[NPT];
  const bool has_ctx = p.ctx_len[b] > 0;
#pragma unroll
  for (int i = 0; i < NPT; ++i) {
    const int n = ns * NPT + i;
    S[i] = (has_ctx && pok && n < N) ? Sg[(long long)n * P + pc] : 0.f;
  }
  const float negA = -expf(p.A_log[h]), dtb = p.dt_bias[h], Dh = p.D_skip[h];
  const float* xrow = p.xBC + (long long)b * p.T * Cd;
  const T* dtp = (const T*)p.dt_raw + (long long)b * p.dt_sb + h;
  const T* zp = (const T*)p.z + (long long)b * p.z_sb + h * P;
  // staging registers: element (t, n) with n = tid + 128 * k for B / C, element i = tid + 128 * k of the [TT][PT] tile for x / z
  float rb[NPT], rc[NPT], rx[2], rz[2], rdt = 0.f;
  auto fetch = [&](int t0) {
    const int tt = min(SCAN_TT, n_tok - t0);
#pragma unroll
    for (int t = 0; t < SCAN_TT; ++t)
#pragma unroll
      for (int k = 0; k < NB; ++k) {
        const int n = tid + SCAN_THREADS * k;
        const bool ok = t < tt && n < N;
        const float* r = xrow + (long long)(t0 + t) * Cd + inner + g * N + n;
        rb[t * NB + k] = ok ? r[0] : 0.f;
        rc[t * NB + k] = ok ? r[p.G * N] : 0.f;
      }
#pragma unroll
    for (int k = 0; k < 2; ++k) {
      const int i = tid + SCAN_THREADS * k, t = i / SCAN_PT, c = p0 + i % SCAN_PT;
      const bool ok = t < tt && c < P;
      rx[k] = ok ? xrow[(long long)(t0 + t) * Cd + h * P + c] : 0.f;
      rz[k] = ok ? ldf(zp + (long long)(t0 + t) * p.z_st + c) : 0.f;
    }
    rdt = tid < tt ? ldf(dtp + (long long)(t0 + tid) * p.dt_st) : 0.f;
  };
  fetch(0);
  for (int t0 = 0; t0 < n_tok; t0 += SCAN_TT) {
    const int tt = min(SCAN_TT, n_tok - t0);
    __syncthreads();                      // the readers of the previous batch are done with the tiles
#pragma unroll
    for (int t = 0; t < SCAN_TT; ++t)
#pragma unroll
      for (int k = 0; k < NB; ++k) {
        const int n = tid + SCAN_THREADS * k, at = t * NP + n + (n >> 4) * 4;
        Bs[at] = rb[t * NB + k];
        Cs[at] = rc[t * NB + k];
      }
#pragma unroll
    for (int k = 0; k < 2; ++k) { xs[tid + SCAN_THREADS * k] = rx[k]; zs[tid + SCAN_THREADS * k] = rz[k]; }
    if (tid < SCAN_TT) {
      const float v = rdt + dtb;
      const float dt = v > 20.f ? v : log1pf(expf(v));
      dts[tid] = dt;
      dAs[tid] = expf(negA * dt);
    }
    __syncthreads();
    if (t0 + SCAN_TT < n_tok) fetch(t0 + SCAN_TT);      // in flight while the current steps are computed
#pragma unroll 4
    for (int t = 0; t < tt; ++t) {       // unrolled: the lane reduction of step t overlaps the state update of step t + 1
      const float dA = dAs[t], dx = dts[t] * xs[t * SCAN_PT + pl];
      const float4* Bt = reinterpret_cast<const float4*>(Bs + t * NP) + ns * (NPT * 5 / 16);
      const float4* Ct = reinterpret_cast<const float4*>(Cs + t * NP) + ns * (NPT * 5 / 16);
      float y0 = 0.f, y1 = 0.f;
#pragma unroll
      for (int q = 0; q < NPT / 4; ++q) {          // B and C are zero past N: those S stay zero and add nothing
        const float4 bv = Bt[q + (q >> 2)], cv = Ct[q + (q >> 2)];
        S[4 * q] = dA * S[4 * q] + dx * bv.x;
        S[4 * q + 1] = dA * S[4 * q + 1] + dx * bv.y;
        S[4 * q + 2] = dA * S[4 * q + 2] + dx * bv.z;
        S[4 * q + 3] = dA * S[4 * q + 3] + dx * bv.w;
        y0 += S[4 * q] * cv.x + S[4 * q + 2] * cv.z;
        y1 += S[4 * q + 1] * cv.y + S[4 * q + 3] * cv.w;
      }
      float y = y0 + y1;
#pragma unroll
      for (int o = SCAN_NS / 2; o > 0; o >>= 1) y += __shfl_xor_sync(0xffffffffu, y, o);
      if (ns == 0) ys[t * SCAN_PT + pl] = y + Dh * xs[t * SCAN_PT + pl];
    }
    __syncthreads();
    for (int i = tid; i < tt * SCAN_PT; i += SCAN_THREADS) {
      const int t = i / SCAN_PT, c = p0 + i % SCAN_PT;
      if (c < P) {
        const float zv = zs[i];
        p.y[((long long)b * p.T + t0 + t) * inner + h * P + c] = ys[i] * (zv * sigmoidf_acc(zv));
      }
    }
  }
#pragma unroll
  for (int i = 0; i < NPT; ++i) {
    const int n = ns * NPT + i;
    if (pok && n < N) Sg[(long long)n * P + pc] = S[i];
  }
}

// ---- grouped RMS norm ---------------------------------------------------------------------------------------------------------
template <typename TO>
__global__ void __launch_bounds__(256) group_rmsnorm_kernel(const float* __restrict__ y, const float* __restrict__ w, TO* __restrict__ out,
                                                            int W, int gw, float eps) {
  __shared__ float red[32];
  const long long base = (long long)blockIdx.x * W + (long long)blockIdx.y * gw;      // rows on grid.x: no 65535 limit
  float ss = 0.f;
  for (int c = threadIdx.x; c < gw; c += blockDim.x) {
    const float v = y[base + c];
    ss += v * v;
  }
  ss = block_sum(ss, red);
  const float r = 1.f / sqrtf(ss / (float)gw + eps);
  for (int c = threadIdx.x; c < gw; c += blockDim.x) stf(out + base + c, y[base + c] * r * w[blockIdx.y * gw + c]);
}

// ---- clamped gate product -----------------------------------------------------------------------------------------------------
template <typename T>
__global__ void __launch_bounds__(256) clamped_glu_kernel(const T* __restrict__ gu, T* __restrict__ out, long long rows, int F, float limit,
                                                          float alpha) {
  const long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x;
  if (i >= rows * F) return;
  const long long r = i / F;
  const int c = (int)(i % F);
  const float g = fminf(ldf(gu + r * 2 * F + c), limit);
  const float u = fminf(fmaxf(ldf(gu + r * 2 * F + F + c), -limit), limit);
  stf(out + i, g * sigmoidf_acc(alpha * g) * (u + 1.f));
}

// 16 bytes of gate and of up per thread (F a multiple of the vector width)
template <typename T>
__global__ void __launch_bounds__(256) clamped_glu_vec_kernel(const T* __restrict__ gu, T* __restrict__ out, long long rows, int F, float limit,
                                                              float alpha) {
  constexpr int VN = Vec<T>::N;
  const int fv = F / VN;
  const long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x;
  if (i >= rows * fv) return;
  const long long r = i / fv;
  const int c = (int)(i % fv) * VN;
  const uint4 gr = *reinterpret_cast<const uint4*>(gu + r * 2 * F + c), ur = *reinterpret_cast<const uint4*>(gu + r * 2 * F + F + c);
  float g[VN], u[VN], y[VN];
  if constexpr (VN == 4) {
    g[0] = __uint_as_float(gr.x); g[1] = __uint_as_float(gr.y); g[2] = __uint_as_float(gr.z); g[3] = __uint_as_float(gr.w);
    u[0] = __uint_as_float(ur.x); u[1] = __uint_as_float(ur.y); u[2] = __uint_as_float(ur.z); u[3] = __uint_as_float(ur.w);
  } else {
    g[0] = bf16lo(gr.x); g[1] = bf16hi(gr.x); g[2] = bf16lo(gr.y); g[3] = bf16hi(gr.y);
    g[4] = bf16lo(gr.z); g[5] = bf16hi(gr.z); g[6] = bf16lo(gr.w); g[7] = bf16hi(gr.w);
    u[0] = bf16lo(ur.x); u[1] = bf16hi(ur.x); u[2] = bf16lo(ur.y); u[3] = bf16hi(ur.y);
    u[4] = bf16lo(ur.z); u[5] = bf16hi(ur.z); u[6] = bf16lo(ur.w); u[7] = bf16hi(ur.w);
  }
#pragma unroll
  for (int e = 0; e < VN; ++e) {
    const float gg = fminf(g[e], limit), uu = fminf(fmaxf(u[e], -limit), limit);
    y[e] = gg * sigmoidf_acc(alpha * gg) * (uu + 1.f);
  }
  uint4 o;
  if constexpr (VN == 4) {
    o = make_uint4(__float_as_uint(y[0]), __float_as_uint(y[1]), __float_as_uint(y[2]), __float_as_uint(y[3]));
  } else {
    o = make_uint4(pack_bf16(y[0], y[1]), pack_bf16(y[2], y[3]), pack_bf16(y[4], y[5]), pack_bf16(y[6], y[7]));
  }
  *reinterpret_cast<uint4*>(out + r * F + c) = o;
}

// ---- fp32 residual stream: s = [x] + [y1] + [y2] + [rms_unit(yn) * wn] + [vec]; h = rms_unit(s) * w -------------------------------
template <typename TY, typename TH>
__global__ void __launch_bounds__(256) stream_add_rmsnorm_kernel(StreamAddParams p) {
  __shared__ float red[32];
  const long long row = blockIdx.x;
  const int W = p.W;
  const float* xr = p.x ? p.x + row * W : nullptr;
  const TY* y1 = p.y1 ? (const TY*)p.y1 + row * W : nullptr;
  const TY* y2 = p.y2 ? (const TY*)p.y2 + row * W : nullptr;
  const TY* yn = p.yn ? (const TY*)p.yn + row * W : nullptr;
  float rn = 0.f;
  if (yn) {
    float ss = 0.f;
    for (int c = threadIdx.x; c < W; c += blockDim.x) { const float v = ldf(yn + c); ss += v * v; }
    rn = 1.f / sqrtf(block_sum(ss, red) / (float)W + p.eps);
  }
  float* so = p.s + row * W;
  __nv_bfloat16* slp = p.s_lp ? (__nv_bfloat16*)p.s_lp + row * W : nullptr;
  float ss = 0.f;
  for (int c = threadIdx.x; c < W; c += blockDim.x) {
    float s = xr ? xr[c] : 0.f;
    if (y1) s += ldf(y1 + c);
    if (y2) s += ldf(y2 + c);
    if (yn) s += ldf(yn + c) * rn * (p.wn ? p.wn[c] : 1.f);
    if (p.vec) s += p.vec[c];
    so[c] = s;
    if (slp) slp[c] = __float2bfloat16_rn(s);
    ss += s * s;
  }
  if (!p.h) return;
  const float r = 1.f / sqrtf(block_sum(ss, red) / (float)W + p.eps);
  TH* ho = (TH*)p.h + row * W;
  for (int c = threadIdx.x; c < W; c += blockDim.x) stf(ho + c, so[c] * r * p.w[c]);      // a thread re-reads only what it wrote itself
}

// The same with four values per thread and access: rows whose width is a multiple of 4 and at most 4 * 256 * NCH; the sums stay in
// registers between the passes.
template <typename T> __device__ __forceinline__ float4 ld4(const T* p);
template <> __device__ __forceinline__ float4 ld4<float>(const float* p) { return *reinterpret_cast<const float4*>(p); }
template <> __device__ __forceinline__ float4 ld4<__nv_bfloat16>(const __nv_bfloat16* p) {
  const uint2 r = *reinterpret_cast<const uint2*>(p);
  return make_float4(bf16lo(r.x), bf16hi(r.x), bf16lo(r.y), bf16hi(r.y));
}
template <typename T> __device__ __forceinline__ void st4(T* p, float4 v);
template <> __device__ __forceinline__ void st4<float>(float* p, float4 v) { *reinterpret_cast<float4*>(p) = v; }
template <> __device__ __forceinline__ void st4<__nv_bfloat16>(__nv_bfloat16* p, float4 v) {
  *reinterpret_cast<uint2*>(p) = make_uint2(pack_bf16(v.x, v.y), pack_bf16(v.z, v.w));
}

template <typename TY, typename TH, int NCH>
__global__ void __launch_bounds__(256) stream_add_rmsnorm_vec_kernel(StreamAddParams p) {
  __shared__ float red[32];
  const long long row = blockIdx.x;
  const int W = p.W;
  const float* xr = p.x ? p.x + row * W : nullptr;
  const TY* y1 = p.y1 ? (const TY*)p.y1 + row * W : nullptr;
  const TY* y2 = p.y2 ? (const TY*)p.y2 + row * W : nullptr;
  const TY* yn = p.yn ? (const TY*)p.yn + row * W : nullptr;
  float4 nv[NCH];
  float rn = 0.f;
  if (yn) {
    float ss = 0.f;
#pragma unroll
    for (int ch = 0; ch < NCH; ++ch) {
      const int c = (ch * 256 + threadIdx.x) * 4;
      nv[ch] = c < W ? ld4(yn + c) : make_float4(0.f, 0.f, 0.f, 0.f);
      ss += nv[ch].x * nv[ch].x + nv[ch].y * nv[ch].y + nv[ch].z * nv[ch].z + nv[ch].w * nv[ch].w;
    }
    rn = 1.f / sqrtf(block_sum(ss, red) / (float)W + p.eps);
  }
  float* so = p.s + row * W;
  __nv_bfloat16* slp = p.s_lp ? (__nv_bfloat16*)p.s_lp + row * W : nullptr;
  float4 sv[NCH];
  float ss = 0.f;
#pragma unroll
  for (int ch = 0; ch < NCH; ++ch) {
    const int c = (ch * 256 + threadIdx.x) * 4;
    if (c >= W) { sv[ch] = make_float4(0.f, 0.f, 0.f, 0.f); continue; }
    float4 s = xr ? ld4(xr + c) : make_float4(0.f, 0.f, 0.f, 0.f);
    if (y1) { const float4 a = ld4(y1 + c); s.x += a.x; s.y += a.y; s.z += a.z; s.w += a.w; }
    if (y2) { const float4 a = ld4(y2 + c); s.x += a.x; s.y += a.y; s.z += a.z; s.w += a.w; }
    if (yn) {
      const float4 g = p.wn ? ld4(p.wn + c) : make_float4(1.f, 1.f, 1.f, 1.f);
      s.x += nv[ch].x * rn * g.x; s.y += nv[ch].y * rn * g.y; s.z += nv[ch].z * rn * g.z; s.w += nv[ch].w * rn * g.w;
    }
    if (p.vec) { const float4 a = ld4(p.vec + c); s.x += a.x; s.y += a.y; s.z += a.z; s.w += a.w; }
    st4(so + c, s);
    if (slp) st4(slp + c, s);
    ss += s.x * s.x + s.y * s.y + s.z * s.z + s.w * s.w;
    sv[ch] = s;
  }
  if (!p.h) return;
  const float r = 1.f / sqrtf(block_sum(ss, red) / (float)W + p.eps);
  TH* ho = (TH*)p.h + row * W;
#pragma unroll
  for (int ch = 0; ch < NCH; ++ch) {
    const int c = (ch * 256 + threadIdx.x) * 4;
    if (c >= W) continue;
    const float4 g = ld4(p.w + c);
    st4(ho + c, make_float4(sv[ch].x * r * g.x, sv[ch].y * r * g.y, sv[ch].z * r * g.z, sv[ch].w * r * g.w));
  }
}

// ---- latent row: RMS norm of a slice of the projection + paged cache write ----------------------------------------------------------
// one warp per token, eight tokens per block: no block-wide synchronisation, the row stays in registers when it is at most 256 wide
template <typename T>
__global__ void __launch_bounds__(256) latent_norm_append_kernel(const T* __restrict__ p, long long p_sb, long long p_st, const float* __restrict__ w,
                                                                 T* __restrict__ cache, const int* __restrict__ block_table,
                                                                 const int* __restrict__ ctx_len, const int* __restrict__ q_len, int B, int Tn, int R,
                                                                 int page, int max_blocks, float eps, T* __restrict__ rows_out, int rot,
                                                                 const float* __restrict__ cosv, const float* __restrict__ sinv,
                                                                 const T* __restrict__ q_in, int q_rank, const float* __restrict__ q_w,
                                                                 T* __restrict__ q_out) {
  const int lane = threadIdx.x & 31;
  const long long tok = (long long)blockIdx.x * 8 + (threadIdx.x >> 5);
  if (tok >= (long long)B * Tn) return;
  const int b = (int)(tok / Tn), t = (int)(tok % Tn);
  if (t >= q_len[b]) return;
  const T* row = p + (long long)b * p_sb + (long long)t * p_st;
  if (q_rank > 0) {      // the query latent of the same token: RMS norm into q_out
    const T* qr = q_in + (long long)b * p_sb + (long long)t * p_st;
    float qs = 0.f;
    for (int c = lane; c < q_rank; c += 32) { const float x = ldf(qr + c); qs += x * x; }
    const float rq = 1.f / sqrtf(warp_sum(qs) / (float)q_rank + eps);
    for (int c = lane; c < q_rank; c += 32) stf(q_out + tok * q_rank + c, ldf(qr + c) * rq * q_w[c]);
  }
  constexpr int KEEP = 8;                       // values per lane held in registers (rows up to 256 wide)
  float v[KEEP];
  float ss = 0.f;
#pragma unroll
  for (int i = 0; i < KEEP; ++i) {
    const int c = lane + 32 * i;
    v[i] = c < R ? ldf(row + c) : 0.f;
    ss += v[i] * v[i];
  }
  for (int c = lane + 32 * KEEP; c < R; c += 32) { const float x = ldf(row + c); ss += x * x; }
  const float r = 1.f / sqrtf(warp_sum(ss) / (float)R + eps);
  const int pos = ctx_len[b] + t;
  const int RW = R + rot;                                 // cache row: the latent, then the rotated key part
  T* dst = cache + ((long long)block_table[(long long)b * max_blocks + pos / page] * page + pos % page) * RW;
  T* dst2 = rows_out ? rows_out + tok * RW : nullptr;     // [B, T, RW]: the same rows in token order
  for (int i = lane; i < rot / 2; i += 32) {              // rotate-half: channel i pairs with i + rot / 2
    const float u = ldf(row + R + i), v = ldf(row + R + rot / 2 + i);
    const float co = cosv[tok * (rot / 2) + i], si = sinv[tok * (rot / 2) + i];
    const float a = u * co - v * si, bb = v * co + u * si;
    stf(dst + R + i, a);
    stf(dst + R + rot / 2 + i, bb);
    if (dst2) { stf(dst2 + R + i, a); stf(dst2 + R + rot / 2 + i, bb); }
  }
#pragma unroll
  for (int i = 0; i < KEEP; ++i) {
    const int c = lane + 32 * i;
    if (c < R) {
      const float o = v[i] * r * w[c];
      stf(dst + c, o);
      if (dst2) stf(dst2 + c, o);
    }
  }
  for (int c = lane + 32 * KEEP; c < R; c += 32) {
    const float o = ldf(row + c) * r * w[c];
    stf(dst + c, o);
    if (dst2) stf(dst2 + c, o);
  }
}

// dst[tok, h, Dd - rot + .] = rotate_half(src[tok, h, Ds - rot + .]); one thread per (token, head, pair)
template <typename T>
__global__ void __launch_bounds__(256) rope_half_tail_kernel(const T* __restrict__ src, T* __restrict__ dst, const float* __restrict__ cosv,
                                                             const float* __restrict__ sinv, long long n, int H, int Ds, int Dd, int rot) {
  const long long idx = (long long)blockIdx.x * blockDim.x + threadIdx.x;
  if (idx >= n) return;
  const int half = rot / 2, i = (int)(idx % half);
  const long long th = idx / half, tok = th / H;
  const T* sr = src + th * Ds + (Ds - rot);
  T* dr = dst + th * Dd + (Dd - rot);
  const float u = ldf(sr + i), v = ldf(sr + half + i);
  const float co = cosv[tok * half + i], si = sinv[tok * half + i];
  stf(dr + i, u * co - v * si);
  stf(dr + half + i, v * co + u * si);
}

// Stream update + norm + short convolution of the normalised rows.  Block = one token; window row j (j < K) is the stream row at
// token index t - K + 1 + j: a new row (x + y1 + y2, formed here) or, before the portion, a carried row of the state line.  Pass 1
// forms the K sums of squares, pass 2 re-reads the rows (cache hits) and writes the result.
__device__ __forceinline__ float ld_any(const void* p, long long i, int lp) {
  return lp ? __bfloat162float(((const __nv_bfloat16*)p)[i]) : ((const float*)p)[i];
}

// rows past q_len are written as zeros by every variant (the outputs are allocated uninitialised)
template <typename TO>
__device__ __forceinline__ void zero_stream_row(const StreamConvParams& p, int b, int t) {
  const long long o = ((long long)b * p.T + t) * p.W;
  for (int c = threadIdx.x; c < p.W; c += blockDim.x) {
    p.s[o + c] = 0.f;
    stf((TO*)p.out + o + c, 0.f);
  }
}

template <typename TO>
__global__ void __launch_bounds__(256) stream_norm_conv_kernel(StreamConvParams p) {
  __shared__ float red[32];
  const int b = blockIdx.y, t = blockIdx.x;
  if (t >= p.q_len[b]) { zero_stream_row<TO>(p, b, t); return; }
  const int W = p.W, K = p.K;
  const bool has_ctx = p.ctx_len[b] > 0;
  const long long base = (long long)b * p.T * W;
  const float* sl = p.state ? p.state + (long long)p.lines[b] * (K - 1) * W : nullptr;
  auto row_value = [&](int j, int c) -> float {
    const int i = t - K + 1 + j;
    if (i >= 0) {
      const long long o = base + (long long)i * W + c;
      float v = p.x[o];
      if (p.y1) v += ld_any(p.y1, o, p.y1_lp);
      if (p.y2) v += ld_any(p.y2, o, p.y2_lp);
      return v;
    }
    return (has_ctx && sl) ? sl[(long long)(K - 1 + i) * W + c] : 0.f;
  };
  float ss[SEQMIX_MAX_TAPS];
#pragma unroll
  for (int j = 0; j < SEQMIX_MAX_TAPS; ++j) ss[j] = 0.f;
  for (int c = threadIdx.x; c < W; c += blockDim.x) {
#pragma unroll
    for (int j = 0; j < SEQMIX_MAX_TAPS; ++j)
      if (j < K) { const float v = row_value(j, c); ss[j] += v * v; }
  }
  float r[SEQMIX_MAX_TAPS];
#pragma unroll
  for (int j = 0; j < SEQMIX_MAX_TAPS; ++j)
    if (j < K) r[j] = 1.f / sqrtf(block_sum(ss[j], red) / (float)W + p.eps);
  const long long o0 = base + (long long)t * W;
  for (int c = threadIdx.x; c < W; c += blockDim.x) {
    const float wc = p.w[c];
    float own = 0.f, acc = 0.f;
#pragma unroll
    for (int j = 0; j < SEQMIX_MAX_TAPS; ++j)
      if (j < K) {
        const float v = row_value(j, c);
        const float h = v * r[j] * wc;
        if (p.cw) acc += p.cw[(long long)c * K + j] * h;
        if (j == K - 1) { own = h; p.s[o0 + c] = v; }
      }
    stf((TO*)p.out + o0 + c, own + acc);
  }
}

// The same with four channels per access and the K window rows held in registers (one pass over the inputs): W a multiple of 4,
// K <= 4, W <= 4 * NCH * blockDim.x.
__device__ __forceinline__ float4 ld4_any(const void* p, long long i, int lp) {
  if (lp) {
    const uint2 r = *reinterpret_cast<const uint2*>((const __nv_bfloat16*)p + i);
    return make_float4(bf16lo(r.x), bf16hi(r.x), bf16lo(r.y), bf16hi(r.y));
  }
  return *reinterpret_cast<const float4*>((const float*)p + i);
}

// addend modes: 0 absent, 1 fp32, 2 bf16.  The mode is a template parameter of the row loader so that the loads of all rows are
// independent straight-line code (a branch per load would serialise them).
template <int M>
__device__ __forceinline__ void add4(float4& a, const void* y, long long o, float m) {
  if constexpr (M == 1) {
    const float4 v = *reinterpret_cast<const float4*>((const float*)y + o);
    a.x += m * v.x; a.y += m * v.y; a.z += m * v.z; a.w += m * v.w;
  } else if constexpr (M == 2) {
    const uint2 r = *reinterpret_cast<const uint2*>((const __nv_bfloat16*)y + o);
    a.x += m * bf16lo(r.x); a.y += m * bf16hi(r.x); a.z += m * bf16lo(r.y); a.w += m * bf16hi(r.y);
  }
}

// window rows first .. first + NR - 1 (token indices; negative: carried rows) of batch row b into registers, with their sums of squares.
// Every load is issued unconditionally from a clamped, valid address and masked afterwards: no branch separates a load from the next,
// so all of a thread's loads are in flight together.
template <int M1, int M2, int K, int NCH, int NR>
__device__ __forceinline__ void load_stream_rows(const StreamConvParams& p, long long base, const float* sl, bool has_ctx, int first, int limit,
                                                 float4 (&v)[NR][NCH], float (&ss)[NR]) {
  const int W = p.W;
  const bool carried = has_ctx && sl != nullptr;
#pragma unroll
  for (int rr = 0; rr < NR; ++rr) {
    const int i = first + rr;
    const bool isnew = i >= 0;
    const int ic = min(max(i, 0), p.T - 1), is = max(K - 1 + i, 0);
    ss[rr] = 0.f;
#pragma unroll
    for (int ch = 0; ch < NCH; ++ch) {
      const int c = (ch * blockDim.x + threadIdx.x) * 4, cc = min(c, W - 4);
      const long long o = base + (long long)ic * W + cc;
      const float* src = (isnew || !carried) ? p.x + o : sl + (long long)is * W + cc;
      float4 a = *reinterpret_cast<const float4*>(src);
      const float m = isnew ? 1.f : 0.f;
      add4<M1>(a, p.y1, o, m);
      add4<M2>(a, p.y2, o, m);
      const bool ok = c < W && (isnew ? i < limit : carried);
      if (!ok) a = make_float4(0.f, 0.f, 0.f, 0.f);
      v[rr][ch] = a;
      ss[rr] += a.x * a.x + a.y * a.y + a.z * a.z + a.w * a.w;
    }
  }
}

template <int K, int NCH, int NR>
__device__ __forceinline__ void load_stream_rows_any(const StreamConvParams& p, long long base, const float* sl, bool has_ctx, int first, int limit,
                                                     float4 (&v)[NR][NCH], float (&ss)[NR]) {
  const int m1 = p.y1 ? (p.y1_lp ? 2 : 1) : 0, m2 = p.y2 ? (p.y2_lp ? 2 : 1) : 0;
  switch (m1 * 3 + m2) {
    case 0: load_stream_rows<0, 0, K, NCH, NR>(p, base, sl, has_ctx, first, limit, v, ss); break;
    case 1: load_stream_rows<0, 1, K, NCH, NR>(p, base, sl, has_ctx, first, limit, v, ss); break;
    case 2: load_stream_rows<0, 2, K, NCH, NR>(p, base, sl, has_ctx, first, limit, v, ss); break;
    case 3: load_stream_rows<1, 0, K, NCH, NR>(p, base, sl, has_ctx, first, limit, v, ss); break;
    case 4: load_stream_rows<1, 1, K, NCH, NR>(p, base, sl, has_ctx, first, limit, v, ss); break;
    case 5: load_stream_rows<1, 2, K, NCH, NR>(p, base, sl, has_ctx, first, limit, v, ss); break;
    case 6: load_stream_rows<2, 0, K, NCH, NR>(p, base, sl, has_ctx, first, limit, v, ss); break;
    case 7: load_stream_rows<2, 1, K, NCH, NR>(p, base, sl, has_ctx, first, limit, v, ss); break;
    default: load_stream_rows<2, 2, K, NCH, NR>(p, base, sl, has_ctx, first, limit, v, ss); break;
  }
}

template <typename TO, int K, int NCH>
__global__ void __launch_bounds__(512) stream_norm_conv_vec_kernel(StreamConvParams p) {
  __shared__ float red[K][32];
  const int b = blockIdx.y, t = blockIdx.x;
  if (t >= p.q_len[b]) { zero_stream_row<TO>(p, b, t); return; }
  const int W = p.W, lane = threadIdx.x & 31, warp = threadIdx.x >> 5, nw = blockDim.x >> 5;
  const bool has_ctx = p.ctx_len[b] > 0;
  const long long base = (long long)b * p.T * W;
  const float* sl = p.state ? p.state + (long long)p.lines[b] * (K - 1) * W : nullptr;
  float4 v[K][NCH];
  float ss[K];
  load_stream_rows_any<K, NCH, K>(p, base, sl, has_ctx, t - K + 1, t + 1, v, ss);
#pragma unroll
  for (int j = 0; j < K; ++j) {
    const float w = warp_sum(ss[j]);
    if (lane == 0) red[j][warp] = w;
  }
  __syncthreads();
  float r[K];
#pragma unroll
  for (int j = 0; j < K; ++j) r[j] = 1.f / sqrtf(warp_sum(lane < nw ? red[j][lane] : 0.f) / (float)W + p.eps);
  const long long o0 = base + (long long)t * W;
#pragma unroll
  for (int ch = 0; ch < NCH; ++ch) {
    const int c = (ch * blockDim.x + threadIdx.x) * 4;
    if (c >= W) continue;
    const float4 wc = *reinterpret_cast<const float4*>(p.w + c);
    const float wv[4] = {wc.x, wc.y, wc.z, wc.w};
    float out[4];
    float taps[4 * K];                                 // the taps of these four channels: cw[c .. c + 3][0 .. K - 1], contiguous
    if (p.cw) {
#pragma unroll
      for (int q = 0; q < K; ++q) {
        const float4 tq = *reinterpret_cast<const float4*>(p.cw + (long long)c * K + 4 * q);
        taps[4 * q] = tq.x; taps[4 * q + 1] = tq.y; taps[4 * q + 2] = tq.z; taps[4 * q + 3] = tq.w;
      }
    }
#pragma unroll
    for (int e = 0; e < 4; ++e) {
      float acc = 0.f, own = 0.f;
#pragma unroll
      for (int j = 0; j < K; ++j) {
        const float4 a = v[j][ch];
        const float val = e == 0 ? a.x : (e == 1 ? a.y : (e == 2 ? a.z : a.w));
        const float h = val * r[j] * wv[e];
        if (p.cw) acc += taps[e * K + j] * h;
        if (j == K - 1) own = h;
      }
      out[e] = own + acc;
    }
    *reinterpret_cast<float4*>(p.s + o0 + c) = v[K - 1][ch];
    if constexpr (std::is_same<TO, float>::value) {
      *reinterpret_cast<float4*>((float*)p.out + o0 + c) = make_float4(out[0], out[1], out[2], out[3]);
    } else {
      *reinterpret_cast<uint2*>((__nv_bfloat16*)p.out + o0 + c) = make_uint2(pack_bf16(out[0], out[1]), pack_bf16(out[2], out[3]));
    }
  }
}

// Block = TT consecutive tokens of one batch row: the TT + K - 1 stream rows they read are loaded once and normalised once (a token's
// row serves the K - 1 tokens after it too), all in registers.  W <= 8 * blockDim.x.
template <typename TO, int K, int NCH, int TT>
__global__ void __launch_bounds__(256, NCH <= 2 ? 3 : 2) stream_norm_conv_tile_kernel(StreamConvParams p) {
  constexpr int NR = TT + K - 1;
  __shared__ float red[NR][32];
  __shared__ float inv[NR];
  const int b = blockIdx.y, t0 = blockIdx.x * TT, qn = p.q_len[b];
  for (int i = 0; i < TT; ++i)
    if (t0 + i >= qn && t0 + i < p.T) zero_stream_row<TO>(p, b, t0 + i);
  if (t0 >= qn) return;
  const int W = p.W, lane = threadIdx.x & 31, warp = threadIdx.x >> 5, nw = blockDim.x >> 5;
  const bool has_ctx = p.ctx_len[b] > 0;
  const long long base = (long long)b * p.T * W;
  const float* sl = p.state ? p.state + (long long)p.lines[b] * (K - 1) * W : nullptr;
  float4 v[NR][NCH];
  float ss[NR];
  load_stream_rows_any<K, NCH, NR>(p, base, sl, has_ctx, t0 - (K - 1), qn, v, ss);
#pragma unroll
  for (int rr = 0; rr < NR; ++rr) {
    const float w = warp_sum(ss[rr]);
    if (lane == 0) red[rr][warp] = w;
  }
  __syncthreads();
  for (int rr = warp; rr < NR; rr += nw) {             // one warp finishes a row: one accurate root and division per row, not per thread
    const float tot = warp_sum(lane < nw ? red[rr][lane] : 0.f);
    if (lane == 0) inv[rr] = 1.f / sqrtf(tot / (float)W + p.eps);
  }
  __syncthreads();
  float r[NR];
#pragma unroll
  for (int rr = 0; rr < NR; ++rr) r[rr] = inv[rr];
#pragma unroll
  for (int ch = 0; ch < NCH; ++ch) {
    const int c = (ch * blockDim.x + threadIdx.x) * 4;
    if (c >= W) continue;
    const float4 wc = *reinterpret_cast<const float4*>(p.w + c);
    float taps[4 * K];                                 // the taps of these four channels: cw[c .. c + 3][0 .. K - 1], contiguous
#pragma unroll
    for (int q = 0; q < K; ++q) {
      const float4 tq = p.cw ? *reinterpret_cast<const float4*>(p.cw + (long long)c * K + 4 * q) : make_float4(0.f, 0.f, 0.f, 0.f);
      taps[4 * q] = tq.x; taps[4 * q + 1] = tq.y; taps[4 * q + 2] = tq.z; taps[4 * q + 3] = tq.w;
    }
#pragma unroll
    for (int i = 0; i < TT; ++i)
      if (t0 + i < qn) *reinterpret_cast<float4*>(p.s + base + (long long)(t0 + i) * W + c) = v[K - 1 + i][ch];
#pragma unroll
    for (int rr = 0; rr < NR; ++rr) {                  // the normalised rows, in place
      float4 a = v[rr][ch];
      a.x *= r[rr] * wc.x; a.y *= r[rr] * wc.y; a.z *= r[rr] * wc.z; a.w *= r[rr] * wc.w;
      v[rr][ch] = a;
    }
#pragma unroll
    for (int i = 0; i < TT; ++i) {
      if (t0 + i >= qn) continue;
      float4 o = v[K - 1 + i][ch];
#pragma unroll
      for (int j = 0; j < K; ++j) {
        const float4 h = v[i + j][ch];
        o.x += taps[j] * h.x; o.y += taps[K + j] * h.y; o.z += taps[2 * K + j] * h.z; o.w += taps[3 * K + j] * h.w;
      }
      const long long oo = base + (long long)(t0 + i) * W + c;
      if constexpr (std::is_same<TO, float>::value) {
        *reinterpret_cast<float4*>((float*)p.out + oo) = o;
      } else {
        *reinterpret_cast<uint2*>((__nv_bfloat16*)p.out + oo) = make_uint2(pack_bf16(o.x, o.y), pack_bf16(o.z, o.w));
      }
    }
  }
}

// y[tok, :] += x[tok, :] * (sum of the weights of the slots routed to ids >= num_experts); block = one token
template <typename T>
__global__ void __launch_bounds__(128) identity_expert_add_kernel(T* __restrict__ y, const T* __restrict__ x, const float* __restrict__ topk_w,
                                                                  const int* __restrict__ topk_i, int H, int k, int num_experts) {
  const long long tok = blockIdx.x;
  float coef = 0.f;
  for (int j = 0; j < k; ++j)
    if (topk_i[tok * k + j] >= num_experts) coef += topk_w[tok * k + j];
  if (coef == 0.f) return;
  for (int c = threadIdx.x; c < H; c += 128) stf(y + tok * H + c, ldf(y + tok * H + c) + ldf(x + tok * H + c) * coef);
}

// x[row, h, :] *= sigmoid(gate[row, h]); 16 bytes per thread, D a multiple of the vector width
template <typename T>
__global__ void __launch_bounds__(256) head_gate_mul_kernel(T* __restrict__ x, const T* __restrict__ gate, long long g_stride, long long nvec, int H,
                                                            int dvec) {
  constexpr int V = Vec<T>::N;
  const long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x;
  if (i >= nvec) return;
  const long long rh = i / dvec, row = rh / H;
  const int h = (int)(rh % H);
  const float g = sigmoidf_acc(ldf(gate + row * g_stride + h));
  uint4 a = *reinterpret_cast<uint4*>(x + i * V);
  if constexpr (V == 4) {
    a = make_uint4(__float_as_uint(__uint_as_float(a.x) * g), __float_as_uint(__uint_as_float(a.y) * g), __float_as_uint(__uint_as_float(a.z) * g),
                   __float_as_uint(__uint_as_float(a.w) * g));
  } else {
    a = make_uint4(pack_bf16(bf16lo(a.x) * g, bf16hi(a.x) * g), pack_bf16(bf16lo(a.y) * g, bf16hi(a.y) * g), pack_bf16(bf16lo(a.z) * g, bf16hi(a.z) * g),
                   pack_bf16(bf16lo(a.w) * g, bf16hi(a.w) * g));
  }
  *reinterpret_cast<uint4*>(x + i * V) = a;
}

// ---- elementwise activations -------------------------------------------------------------------------------------------------------
__device__ __forceinline__ float unary_apply(int act, float v) {
  switch (act) {
    case 1: return fmaxf(v, 0.f);
    case 2: { const float r = fmaxf(v, 0.f); return r * r; }
    case 3: return v / (1.f + expf(-v));
    case 4: return 0.5f * v * (1.f + tanhf(0.7978845608028654f * (v + 0.044715f * v * v * v)));
    case 5: return 1.f / (1.f + expf(-v));
    case 6: return 0.5f * v * (1.f + erff(v * 0.7071067811865476f));
    default: return v;
  }
}

template <typename T>
__global__ void __launch_bounds__(256) gated_act_mul_kernel(const T* __restrict__ gate, long long g_stride, const T* __restrict__ other,
                                                            long long o_stride, T* __restrict__ out, long long rows, int C, int act, int on_other) {
  const long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x;
  if (i >= rows * C) return;
  const long long r = i / C;
  const int c = (int)(i % C);
  const float g = ldf(gate + r * g_stride + c), o = ldf(other + r * o_stride + c);
  stf(out + i, on_other ? g * unary_apply(act, o) : unary_apply(act, g) * o);
}

template <typename T>
__global__ void __launch_bounds__(256) unary_act_kernel(const T* __restrict__ x, T* __restrict__ out, long long n, int act) {
  const long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x;
  if (i < n) stf(out + i, unary_apply(act, ldf(x + i)));
}

// 16 bytes per thread: `other` rows start at o_stride elements (a multiple of the vector width), C a multiple of it too
template <typename T, bool MUL>
__global__ void __launch_bounds__(256) act_vec_kernel(const T* __restrict__ x, const T* __restrict__ other, long long o_stride, T* __restrict__ out,
                                                      long long nvec, int cvec, int act, long long x_stride = 0, int on_other = 0) {
  constexpr int V = Vec<T>::N;
  const long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x;
  if (i >= nvec) return;
  const uint4 a = *reinterpret_cast<const uint4*>(MUL ? x + (i / cvec) * x_stride + (i % cvec) * V : x + i * V);
  uint4 b = make_uint4(0u, 0u, 0u, 0u);
  if constexpr (MUL) b = *reinterpret_cast<const uint4*>(other + (i / cvec) * o_stride + (i % cvec) * V);
  uint4 o;
  if constexpr (V == 4) {
    float f[4] = {__uint_as_float(a.x), __uint_as_float(a.y), __uint_as_float(a.z), __uint_as_float(a.w)};
    const float m[4] = {__uint_as_float(b.x), __uint_as_float(b.y), __uint_as_float(b.z), __uint_as_float(b.w)};
#pragma unroll
    for (int e = 0; e < 4; ++e) f[e] = (MUL && on_other) ? f[e] * unary_apply(act, m[e]) : unary_apply(act, f[e]) * (MUL ? m[e] : 1.f);
    o = make_uint4(__float_as_uint(f[0]), __float_as_uint(f[1]), __float_as_uint(f[2]), __float_as_uint(f[3]));
  } else {
    float f[8] = {bf16lo(a.x), bf16hi(a.x), bf16lo(a.y), bf16hi(a.y), bf16lo(a.z), bf16hi(a.z), bf16lo(a.w), bf16hi(a.w)};
    const float m[8] = {bf16lo(b.x), bf16hi(b.x), bf16lo(b.y), bf16hi(b.y), bf16lo(b.z), bf16hi(b.z), bf16lo(b.w), bf16hi(b.w)};
#pragma unroll
    for (int e = 0; e < 8; ++e) f[e] = (MUL && on_other) ? f[e] * unary_apply(act, m[e]) : unary_apply(act, f[e]) * (MUL ? m[e] : 1.f);
    o = make_uint4(pack_bf16(f[0], f[1]), pack_bf16(f[2], f[3]), pack_bf16(f[4], f[5]), pack_bf16(f[6], f[7]));
  }
  *reinterpret_cast<uint4*>(out + i * V) = o;
}


// ---- sandwich-norm stream update: y = sa f(a) + sb f(b); s = x + mult ls norm(y) post_w; h = norm(s) next_w ------------------------
// One block per row; the row lives in shared memory (y, then s), so the centred second moments are true two-pass sums.
template <typename TY, typename TH>
__global__ void __launch_bounds__(256) stream_sandwich_norm_kernel(SandwichParams p) {
  extern __shared__ float rowbuf[];      // [W]
  __shared__ float red[32];
  const long long row = blockIdx.x;
  const int W = p.W;
  const float inv_w = 1.f / (float)W;
  const float* xr = p.x + row * W;
  float* so = p.s + row * W;
  if (p.a) {
    const TY* ar = (const TY*)p.a + row * W;
    const TY* br = p.b ? (const TY*)p.b + row * W : nullptr;
    float ra = 1.f, rb = 1.f;
    if (p.a_w || (br && p.b_w)) {
      float sa = 0.f, sb = 0.f;
      for (int c = threadIdx.x; c < W; c += blockDim.x) {
        const float va = ldf(ar + c);
        sa += va * va;
        if (br) { const float vb = ldf(br + c); sb += vb * vb; }
      }
      if (p.a_w) ra = 1.f / sqrtf(block_sum(sa, red) * inv_w + p.eps);
      if (br && p.b_w) rb = 1.f / sqrtf(block_sum(sb, red) * inv_w + p.eps);
    }
    float sum = 0.f;
    for (int c = threadIdx.x; c < W; c += blockDim.x) {
      float y = p.a_scale * (p.a_w ? ldf(ar + c) * ra * p.a_w[c] : ldf(ar + c));
      if (br) y += p.b_scale * (p.b_w ? ldf(br + c) * rb * p.b_w[c] : ldf(br + c));
      rowbuf[c] = y;
      sum += y;
    }
    const float mean = p.center ? block_sum(sum, red) * inv_w : 0.f;
    float sq = 0.f;
    for (int c = threadIdx.x; c < W; c += blockDim.x) { const float d = rowbuf[c] - mean; sq += d * d; }
    const float r = 1.f / sqrtf(block_sum(sq, red) * inv_w + p.eps);
    for (int c = threadIdx.x; c < W; c += blockDim.x) {
      float y = (rowbuf[c] - mean) * r;
      if (p.post_w) y *= p.post_w[c];
      if (p.ls) y *= p.ls[c];
      const float s = xr[c] + p.mult * y;
      so[c] = s;
      rowbuf[c] = s;
    }
  } else {
    for (int c = threadIdx.x; c < W; c += blockDim.x) { const float s = xr[c]; so[c] = s; rowbuf[c] = s; }
  }
  if (!p.h) return;
  float sum = 0.f;
  for (int c = threadIdx.x; c < W; c += blockDim.x) sum += rowbuf[c];      // a thread re-reads only what it wrote itself
  const float mean = p.center ? block_sum(sum, red) * inv_w : 0.f;
  float sq = 0.f;
  for (int c = threadIdx.x; c < W; c += blockDim.x) { const float d = rowbuf[c] - mean; sq += d * d; }
  const float r = 1.f / sqrtf(block_sum(sq, red) * inv_w + p.eps);
  TH* ho = (TH*)p.h + row * W;
  for (int c = threadIdx.x; c < W; c += blockDim.x) stf(ho + c, (rowbuf[c] - mean) * r * p.next_w[c]);
}


// The same with four values per thread and access: rows whose width is a multiple of 4 and at most 4 * 256 * NCH; the row stays in
// registers from the first load to the last store (y, then s), every input is read once.
__device__ __forceinline__ float sum4(float4 v) { return (v.x + v.y) + (v.z + v.w); }
__device__ __forceinline__ float sq4(float4 v) { return v.x * v.x + v.y * v.y + v.z * v.z + v.w * v.w; }

template <typename TY, typename TH, int NCH>
__global__ void __launch_bounds__(256) stream_sandwich_norm_vec_kernel(SandwichParams p) {
  __shared__ float red[32];
  const long long row = blockIdx.x;
  const int W = p.W;
  const float inv_w = 1.f / (float)W;
  const float* xr = p.x + row * W;
  float* so = p.s + row * W;
  const float4 zero = make_float4(0.f, 0.f, 0.f, 0.f), one = make_float4(1.f, 1.f, 1.f, 1.f);
  float4 v[NCH];
  if (p.a) {
    const TY* ar = (const TY*)p.a + row * W;
    const TY* br = p.b ? (const TY*)p.b + row * W : nullptr;
    float4 bv[NCH];
    float sa = 0.f, sb = 0.f;
#pragma unroll
    for (int ch = 0; ch < NCH; ++ch) {
      const int c = (ch * 256 + threadIdx.x) * 4;
      const bool in = c < W;
      v[ch] = in ? ld4(ar + c) : zero;
      bv[ch] = (in && br) ? ld4(br + c) : zero;
      sa += sq4(v[ch]);
      sb += sq4(bv[ch]);
    }
    float ra = 1.f, rb = 1.f;
    if (p.a_w) ra = 1.f / sqrtf(block_sum(sa, red) * inv_w + p.eps);
    if (br && p.b_w) rb = 1.f / sqrtf(block_sum(sb, red) * inv_w + p.eps);
    ra *= p.a_scale;
    rb *= p.b_scale;
    float sum = 0.f;
#pragma unroll
    for (int ch = 0; ch < NCH; ++ch) {
      const int c = (ch * 256 + threadIdx.x) * 4;
      if (c >= W) continue;
      const float4 wa = p.a_w ? ld4(p.a_w + c) : one;
      float4 y = make_float4(v[ch].x * ra * wa.x, v[ch].y * ra * wa.y, v[ch].z * ra * wa.z, v[ch].w * ra * wa.w);
      if (br) {
        const float4 wb = p.b_w ? ld4(p.b_w + c) : one;
        y.x += bv[ch].x * rb * wb.x; y.y += bv[ch].y * rb * wb.y; y.z += bv[ch].z * rb * wb.z; y.w += bv[ch].w * rb * wb.w;
      }
      v[ch] = y;
      sum += sum4(y);
    }
    const float mean = p.center ? block_sum(sum, red) * inv_w : 0.f;
    float sq = 0.f;
#pragma unroll
    for (int ch = 0; ch < NCH; ++ch) {
      const int c = (ch * 256 + threadIdx.x) * 4;
      if (c >= W) continue;
      v[ch] = make_float4(v[ch].x - mean, v[ch].y - mean, v[ch].z - mean, v[ch].w - mean);
      sq += sq4(v[ch]);
    }
    const float r = p.mult / sqrtf(block_sum(sq, red) * inv_w + p.eps);
#pragma unroll
    for (int ch = 0; ch < NCH; ++ch) {
      const int c = (ch * 256 + threadIdx.x) * 4;
      if (c >= W) continue;
      float4 g = p.post_w ? ld4(p.post_w + c) : one;
      if (p.ls) { const float4 l = ld4(p.ls + c); g.x *= l.x; g.y *= l.y; g.z *= l.z; g.w *= l.w; }
      const float4 x = ld4(xr + c);
      v[ch] = make_float4(x.x + v[ch].x * r * g.x, x.y + v[ch].y * r * g.y, x.z + v[ch].z * r * g.z, x.w + v[ch].w * r * g.w);
      st4(so + c, v[ch]);
    }
  } else {
#pragma unroll
    for (int ch = 0; ch < NCH; ++ch) {
      const int c = (ch * 256 + threadIdx.x) * 4;
      v[ch] = c < W ? ld4(xr + c) : zero;
      if (c < W) st4(so + c, v[ch]);
    }
  }
  if (!p.h) return;
  float sum = 0.f;
#pragma unroll
  for (int ch = 0; ch < NCH; ++ch) sum += ((ch * 256 + threadIdx.x) * 4 < W) ? sum4(v[ch]) : 0.f;
  const float mean = p.center ? block_sum(sum, red) * inv_w : 0.f;
  float sq = 0.f;
#pragma unroll
  for (int ch = 0; ch < NCH; ++ch) {
    if ((ch * 256 + threadIdx.x) * 4 >= W) continue;
    v[ch] = make_float4(v[ch].x - mean, v[ch].y - mean, v[ch].z - mean, v[ch].w - mean);
    sq += sq4(v[ch]);
  }
  const float r = 1.f / sqrtf(block_sum(sq, red) * inv_w + p.eps);
  TH* ho = (TH*)p.h + row * W;
#pragma unroll
  for (int ch = 0; ch < NCH; ++ch) {
    const int c = (ch * 256 + threadIdx.x) * 4;
    if (c >= W) continue;
    const float4 g = ld4(p.next_w + c);
    st4(ho + c, make_float4(v[ch].x * r * g.x, v[ch].y * r * g.y, v[ch].z * r * g.z, v[ch].w * r * g.w));
  }
}

// ---- per-head q / k norm + rotate-half rotation + paged cache write -------------------------------------------------------------------
// Block = one token, 8 warps; a warp takes heads warp, warp + 8, ... of the n_q + n_kv heads; lane l holds channels l, l + 32, ...
constexpr int HNR_WARPS = 8;
constexpr int HNR_CPL = 8;               // channels per lane: head sizes up to 256
template <typename T>
__global__ void __launch_bounds__(HNR_WARPS * 32) head_norm_rope_append_kernel(HeadNormRopeParams p) {
  __shared__ float sh[HNR_WARPS][HNR_CPL * 32];
  const int b = blockIdx.y, t = blockIdx.x;
  if (t >= p.q_len[b]) return;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int D = p.D, Dv = p.Dv, R = p.R, half = R >> 1;
  const long long tok = (long long)b * p.T + t;
  const T* row = (const T*)p.p + (long long)b * p.p_sb + (long long)t * p.p_st;
  const float* cs = p.cos ? p.cos + tok * half : nullptr;
  const float* sn = p.sin ? p.sin + tok * half : nullptr;
  const int pos = p.ctx_len[b] + t;
  const long long slot = (long long)p.block_table[(long long)b * p.max_blocks + pos / p.page] * p.page + pos % p.page;
  const int Cq = p.n_q * D, Ck = p.n_kv * D;
  float* mine = sh[warp];
  for (int hh = warp; hh < p.n_q + p.n_kv; hh += HNR_WARPS) {
    const bool isq = hh < p.n_q;
    const int g = isq ? hh : hh - p.n_q;
    const T* src = row + (isq ? (long long)hh * D : (long long)Cq + (long long)g * D);
    const float* nw = isq ? p.q_w : p.k_w;
    float x[HNR_CPL];
    float ss = 0.f;
#pragma unroll
    for (int i = 0; i < HNR_CPL; ++i) {
      const int d = lane + 32 * i;
      x[i] = d < D ? ldf(src + d) : 0.f;
      ss += x[i] * x[i];
    }
    if (!isq && p.value_from_key) {          // the raw key doubles as the value
      T* vo = (T*)p.v_cache + (slot * p.n_kv + g) * Dv;
#pragma unroll
      for (int i = 0; i < HNR_CPL; ++i) { const int d = lane + 32 * i; if (d < Dv) stf(vo + d, x[i]); }
    }
    if (p.norm_at == 1) {
      const float r = 1.f / sqrtf(warp_sum(ss) / (float)D + p.eps);
#pragma unroll
      for (int i = 0; i < HNR_CPL; ++i) { const int d = lane + 32 * i; x[i] = d < D ? x[i] * r * (nw ? nw[d] : 1.f) : 0.f; }
    }
    if (cs) {
      __syncwarp();
#pragma unroll
      for (int i = 0; i < HNR_CPL; ++i) { const int d = lane + 32 * i; if (d < R) mine[d] = x[i]; }
      __syncwarp();
#pragma unroll
      for (int i = 0; i < HNR_CPL; ++i) {
        const int d = lane + 32 * i;
        if (d < R) {
          const int f = d < half ? d : d - half;
          const float co = cs[f], si = sn[f], other = mine[d < half ? d + half : d - half];
          x[i] = d < half ? x[i] * co - other * si : x[i] * co + other * si;
        }
      }
    }
    if (p.norm_at == 2) {
      float s2 = 0.f;
#pragma unroll
      for (int i = 0; i < HNR_CPL; ++i) s2 += x[i] * x[i];
      const float r = 1.f / sqrtf(warp_sum(s2) / (float)D + p.eps);
#pragma unroll
      for (int i = 0; i < HNR_CPL; ++i) { const int d = lane + 32 * i; x[i] = d < D ? x[i] * r * (nw ? nw[d] : 1.f) : 0.f; }
    }
    T* dst = isq ? (T*)p.q_out + (tok * p.n_q + hh) * D : (T*)p.k_cache + (slot * p.n_kv + g) * D;
#pragma unroll
    for (int i = 0; i < HNR_CPL; ++i) { const int d = lane + 32 * i; if (d < D) stf(dst + d, x[i]); }
  }
  if (!p.value_from_key) {
    const T* vs = row + Cq + Ck;
    T* vo = (T*)p.v_cache + slot * p.n_kv * Dv;
    for (int c = threadIdx.x; c < p.n_kv * Dv; c += blockDim.x) vo[c] = vs[c];
  }
}


// Head sizes of 32 * VPL (64, 128, 256) with rotated halves that are multiples of VPL: lane l holds channels [l VPL, (l + 1) VPL) as ONE
// vector access, and the rotation partner of a channel sits in the same register of lane l +- (R / 2) / VPL: a shuffle, no shared memory.
template <typename T, int VPL>
__device__ __forceinline__ void ld_vpl(const T* p, float* x) {
  if constexpr (std::is_same<T, float>::value) {
#pragma unroll
    for (int e = 0; e < VPL; e += 2) { const float2 v = *reinterpret_cast<const float2*>(p + e); x[e] = v.x; x[e + 1] = v.y; }
  } else if constexpr (VPL == 2) {
    const float2 v = ld2(p); x[0] = v.x; x[1] = v.y;
  } else if constexpr (VPL == 4) {
    const float4 v = ld4(p); x[0] = v.x; x[1] = v.y; x[2] = v.z; x[3] = v.w;
  } else {
    const uint4 r = *reinterpret_cast<const uint4*>(p);
    x[0] = bf16lo(r.x); x[1] = bf16hi(r.x); x[2] = bf16lo(r.y); x[3] = bf16hi(r.y); x[4] = bf16lo(r.z); x[5] = bf16hi(r.z); x[6] = bf16lo(r.w); x[7] = bf16hi(r.w);
  }
}
template <typename T, int VPL>
__device__ __forceinline__ void st_vpl(T* p, const float* x) {
  if constexpr (std::is_same<T, float>::value) {
#pragma unroll
    for (int e = 0; e < VPL; e += 2) *reinterpret_cast<float2*>(p + e) = make_float2(x[e], x[e + 1]);
  } else if constexpr (VPL == 2) {
    st2(p, x[0], x[1]);
  } else if constexpr (VPL == 4) {
    st4(p, make_float4(x[0], x[1], x[2], x[3]));
  } else {
    *reinterpret_cast<uint4*>(p) = make_uint4(pack_bf16(x[0], x[1]), pack_bf16(x[2], x[3]), pack_bf16(x[4], x[5]), pack_bf16(x[6], x[7]));
  }
}

template <typename T, int VPL>
__global__ void __launch_bounds__(HNR_WARPS * 32) head_norm_rope_append_lane_kernel(HeadNormRopeParams p) {
  const int b = blockIdx.y, t = blockIdx.x;
  if (t >= p.q_len[b]) return;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  constexpr int D = 32 * VPL;
  const int Dv = p.Dv, R = p.R, half = R >> 1, d0 = lane * VPL;
  const long long tok = (long long)b * p.T + t;
  const T* row = (const T*)p.p + (long long)b * p.p_sb + (long long)t * p.p_st;
  const int pos = p.ctx_len[b] + t;
  const long long slot = (long long)p.block_table[(long long)b * p.max_blocks + pos / p.page] * p.page + pos % p.page;
  const int Cq = p.n_q * D, Ck = p.n_kv * D;
  // this lane's cos / sin (the same for every head of the token) and where its rotation partner sits
  const bool rot = p.cos && d0 < R, low = d0 < half;
  const int f0 = low ? d0 : d0 - half, partner = low ? lane + half / VPL : lane - half / VPL;
  float co[VPL], si[VPL];
#pragma unroll
  for (int e = 0; e < VPL; ++e) {
    co[e] = rot ? p.cos[tok * half + f0 + e] : 1.f;
    si[e] = rot ? p.sin[tok * half + f0 + e] : 0.f;
    if (low) si[e] = -si[e];          // x_lo' = x_lo c - x_hi s, x_hi' = x_hi c + x_lo s: the low half takes the minus sign
  }
  for (int hh = warp; hh < p.n_q + p.n_kv; hh += HNR_WARPS) {
    const bool isq = hh < p.n_q;
    const int g = isq ? hh : hh - p.n_q;
    const T* src = row + (isq ? (long long)hh * D : (long long)Cq + (long long)g * D) + d0;
    const float* nw = isq ? p.q_w : p.k_w;
    float x[VPL];
    ld_vpl<T, VPL>(src, x);
    if (!isq && p.value_from_key) st_vpl<T, VPL>((T*)p.v_cache + (slot * p.n_kv + g) * Dv + d0, x);      // the raw key doubles as the value
    if (p.norm_at == 1) {
      float ss = 0.f;
#pragma unroll
      for (int e = 0; e < VPL; ++e) ss += x[e] * x[e];
      const float r = 1.f / sqrtf(warp_sum(ss) / (float)D + p.eps);
#pragma unroll
      for (int e = 0; e < VPL; ++e) x[e] = x[e] * r * (nw ? nw[d0 + e] : 1.f);
    }
    if (p.cos) {
#pragma unroll
      for (int e = 0; e < VPL; ++e) {
        const float other = __shfl_sync(0xffffffffu, x[e], partner & 31);
        x[e] = x[e] * co[e] + other * si[e];
      }
    }
    if (p.norm_at == 2) {
      float ss = 0.f;
#pragma unroll
      for (int e = 0; e < VPL; ++e) ss += x[e] * x[e];
      const float r = 1.f / sqrtf(warp_sum(ss) / (float)D + p.eps);
#pragma unroll
      for (int e = 0; e < VPL; ++e) x[e] = x[e] * r * (nw ? nw[d0 + e] : 1.f);
    }
    st_vpl<T, VPL>((isq ? (T*)p.q_out + (tok * p.n_q + hh) * D : (T*)p.k_cache + (slot * p.n_kv + g) * D) + d0, x);
  }
  if (!p.value_from_key) {
    const T* vs = row + Cq + Ck;
    T* vo = (T*)p.v_cache + slot * p.n_kv * Dv;
    constexpr int VN = Vec<T>::N;
    const int n = p.n_kv * Dv;
    if (n % VN == 0 && (((uintptr_t)vs | (uintptr_t)vo) & 15) == 0) {
      for (int c = threadIdx.x * VN; c < n; c += blockDim.x * VN) *reinterpret_cast<uint4*>(vo + c) = *reinterpret_cast<const uint4*>(vs + c);
    } else {
      for (int c = threadIdx.x; c < n; c += blockDim.x) vo[c] = vs[c];
    }
  }
}

// ---- gated delta rule with a carried state -------------------------------------------------------------------------------------------
// Block = one (row, head, 16 value channels); 8 lanes split the key axis of a state column and hold their share in registers.  The
// columns of S are independent: with the OLD column s, r = g (s . k), u = beta (v - r), o = g (s . q) + u (k . q), s <- g s + k u, so both
// dot products of a step run on the old state and share one lane reduction.  Time runs in batches of 16 steps: raw q / k of batch
// r + 1 are fetched into registers while batch r is computed out of shared memory; their unit norms, k . q, beta and the decay are
// formed once per batch and folded into per-step scalars.
constexpr int DLT_PT = 16, DLT_NS = 8, DLT_TT = 16, DLT_THREADS = DLT_PT * DLT_NS;

template <typename T, int NB>
__global__ void __launch_bounds__(DLT_THREADS, NB == 1 ? 4 : 2) gated_delta_scan_kernel(DeltaScanParams p) {
  extern __shared__ float sm[];
  constexpr int DPT = 16 * NB;             // key channels per lane: d = ns * DPT + i
  constexpr int DP = 160 * NB;             // padded staged row: 4 floats after every 16
  const int D = p.D, Dv = p.Dv;
  float* qs = sm;                          // [TT][DP] raw q, zero past D
  float* ks = qs + DLT_TT * DP;            // [TT][DP] raw k
  float* vs = ks + DLT_TT * DP;            // [TT][PT]
  float* os = vs + DLT_TT * DLT_PT;        // [TT][PT]
  float* cg = os + DLT_TT * DLT_PT;        // [TT] decay
  float* cb = cg + DLT_TT;                 // [TT] beta
  float* cq = cb + DLT_TT;                 // [TT] 1 / |q| * D^-1/2
  float* ck = cq + DLT_TT;                 // [TT] 1 / |k|
  float* ckq = ck + DLT_TT;                // [TT] unit k . scaled unit q
  const int b = blockIdx.z, h = blockIdx.y, p0 = blockIdx.x * DLT_PT;
  const int n_tok = p.q_len[b];
  if (n_tok <= 0) return;
  const int tid = threadIdx.x, pl = tid / DLT_NS, ns = tid % DLT_NS, warp = tid >> 5, lane = tid & 31;
  const int pc = p0 + pl;
  const bool pok = pc < Dv;
  const int gq = h / (p.nh / p.n_qk);
  const int Cq = p.n_qk * D, C = 2 * Cq + p.nh * Dv;
  float* Sg = p.state + ((long long)p.lines[b] * p.nh + h) * D * Dv;
  float S[DPT];
  const bool has_ctx = p.ctx_len[b] > 0;
#pragma unroll
  for (int i = 0; i < DPT; ++i) {
    const int d = ns * DPT + i;
    S[i] = (has_ctx && pok && d < D) ? Sg[(long long)d * Dv + pc] : 0.f;
  }
  const float negA = -expf(p.A_log[h]), dtb = p.dt_bias[h], qmul = 1.f / sqrtf((float)D);
  const float* xrow = p.qkv + (long long)b * p.T * C;
  const T* bp = (const T*)p.beta_raw + (long long)b * p.beta_sb + h;
  const T* ap = (const T*)p.a_raw + (long long)b * p.a_sb + h;
  float rq[DPT], rk[DPT], rv[2], rbeta = 0.f, ra = 0.f;
  auto fetch = [&](int t0) {
    const int tt = min(DLT_TT, n_tok - t0);
#pragma unroll
    for (int t = 0; t < DLT_TT; ++t)
#pragma unroll
      for (int k = 0; k < NB; ++k) {
        const int d = tid + DLT_THREADS * k;
        const bool ok = t < tt && d < D;
        const float* r = xrow + (long long)(t0 + t) * C + gq * D + d;
        rq[t * NB + k] = ok ? r[0] : 0.f;
        rk[t * NB + k] = ok ? r[Cq] : 0.f;
      }
#pragma unroll
    for (int k = 0; k < 2; ++k) {
      const int i = tid + DLT_THREADS * k, t = i / DLT_PT, c = p0 + i % DLT_PT;
      rv[k] = (t < tt && c < Dv) ? xrow[(long long)(t0 + t) * C + 2 * Cq + h * Dv + c] : 0.f;
    }
    rbeta = tid < tt ? ldf(bp + (long long)(t0 + tid) * p.beta_st) : 0.f;
    ra = tid < tt ? ldf(ap + (long long)(t0 + tid) * p.a_st) : 0.f;
  };
  fetch(0);
  for (int t0 = 0; t0 < n_tok; t0 += DLT_TT) {
    const int tt = min(DLT_TT, n_tok - t0);
    __syncthreads();                      // the readers of the previous batch are done with the tiles
#pragma unroll
    for (int t = 0; t < DLT_TT; ++t)
#pragma unroll
      for (int k = 0; k < NB; ++k) {
        const int d = tid + DLT_THREADS * k, at = t * DP + d + (d >> 4) * 4;
        qs[at] = rq[t * NB + k];
        ks[at] = rk[t * NB + k];
      }
#pragma unroll
    for (int k = 0; k < 2; ++k) vs[tid + DLT_THREADS * k] = rv[k];
    if (tid < DLT_TT) {
      const float v = ra + dtb;
      const float sp = v > 20.f ? v : log1pf(expf(v));
      cg[tid] = expf(negA * sp);
      cb[tid] = sigmoidf_acc(rbeta);
    }
    __syncthreads();
    // unit norms and k . q of the batch: warp w takes steps w, w + 4, ...
    for (int t = warp; t < DLT_TT; t += DLT_THREADS / 32) {
      float qq = 0.f, kk = 0.f, kq = 0.f;
      for (int d = lane; d < D; d += 32) {
        const int at = t * DP + d + (d >> 4) * 4;
        const float a = qs[at], c = ks[at];
        qq += a * a; kk += c * c; kq += a * c;
      }
      qq = warp_sum(qq); kk = warp_sum(kk); kq = warp_sum(kq);
      if (lane == 0) {
        const float iq = qmul / sqrtf(qq + p.unit_eps), ik = 1.f / sqrtf(kk + p.unit_eps);
        cq[t] = iq; ck[t] = ik; ckq[t] = kq * iq * ik;
      }
    }
    __syncthreads();
    if (t0 + DLT_TT < n_tok) fetch(t0 + DLT_TT);      // in flight while the current steps are computed
#pragma unroll 2
    for (int t = 0; t < tt; ++t) {
      const float4* Kt = reinterpret_cast<const float4*>(ks + t * DP) + ns * (DPT * 5 / 16);
      const float4* Qt = reinterpret_cast<const float4*>(qs + t * DP) + ns * (DPT * 5 / 16);
      float4 kv[DPT / 4];
      float k0 = 0.f, k1 = 0.f, q0 = 0.f, q1 = 0.f;
#pragma unroll
      for (int q = 0; q < DPT / 4; ++q) {
        kv[q] = Kt[q + (q >> 2)];
        const float4 qv = Qt[q + (q >> 2)];
        k0 += S[4 * q] * kv[q].x + S[4 * q + 2] * kv[q].z;
        k1 += S[4 * q + 1] * kv[q].y + S[4 * q + 3] * kv[q].w;
        q0 += S[4 * q] * qv.x + S[4 * q + 2] * qv.z;
        q1 += S[4 * q + 1] * qv.y + S[4 * q + 3] * qv.w;
      }
      float sk = k0 + k1, sq = q0 + q1;
#pragma unroll
      for (int o = DLT_NS / 2; o > 0; o >>= 1) {
        sk += __shfl_xor_sync(0xffffffffu, sk, o);
        sq += __shfl_xor_sync(0xffffffffu, sq, o);
      }
      const float g = cg[t], ikn = ck[t];
      const float u = cb[t] * (vs[t * DLT_PT + pl] - g * ikn * sk);
      const float ku = ikn * u;
#pragma unroll
      for (int q = 0; q < DPT / 4; ++q) {
        S[4 * q] = g * S[4 * q] + ku * kv[q].x;
        S[4 * q + 1] = g * S[4 * q + 1] + ku * kv[q].y;
        S[4 * q + 2] = g * S[4 * q + 2] + ku * kv[q].z;
        S[4 * q + 3] = g * S[4 * q + 3] + ku * kv[q].w;
      }
      if (ns == 0) os[t * DLT_PT + pl] = g * cq[t] * sq + u * ckq[t];
    }
    __syncthreads();
    for (int i = tid; i < tt * DLT_PT; i += DLT_THREADS) {
      const int t = i / DLT_PT, c = p0 + i % DLT_PT;
      if (c < Dv) p.o[((long long)b * p.T + t0 + t) * p.nh * Dv + h * Dv + c] = os[i];
    }
  }
#pragma unroll
  for (int i = 0; i < DPT; ++i) {
    const int d = ns * DPT + i;
    if (pok && d < D) Sg[(long long)d * Dv + pc] = S[i];
  }
}


// The same recurrence with TWO state columns per thread (8 lanes x DPT key channels each): the k / q values a thread reads from
// shared memory serve both columns, which halves the shared-memory traffic per state element (the recurrent form is bound by it: every
// column needs the whole k and q of every step), and q / k / v of the next 16 steps are copied straight into a second shared-memory
// stage with cp.async, so no registers are spent on prefetching.  Thread (t, part) forms the unit norms and k . q of step t from a
// quarter of the row (one short lane reduction instead of a warp-wide one); the per-step scalars are folded into one float4 and one
// float2.  Taken when every 16-byte copy is aligned (row width, head size and value size multiples of 4).
constexpr int DL2_PT = 16, DL2_TT = 16, DL2_NS = 8, DL2_CPT = 2, DL2_THREADS = (DL2_PT / DL2_CPT) * DL2_NS;

__device__ __forceinline__ void cp_async16(void* smem_dst, const void* gsrc, bool on) {
  const uint32_t d = (uint32_t)__cvta_generic_to_shared(smem_dst);
  const int n = on ? 16 : 0;          // 0 bytes read: the 16 bytes are filled with zeros
  asm volatile("cp.async.cg.shared.global [%0], [%1], 16, %2;" ::"r"(d), "l"(gsrc), "r"(n));
}

template <typename T, int DPT>           // DPT key channels per lane: 16 (D <= 128) or 32 (D <= 256)
__global__ void __launch_bounds__(DL2_THREADS) gated_delta_scan_wide_kernel(DeltaScanParams p) {
  extern __shared__ __align__(16) float sm2[];
  constexpr int THREADS = DL2_THREADS, NS = DL2_NS, CPT = DL2_CPT;
  constexpr int DPAD = DPT * NS;                           // staged key channels (zero past D)
  constexpr int DP = DPAD + (DPAD / 16) * 4 + 4;           // row stride: 4 floats after every 16, 4 more so that rows start 4 banks apart
  constexpr int STAGE = 2 * DL2_TT * DP + DL2_TT * DL2_PT; // q rows, k rows, v tile
  constexpr int QPART = DPAD / 4;                          // channels per thread in the norm phase (4 threads per step)
  float* stage0 = sm2;
  float4* coefA = reinterpret_cast<float4*>(sm2 + 2 * STAGE);           // [TT] decay, decay / |k|, beta, 1 / |k|
  float2* coefB = reinterpret_cast<float2*>(coefA + DL2_TT);            // [TT] decay D^-1/2 / |q|, unit k . scaled unit q
  float* os = reinterpret_cast<float*>(coefB + DL2_TT);                 // [TT][PT]
  const int D = p.D, Dv = p.Dv;
  const int b = blockIdx.z, h = blockIdx.y, p0 = blockIdx.x * DL2_PT;
  const int n_tok = p.q_len[b];
  if (n_tok <= 0) return;
  const int tid = threadIdx.x, pl = tid / NS, ns = tid % NS;            // pl: this thread's pair of columns
  const int nt = tid / 4, npart = tid % 4;                              // norm phase: step and quarter of the row
  const int gq = h / (p.nh / p.n_qk);
  const int Cq = p.n_qk * D, C = 2 * Cq + p.nh * Dv;
  float* Sg = p.state + ((long long)p.lines[b] * p.nh + h) * D * Dv;
  float S[CPT][DPT];
  const bool has_ctx = p.ctx_len[b] > 0;
#pragma unroll
  for (int c = 0; c < CPT; ++c)
#pragma unroll
    for (int i = 0; i < DPT; ++i) {
      const int d = ns * DPT + i, pc = p0 + pl * CPT + c;
      S[c][i] = (has_ctx && pc < Dv && d < D) ? Sg[(long long)d * Dv + pc] : 0.f;
    }
  const float negA = -expf(p.A_log[h]), dtb = p.dt_bias[h], qmul = 1.f / sqrtf((float)D);
  const float* xrow = p.qkv + (long long)b * p.T * C;
  const T* bp = (const T*)p.beta_raw + (long long)b * p.beta_sb + h;
  const T* ap = (const T*)p.a_raw + (long long)b * p.a_sb + h;
  float rbeta = 0.f, ra = 0.f;           // raw beta / a of step `nt` of the batch in flight (thread (nt, 0) turns them into coefficients)
  auto issue = [&](int t0, int st) {
    const int tt = min(DL2_TT, n_tok - t0);
    float* qd = stage0 + st * STAGE;
    float* kd = qd + DL2_TT * DP;
    float* vd = kd + DL2_TT * DP;
    constexpr int CPR = DPAD / 4;          // 16-byte chunks per staged row
    for (int c = tid; c < DL2_TT * CPR; c += THREADS) {
      const int t = c / CPR, d = (c % CPR) * 4;
      const bool on = t < tt && d < D;
      const float* src = on ? xrow + (long long)(t0 + t) * C + gq * D + d : xrow;
      const int at = t * DP + d + (d >> 4) * 4;
      cp_async16(qd + at, src, on);
      cp_async16(kd + at, on ? src + Cq : xrow, on);
    }
    for (int c = tid; c < DL2_TT * (DL2_PT / 4); c += THREADS) {
      const int t = c / (DL2_PT / 4), col = (c % (DL2_PT / 4)) * 4;
      const bool on = t < tt && p0 + col < Dv;
      cp_async16(vd + t * DL2_PT + col, on ? xrow + (long long)(t0 + t) * C + 2 * Cq + h * Dv + p0 + col : xrow, on);
    }
    asm volatile("cp.async.commit_group;");
    const bool mine = npart == 0 && nt < tt;
    rbeta = mine ? ldf(bp + (long long)(t0 + nt) * p.beta_st) : 0.f;
    ra = mine ? ldf(ap + (long long)(t0 + nt) * p.a_st) : 0.f;
  };
  issue(0, 0);
  int st = 0;
  for (int t0 = 0; t0 < n_tok; t0 += DL2_TT, st ^= 1) {
    const int tt = min(DL2_TT, n_tok - t0);
    asm volatile("cp.async.wait_group 0;");
    __syncthreads();                      // this batch has landed; everyone is done with the other stage, the coefficients and the outputs
    const float* qs = stage0 + st * STAGE;
    const float* ks = qs + DL2_TT * DP;
    const float* vs = ks + DL2_TT * DP;
    {
      // thread (nt, npart): a quarter of step nt's raw q and k
      const float4* Kt = reinterpret_cast<const float4*>(ks + nt * DP) + npart * (QPART * 5 / 16);
      const float4* Qt = reinterpret_cast<const float4*>(qs + nt * DP) + npart * (QPART * 5 / 16);
      float qq = 0.f, kk = 0.f, kq = 0.f;
#pragma unroll
      for (int q = 0; q < QPART / 4; ++q) {
        const float4 a = Qt[q + (q >> 2)], c = Kt[q + (q >> 2)];
        qq += a.x * a.x + a.y * a.y + a.z * a.z + a.w * a.w;
        kk += c.x * c.x + c.y * c.y + c.z * c.z + c.w * c.w;
        kq += a.x * c.x + a.y * c.y + a.z * c.z + a.w * c.w;
      }
#pragma unroll
      for (int o = 2; o > 0; o >>= 1) {
        qq += __shfl_xor_sync(0xffffffffu, qq, o);
        kk += __shfl_xor_sync(0xffffffffu, kk, o);
        kq += __shfl_xor_sync(0xffffffffu, kq, o);
      }
      if (npart == 0) {
        const float v = ra + dtb;
        const float sp = v > 20.f ? v : log1pf(expf(v));
        const float g = expf(negA * sp), beta = sigmoidf_acc(rbeta);
        const float iq = qmul / sqrtf(qq + p.unit_eps), ik = 1.f / sqrtf(kk + p.unit_eps);
        coefA[nt] = make_float4(g, g * ik, beta, ik);
        coefB[nt] = make_float2(g * iq, kq * iq * ik);
      }
    }
    __syncthreads();
    if (t0 + DL2_TT < n_tok) issue(t0 + DL2_TT, st ^ 1);      // lands while the current steps are computed
#pragma unroll 2
    for (int t = 0; t < tt; ++t) {
      const float4* Kt = reinterpret_cast<const float4*>(ks + t * DP) + ns * (DPT * 5 / 16);
      const float4* Qt = reinterpret_cast<const float4*>(qs + t * DP) + ns * (DPT * 5 / 16);
      float4 kv[DPT / 4];
      float sk[CPT], sq[CPT];
#pragma unroll
      for (int c = 0; c < CPT; ++c) sk[c] = sq[c] = 0.f;
#pragma unroll
      for (int q = 0; q < DPT / 4; ++q) {
        kv[q] = Kt[q + (q >> 2)];
        const float4 qv = Qt[q + (q >> 2)];
#pragma unroll
        for (int c = 0; c < CPT; ++c) {
          sk[c] += (S[c][4 * q] * kv[q].x + S[c][4 * q + 2] * kv[q].z) + (S[c][4 * q + 1] * kv[q].y + S[c][4 * q + 3] * kv[q].w);
          sq[c] += (S[c][4 * q] * qv.x + S[c][4 * q + 2] * qv.z) + (S[c][4 * q + 1] * qv.y + S[c][4 * q + 3] * qv.w);
        }
      }
#pragma unroll
      for (int o = NS / 2; o > 0; o >>= 1)
#pragma unroll
        for (int c = 0; c < CPT; ++c) {
          sk[c] += __shfl_xor_sync(0xffffffffu, sk[c], o);
          sq[c] += __shfl_xor_sync(0xffffffffu, sq[c], o);
        }
      const float4 cA = coefA[t];
      const float2 cB = coefB[t];
      const float g = cA.x;
#pragma unroll
      for (int c = 0; c < CPT; ++c) {
        const float u = cA.z * (vs[t * DL2_PT + pl * CPT + c] - cA.y * sk[c]);
        const float ku = cA.w * u;
#pragma unroll
        for (int q = 0; q < DPT / 4; ++q) {
          S[c][4 * q] = g * S[c][4 * q] + ku * kv[q].x;
          S[c][4 * q + 1] = g * S[c][4 * q + 1] + ku * kv[q].y;
          S[c][4 * q + 2] = g * S[c][4 * q + 2] + ku * kv[q].z;
          S[c][4 * q + 3] = g * S[c][4 * q + 3] + ku * kv[q].w;
        }
        if (ns == 0) os[t * DL2_PT + pl * CPT + c] = cB.x * sq[c] + u * cB.y;
      }
    }
    __syncthreads();
    for (int i = tid; i < tt * DL2_PT; i += THREADS) {
      const int t = i / DL2_PT, c = p0 + i % DL2_PT;
      if (c < Dv) p.o[((long long)b * p.T + t0 + t) * p.nh * Dv + h * Dv + c] = os[i];
    }
  }
#pragma unroll
  for (int c = 0; c < CPT; ++c)
#pragma unroll
    for (int i = 0; i < DPT; ++i) {
      const int d = ns * DPT + i, pc = p0 + pl * CPT + c;
      if (pc < Dv && d < D) Sg[(long long)d * Dv + pc] = S[c][i];
    }
}

// ---- per-head RMS norm with a shared weight, times an activated gate: one warp per (row, head) ------------------------------------------
template <typename TG, typename TO>
__global__ void __launch_bounds__(128) head_rmsnorm_gate_kernel(const float* __restrict__ y, const float* __restrict__ w, const TG* __restrict__ gate,
                                                                long long g_stride, TO* __restrict__ out, long long nrh, int H, int Dv, float eps,
                                                                int act) {
  const long long i = (long long)blockIdx.x * 4 + (threadIdx.x >> 5);
  if (i >= nrh) return;
  const int lane = threadIdx.x & 31, h = (int)(i % H);
  const long long row = i / H;
  const float* yr = y + i * Dv;
  float v[SEQMIX_MAX_VDIM / 32], ss = 0.f;
#pragma unroll
  for (int k = 0; k < SEQMIX_MAX_VDIM / 32; ++k) {
    const int d = lane + 32 * k;
    v[k] = d < Dv ? yr[d] : 0.f;
    ss += v[k] * v[k];
  }
  const float r = 1.f / sqrtf(warp_sum(ss) / (float)Dv + eps);
  const TG* gr = gate + row * g_stride + (long long)h * Dv;
  TO* orow = out + i * Dv;
#pragma unroll
  for (int k = 0; k < SEQMIX_MAX_VDIM / 32; ++k) {
    const int d = lane + 32 * k;
    if (d < Dv) stf(orow + d, v[k] * r * w[d] * unary_apply(act, ldf(gr + d)));
  }
}

template <typename K>
void opt_in_smem(K kernel, size_t bytes) {
  if (bytes > 48 * 1024) cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)bytes);
}

}  // namespace

void scaled_add_rmsnorm_launch(const float* x, const void* y, bool y_lp, const float* w, float* out, void* out_lp, int rows, int W,
                               float alpha, float eps, float offset, cudaStream_t st) {
  if (rows <= 0) return;
  if (y_lp)
    scaled_add_rmsnorm_kernel<__nv_bfloat16><<<rows, 256, 0, st>>>(x, (const __nv_bfloat16*)y, w, out, (__nv_bfloat16*)out_lp, W, alpha, eps, offset);
  else
    scaled_add_rmsnorm_kernel<float><<<rows, 256, 0, st>>>(x, (const float*)y, w, out, (__nv_bfloat16*)out_lp, W, alpha, eps, offset);
}

void stream_add_rmsnorm_launch(const StreamAddParams& p, bool y_lp, bool h_lp, cudaStream_t st) {
  if (p.rows <= 0) return;
  auto al = [](const void* q, size_t a) { return ((uintptr_t)q & (a - 1)) == 0; };
  const size_t ya = y_lp ? 8 : 16;
  if (p.W % 4 == 0 && p.W <= 8192 && p.W >= 256 && al(p.x, 16) && al(p.y1, ya) && al(p.y2, ya) && al(p.yn, ya) && al(p.wn, 16) && al(p.vec, 16) &&
      al(p.w, 16) && al(p.s, 16) && al(p.s_lp, 8) && al(p.h, h_lp ? 8 : 16)) {
    const int nch = (p.W + 1023) / 1024;
    auto go = [&](auto k1, auto k2, auto k4, auto k8) {
      if (nch <= 1) k1<<<p.rows, 256, 0, st>>>(p);
      else if (nch <= 2) k2<<<p.rows, 256, 0, st>>>(p);
      else if (nch <= 4) k4<<<p.rows, 256, 0, st>>>(p);
      else k8<<<p.rows, 256, 0, st>>>(p);
    };
#define NXDI_STREAM_VEC(TY, TH) go(stream_add_rmsnorm_vec_kernel<TY, TH, 1>, stream_add_rmsnorm_vec_kernel<TY, TH, 2>, \
                                   stream_add_rmsnorm_vec_kernel<TY, TH, 4>, stream_add_rmsnorm_vec_kernel<TY, TH, 8>)
    if (y_lp) { if (h_lp) NXDI_STREAM_VEC(__nv_bfloat16, __nv_bfloat16); else NXDI_STREAM_VEC(__nv_bfloat16, float); }
    else { if (h_lp) NXDI_STREAM_VEC(float, __nv_bfloat16); else NXDI_STREAM_VEC(float, float); }
#undef NXDI_STREAM_VEC
    return;
  }
  const int threads = p.W >= 1024 ? 256 : 128;
  if (y_lp) {
    if (h_lp) stream_add_rmsnorm_kernel<__nv_bfloat16, __nv_bfloat16><<<p.rows, threads, 0, st>>>(p);
    else stream_add_rmsnorm_kernel<__nv_bfloat16, float><<<p.rows, threads, 0, st>>>(p);
  } else {
    if (h_lp) stream_add_rmsnorm_kernel<float, __nv_bfloat16><<<p.rows, threads, 0, st>>>(p);
    else stream_add_rmsnorm_kernel<float, float><<<p.rows, threads, 0, st>>>(p);
  }
}

void latent_norm_append_launch(const void* p, long long p_sb, long long p_st, const float* w, void* cache, const int* block_table,
                               const int* ctx_len, const int* q_len, int B, int T, int R, int page, int max_blocks, float eps, bool lp,
                               void* rows_out, int rot, const float* cos, const float* sin, const void* q_in, int q_rank, const float* q_w,
                               void* q_out, cudaStream_t st) {
  if (B <= 0 || T <= 0) return;
  const unsigned grid = (unsigned)(((long long)B * T + 7) / 8);
  if (lp)
    latent_norm_append_kernel<__nv_bfloat16><<<grid, 256, 0, st>>>((const __nv_bfloat16*)p, p_sb, p_st, w, (__nv_bfloat16*)cache, block_table, ctx_len,
                                                                   q_len, B, T, R, page, max_blocks, eps, (__nv_bfloat16*)rows_out, rot, cos, sin,
                                                                   (const __nv_bfloat16*)q_in, q_rank, q_w, (__nv_bfloat16*)q_out);
  else
    latent_norm_append_kernel<float><<<grid, 256, 0, st>>>((const float*)p, p_sb, p_st, w, (float*)cache, block_table, ctx_len, q_len, B, T, R, page,
                                                           max_blocks, eps, (float*)rows_out, rot, cos, sin, (const float*)q_in, q_rank, q_w,
                                                           (float*)q_out);
}

void rope_half_tail_launch(const void* src, void* dst, const float* cos, const float* sin, long long tokens, int H, int Ds, int Dd, int rot, bool lp,
                           cudaStream_t st) {
  const long long n = tokens * H * (rot / 2);
  if (n <= 0) return;
  const unsigned grid = (unsigned)((n + 255) / 256);
  if (lp) rope_half_tail_kernel<__nv_bfloat16><<<grid, 256, 0, st>>>((const __nv_bfloat16*)src, (__nv_bfloat16*)dst, cos, sin, n, H, Ds, Dd, rot);
  else rope_half_tail_kernel<float><<<grid, 256, 0, st>>>((const float*)src, (float*)dst, cos, sin, n, H, Ds, Dd, rot);
}

void stream_norm_conv_launch(const StreamConvParams& p, bool out_lp, cudaStream_t st) {
  if (p.B <= 0 || p.T <= 0) return;
  dim3 grid(p.T, p.B);
  auto al = [](const void* q, size_t a) { return ((uintptr_t)q & (a - 1)) == 0; };
  const int vt = p.W <= 512 ? 128 : (p.W <= 4096 ? 256 : 512);
  const int need = (p.W + 4 * vt - 1) / (4 * vt), nch = need <= 1 ? 1 : (need <= 2 ? 2 : 4);
  if (p.W % 4 == 0 && p.K <= 4 && need <= 4 && al(p.x, 16) && al(p.y1, p.y1_lp ? 8 : 16) && al(p.y2, p.y2_lp ? 8 : 16) && al(p.w, 16) && al(p.cw, 16) &&
      al(p.state, 16) && al(p.s, 16) && al(p.out, out_lp ? 8 : 16)) {
    if (p.W <= 4096 && p.T >= 2) {
      // portions: two tokens per block share the rows they read (K + 1 rows instead of 2 K); 4 to 16 channels per thread
      const int tt = p.W <= 1024 ? 128 : 256;
      const int nc = p.W <= 4 * tt ? 1 : (p.W <= 8 * tt ? 2 : 4);
      dim3 tg((p.T + 1) / 2, p.B);
#define NXDI_SNT(TO, KK) if (nc == 4) stream_norm_conv_tile_kernel<TO, KK, 4, 2><<<tg, tt, 0, st>>>(p); \
                         else if (nc == 2) stream_norm_conv_tile_kernel<TO, KK, 2, 2><<<tg, tt, 0, st>>>(p); \
                         else stream_norm_conv_tile_kernel<TO, KK, 1, 2><<<tg, tt, 0, st>>>(p)
#define NXDI_SNT_K(TO) switch (p.K) { case 1: NXDI_SNT(TO, 1); break; case 2: NXDI_SNT(TO, 2); break; case 3: NXDI_SNT(TO, 3); break; default: NXDI_SNT(TO, 4); }
      if (out_lp) { NXDI_SNT_K(__nv_bfloat16) } else { NXDI_SNT_K(float) }
#undef NXDI_SNT_K
#undef NXDI_SNT
      return;
    }
    auto go = [&](auto k1, auto k2, auto k4) {
      if (nch == 1) k1<<<grid, vt, 0, st>>>(p);
      else if (nch == 2) k2<<<grid, vt, 0, st>>>(p);
      else k4<<<grid, vt, 0, st>>>(p);
    };
#define NXDI_SNC(TO, KK) go(stream_norm_conv_vec_kernel<TO, KK, 1>, stream_norm_conv_vec_kernel<TO, KK, 2>, stream_norm_conv_vec_kernel<TO, KK, 4>)
#define NXDI_SNC_K(TO) switch (p.K) { case 1: NXDI_SNC(TO, 1); break; case 2: NXDI_SNC(TO, 2); break; case 3: NXDI_SNC(TO, 3); break; default: NXDI_SNC(TO, 4); }
    if (out_lp) { NXDI_SNC_K(__nv_bfloat16) } else { NXDI_SNC_K(float) }
#undef NXDI_SNC_K
#undef NXDI_SNC
    return;
  }
  const int threads = p.W >= 1024 ? 256 : 128;
  if (out_lp) stream_norm_conv_kernel<__nv_bfloat16><<<grid, threads, 0, st>>>(p);
  else stream_norm_conv_kernel<float><<<grid, threads, 0, st>>>(p);
}

void identity_expert_add_launch(void* y, const void* x, const float* topk_w, const int* topk_i, int N, int H, int k, int num_experts, bool lp,
                                cudaStream_t st) {
  if (N <= 0) return;
  if (lp) identity_expert_add_kernel<__nv_bfloat16><<<N, 128, 0, st>>>((__nv_bfloat16*)y, (const __nv_bfloat16*)x, topk_w, topk_i, H, k, num_experts);
  else identity_expert_add_kernel<float><<<N, 128, 0, st>>>((float*)y, (const float*)x, topk_w, topk_i, H, k, num_experts);
}

void head_gate_mul_launch(void* x, const void* gate, long long g_stride, long long rows, int H, int D, bool lp, cudaStream_t st) {
  const int V = lp ? 8 : 4;
  const long long nvec = rows * H * (D / V);
  if (nvec <= 0) return;
  const unsigned grid = (unsigned)((nvec + 255) / 256);
  if (lp) head_gate_mul_kernel<__nv_bfloat16><<<grid, 256, 0, st>>>((__nv_bfloat16*)x, (const __nv_bfloat16*)gate, g_stride, nvec, H, D / V);
  else head_gate_mul_kernel<float><<<grid, 256, 0, st>>>((float*)x, (const float*)gate, g_stride, nvec, H, D / V);
}

void gated_act_mul_launch(const void* gate, long long g_stride, const void* other, long long o_stride, void* out, long long rows, int C, int act,
                          bool on_other, bool lp, cudaStream_t st) {
  const long long n = rows * C;
  if (n <= 0) return;
  const int V = lp ? 8 : 4;
  if (C % V == 0 && o_stride % V == 0 && g_stride % V == 0 && (((uintptr_t)gate | (uintptr_t)other | (uintptr_t)out) & 15) == 0) {
    const long long nvec = n / V;
    const unsigned gv = (unsigned)((nvec + 255) / 256);
    if (lp)
      act_vec_kernel<__nv_bfloat16, true><<<gv, 256, 0, st>>>((const __nv_bfloat16*)gate, (const __nv_bfloat16*)other, o_stride, (__nv_bfloat16*)out, nvec,
                                                              C / V, act, g_stride, (int)on_other);
    else
      act_vec_kernel<float, true><<<gv, 256, 0, st>>>((const float*)gate, (const float*)other, o_stride, (float*)out, nvec, C / V, act, g_stride,
                                                      (int)on_other);
    return;
  }
  const unsigned grid = (unsigned)((n + 255) / 256);
  if (lp)
    gated_act_mul_kernel<__nv_bfloat16><<<grid, 256, 0, st>>>((const __nv_bfloat16*)gate, g_stride, (const __nv_bfloat16*)other, o_stride,
                                                              (__nv_bfloat16*)out, rows, C, act, (int)on_other);
  else
    gated_act_mul_kernel<float><<<grid, 256, 0, st>>>((const float*)gate, g_stride, (const float*)other, o_stride, (float*)out, rows, C, act,
                                                      (int)on_other);
}

void unary_act_launch(const void* x, void* out, long long n, int act, bool lp, cudaStream_t st) {
  if (n <= 0) return;
  const int V = lp ? 8 : 4;
  if (n % V == 0 && (((uintptr_t)x | (uintptr_t)out) & 15) == 0) {
    const long long nvec = n / V;
    const unsigned gv = (unsigned)((nvec + 255) / 256);
    if (lp) act_vec_kernel<__nv_bfloat16, false><<<gv, 256, 0, st>>>((const __nv_bfloat16*)x, nullptr, 0, (__nv_bfloat16*)out, nvec, 1, act);
    else act_vec_kernel<float, false><<<gv, 256, 0, st>>>((const float*)x, nullptr, 0, (float*)out, nvec, 1, act);
    return;
  }
  const unsigned grid = (unsigned)((n + 255) / 256);
  if (lp) unary_act_kernel<__nv_bfloat16><<<grid, 256, 0, st>>>((const __nv_bfloat16*)x, (__nv_bfloat16*)out, n, act);
  else unary_act_kernel<float><<<grid, 256, 0, st>>>((const float*)x, (float*)out, n, act);
}

void short_conv_launch(const void* u, long long u_sb, long long u_st, const float* w, const float* bias, const void* state,
                       const int* lines, const int* ctx_len, const int* q_len, float* y, int B, int T, int C, int K, bool silu, bool lp,
                       cudaStream_t st) {
  if (B <= 0 || T <= 0) return;
  dim3 grid(T, (C + 255) / 256, B);
  if (lp)
    short_conv_kernel<__nv_bfloat16><<<grid, 256, 0, st>>>((const __nv_bfloat16*)u, u_sb, u_st, w, bias, (const __nv_bfloat16*)state, lines,
                                                           ctx_len, q_len, y, T, C, K, silu);
  else
    short_conv_kernel<float><<<grid, 256, 0, st>>>((const float*)u, u_sb, u_st, w, bias, (const float*)state, lines, ctx_len, q_len, y, T, C, K, silu);
}

void short_conv_update_launch(const void* u, long long u_sb, long long u_st, void* state, const int* lines, const int* ctx_len,
                              const int* q_len, int B, int T, int C, int K, bool lp, cudaStream_t st) {
  if (B <= 0 || K <= 1) return;
  dim3 grid((C + 255) / 256, B);
  if (lp)
    short_conv_update_kernel<__nv_bfloat16><<<grid, 256, 0, st>>>((const __nv_bfloat16*)u, u_sb, u_st, (__nv_bfloat16*)state, lines, ctx_len, q_len, C, K);
  else
    short_conv_update_kernel<float><<<grid, 256, 0, st>>>((const float*)u, u_sb, u_st, (float*)state, lines, ctx_len, q_len, C, K);
}

void conv_qknorm_rope_append_launch(const ConvQkParams& p, bool lp, cudaStream_t st) {
  if (p.B <= 0 || p.T <= 0) return;
  const size_t smem = sizeof(float) * (size_t)(p.n_q * p.D + p.n_kv * (p.D + p.Dv));
  dim3 grid(p.T, p.B);
  const size_t esz = lp ? 2 : 4;
  const bool pairs = p.Dv % 2 == 0 && p.R % 2 == 0 && p.p_sb % 2 == 0 && p.p_st % 2 == 0 && ((uintptr_t)p.p % (2 * esz)) == 0;
  auto go = [&](auto kernel) {
    opt_in_smem(kernel, smem);
    kernel<<<grid, 256, smem, st>>>(p);
  };
  if (lp) {
    if (pairs) go(conv_qknorm_rope_append_pair_kernel<__nv_bfloat16>); else go(conv_qknorm_rope_append_kernel<__nv_bfloat16>);
  } else {
    if (pairs) go(conv_qknorm_rope_append_pair_kernel<float>); else go(conv_qknorm_rope_append_kernel<float>);
  }
}

void paged_window_attention_launch(const WindowAttnParams& p, bool lp, cudaStream_t st) {
  const long long nq = (long long)p.B * p.T * p.Hq;
  if (nq <= 0) return;
  // values that are a prefix of the key rows of the same cache (latent rows with a rotated tail): one shared-memory tile serves both
  const bool prefix = p.v_cache == p.k_cache && p.v_rs == p.D && p.G == 1;
  const bool rows16 = (p.v_rs * 2) % 16 == 0;
  if (lp && p.T >= 16 && rows16 && ((!prefix && (p.D == 64 || p.D == 128) && (p.Dv == 64 || p.Dv == 128)) ||
                                    (prefix && ((p.D == 80 && p.Dv == 64) || (p.D == 192 && p.Dv == 128) || (p.D == p.Dv && (p.D == 64 || p.D == 128)))))) {
    // prompt portions in bf16: tensor-core kernel
    dim3 grid((p.T + MMA_MT - 1) / MMA_MT, p.Hq, p.B);
    const size_t smem = 2 * (size_t)MMA_KT * (prefix ? p.D + 8 : p.D + 8 + p.Dv + 8) * sizeof(__nv_bfloat16);
    auto go = [&](auto kernel) {
      opt_in_smem(kernel, smem);
      kernel<<<grid, 128, smem, st>>>(p);
    };
    if (prefix) {
      if (p.D == 80) go(paged_window_attention_mma_kernel<80, 64, true>);
      else if (p.D == 192) go(paged_window_attention_mma_kernel<192, 128, true>);
      else if (p.D == 64) go(paged_window_attention_mma_kernel<64, 64, true>);
      else go(paged_window_attention_mma_kernel<128, 128, true>);
    } else if (p.D == 64 && p.Dv == 64) go(paged_window_attention_mma_kernel<64, 64, false>);
    else if (p.D == 64) go(paged_window_attention_mma_kernel<64, 128, false>);
    else if (p.Dv == 64) go(paged_window_attention_mma_kernel<128, 64, false>);
    else go(paged_window_attention_mma_kernel<128, 128, false>);
    return;
  }
  // few queries (decode steps): one block per query, its warps split the keys; otherwise one warp per query
  const bool split = nq <= 2LL * kNumSMs * 4;
  // split mode: one warp per 32 visible keys (bounded by the window or by the pages a row can hold), 4 to 32 warps
  long long span = (long long)p.max_blocks * p.page;
  if (p.window > 0) span = std::min<long long>(span, (long long)p.window + p.keep_first);
  if (p.chunk > 0) span = std::min<long long>(span, (long long)p.chunk);
  const int nwarps = split ? (int)std::min<long long>(32, std::max<long long>(ATT_WARPS, (span + 31) / 32)) : ATT_WARPS;
  const size_t smem = sizeof(float) * (size_t)(nwarps * (p.D + p.Dv + 2));
  const unsigned grid = (unsigned)(split ? nq : (nq + ATT_WARPS - 1) / ATT_WARPS);
  auto go = [&](auto kernel) {
    opt_in_smem(kernel, smem);
    kernel<<<grid, nwarps * 32, smem, st>>>(p);
  };
  if (lp) {
    if (split) go(paged_window_attention_kernel<__nv_bfloat16, true>); else go(paged_window_attention_kernel<__nv_bfloat16, false>);
  } else {
    if (split) go(paged_window_attention_kernel<float, true>); else go(paged_window_attention_kernel<float, false>);
  }
}

void ssd_scan_launch(const SsdScanParams& p, bool lp, cudaStream_t st) {
  if (p.B <= 0 || p.T <= 0) return;
  const size_t smem = sizeof(float) * (size_t)(2 * SCAN_TT * 160 * (p.N <= 128 ? 1 : 2) + 3 * SCAN_TT * SCAN_PT + 2 * SCAN_TT);
  dim3 grid((p.P + SCAN_PT - 1) / SCAN_PT, p.nh, p.B);
  auto go = [&](auto kernel) {
    opt_in_smem(kernel, smem);
    kernel<<<grid, SCAN_THREADS, smem, st>>>(p);
  };
  if (p.N <= 128) {
    if (lp) go(ssd_scan_kernel<__nv_bfloat16, 1>); else go(ssd_scan_kernel<float, 1>);
  } else {
    if (lp) go(ssd_scan_kernel<__nv_bfloat16, 2>); else go(ssd_scan_kernel<float, 2>);
  }
}

void stream_sandwich_norm_launch(const SandwichParams& p, bool y_lp, bool h_lp, cudaStream_t st) {
  if (p.rows <= 0) return;
  const size_t smem = sizeof(float) * (size_t)p.W;
  const uintptr_t ptrs = (uintptr_t)p.x | (uintptr_t)p.a | (uintptr_t)p.b | (uintptr_t)p.a_w | (uintptr_t)p.b_w | (uintptr_t)p.post_w | (uintptr_t)p.ls |
                         (uintptr_t)p.next_w | (uintptr_t)p.s | (uintptr_t)p.h;
  if (p.W % 4 == 0 && p.W <= 8192 && (ptrs & 15) == 0) {
    // the mixed-type instantiations (bf16 results into an fp32 norm and the reverse) stay on the scalar kernel
    auto pick = [&](auto ty, auto th) {
      using TY = decltype(ty);
      using TH = decltype(th);
      if (p.W <= 1024) stream_sandwich_norm_vec_kernel<TY, TH, 1><<<p.rows, 256, 0, st>>>(p);
      else if (p.W <= 2048) stream_sandwich_norm_vec_kernel<TY, TH, 2><<<p.rows, 256, 0, st>>>(p);
      else if (p.W <= 4096) stream_sandwich_norm_vec_kernel<TY, TH, 4><<<p.rows, 256, 0, st>>>(p);
      else stream_sandwich_norm_vec_kernel<TY, TH, 8><<<p.rows, 256, 0, st>>>(p);
    };
    if (y_lp && h_lp) { pick(__nv_bfloat16{}, __nv_bfloat16{}); return; }
    if (!y_lp && !h_lp) { pick(float{}, float{}); return; }
  }
  auto go = [&](auto kernel) {
    opt_in_smem(kernel, smem);
    kernel<<<p.rows, 256, smem, st>>>(p);
  };
  if (y_lp) {
    if (h_lp) go(stream_sandwich_norm_kernel<__nv_bfloat16, __nv_bfloat16>); else go(stream_sandwich_norm_kernel<__nv_bfloat16, float>);
  } else {
    if (h_lp) go(stream_sandwich_norm_kernel<float, __nv_bfloat16>); else go(stream_sandwich_norm_kernel<float, float>);
  }
}

void head_norm_rope_append_launch(const HeadNormRopeParams& p, bool lp, cudaStream_t st) {
  if (p.B <= 0 || p.T <= 0) return;
  dim3 grid(p.T, p.B);
  const int vpl = p.D / 32;
  const size_t esz = lp ? 2 : 4;
  // one vector access per lane: head size 64 / 128 / 256, rotated halves in whole lanes, every row a multiple of the access size
  const bool lanes = p.D % 32 == 0 && (vpl == 2 || vpl == 4 || vpl == 8) && (!p.cos || (p.R / 2) % vpl == 0) && (!p.value_from_key || p.Dv == p.D) &&
                     ((uintptr_t)p.p % 16) == 0 && (p.p_sb * esz) % 16 == 0 && (p.p_st * esz) % 16 == 0;
  if (lanes) {
    auto go = [&](auto kernel) { kernel<<<grid, HNR_WARPS * 32, 0, st>>>(p); };
    if (lp) {
      if (vpl == 2) go(head_norm_rope_append_lane_kernel<__nv_bfloat16, 2>);
      else if (vpl == 4) go(head_norm_rope_append_lane_kernel<__nv_bfloat16, 4>);
      else go(head_norm_rope_append_lane_kernel<__nv_bfloat16, 8>);
    } else {
      if (vpl == 2) go(head_norm_rope_append_lane_kernel<float, 2>);
      else if (vpl == 4) go(head_norm_rope_append_lane_kernel<float, 4>);
      else go(head_norm_rope_append_lane_kernel<float, 8>);
    }
    return;
  }
  if (lp) head_norm_rope_append_kernel<__nv_bfloat16><<<grid, HNR_WARPS * 32, 0, st>>>(p);
  else head_norm_rope_append_kernel<float><<<grid, HNR_WARPS * 32, 0, st>>>(p);
}

void gated_delta_scan_launch(const DeltaScanParams& p, bool lp, cudaStream_t st) {
  if (p.B <= 0 || p.T <= 0) return;
  const int nb = p.D <= 128 ? 1 : 2;
  dim3 grid((p.Dv + DLT_PT - 1) / DLT_PT, p.nh, p.B);
  const long long C = 2LL * p.n_qk * p.D + (long long)p.nh * p.Dv;
  if (p.D % 4 == 0 && p.Dv % 4 == 0 && C % 4 == 0 && ((uintptr_t)p.qkv % 16) == 0) {
    // every 16-byte copy of q / k / v rows is aligned: the two-stage kernel with two state columns per thread
    const int dpad = 16 * nb * DL2_NS, dp = dpad + (dpad / 16) * 4 + 4;
    const size_t smem2 = sizeof(float) * (size_t)(2 * (2 * DL2_TT * dp + DL2_TT * DL2_PT) + 4 * DL2_TT + 2 * DL2_TT + DL2_TT * DL2_PT);
    auto go2 = [&](auto kernel) {
      opt_in_smem(kernel, smem2);
      kernel<<<grid, DL2_THREADS, smem2, st>>>(p);
    };
    if (nb == 1) {
      if (lp) go2(gated_delta_scan_wide_kernel<__nv_bfloat16, 16>); else go2(gated_delta_scan_wide_kernel<float, 16>);
    } else {
      if (lp) go2(gated_delta_scan_wide_kernel<__nv_bfloat16, 32>); else go2(gated_delta_scan_wide_kernel<float, 32>);
    }
    return;
  }
  const size_t smem = sizeof(float) * (size_t)(2 * DLT_TT * 160 * nb + 2 * DLT_TT * DLT_PT + 5 * DLT_TT);
  auto go = [&](auto kernel) {
    opt_in_smem(kernel, smem);
    kernel<<<grid, DLT_THREADS, smem, st>>>(p);
  };
  if (nb == 1) {
    if (lp) go(gated_delta_scan_kernel<__nv_bfloat16, 1>); else go(gated_delta_scan_kernel<float, 1>);
  } else {
    if (lp) go(gated_delta_scan_kernel<__nv_bfloat16, 2>); else go(gated_delta_scan_kernel<float, 2>);
  }
}

void head_rmsnorm_gate_launch(const float* y, const float* w, const void* gate, long long g_stride, void* out, long long rows, int H, int Dv,
                              float eps, int act, bool gate_lp, bool out_lp, cudaStream_t st) {
  const long long nrh = rows * H;
  if (nrh <= 0) return;
  const unsigned grid = (unsigned)((nrh + 3) / 4);
  if (gate_lp) {
    if (out_lp) head_rmsnorm_gate_kernel<__nv_bfloat16, __nv_bfloat16><<<grid, 128, 0, st>>>(y, w, (const __nv_bfloat16*)gate, g_stride, (__nv_bfloat16*)out, nrh, H, Dv, eps, act);
    else head_rmsnorm_gate_kernel<__nv_bfloat16, float><<<grid, 128, 0, st>>>(y, w, (const __nv_bfloat16*)gate, g_stride, (float*)out, nrh, H, Dv, eps, act);
  } else {
    if (out_lp) head_rmsnorm_gate_kernel<float, __nv_bfloat16><<<grid, 128, 0, st>>>(y, w, (const float*)gate, g_stride, (__nv_bfloat16*)out, nrh, H, Dv, eps, act);
    else head_rmsnorm_gate_kernel<float, float><<<grid, 128, 0, st>>>(y, w, (const float*)gate, g_stride, (float*)out, nrh, H, Dv, eps, act);
  }
}

void group_rmsnorm_launch(const float* y, const float* w, void* out, bool out_lp, int rows, int W, int groups, float eps, cudaStream_t st) {
  if (rows <= 0) return;
  dim3 grid(rows, groups);
  if (out_lp)
    group_rmsnorm_kernel<__nv_bfloat16><<<grid, 256, 0, st>>>(y, w, (__nv_bfloat16*)out, W, W / groups, eps);
  else
    group_rmsnorm_kernel<float><<<grid, 256, 0, st>>>(y, w, (float*)out, W, W / groups, eps);
}

void clamped_glu_launch(const void* gu, void* out, long long rows, int F, float limit, float alpha, bool lp, cudaStream_t st) {
  const long long n = rows * F;
  if (n <= 0) return;
  const int vn = lp ? 8 : 4;
  if (F % vn == 0 && ((uintptr_t)gu % 16) == 0 && ((uintptr_t)out % 16) == 0) {
    const unsigned grid = (unsigned)((n / vn + 255) / 256);
    if (lp)
      clamped_glu_vec_kernel<__nv_bfloat16><<<grid, 256, 0, st>>>((const __nv_bfloat16*)gu, (__nv_bfloat16*)out, rows, F, limit, alpha);
    else
      clamped_glu_vec_kernel<float><<<grid, 256, 0, st>>>((const float*)gu, (float*)out, rows, F, limit, alpha);
    return;
  }
  const unsigned grid = (unsigned)((n + 255) / 256);
  if (lp)
    clamped_glu_kernel<__nv_bfloat16><<<grid, 256, 0, st>>>((const __nv_bfloat16*)gu, (__nv_bfloat16*)out, rows, F, limit, alpha);
  else
    clamped_glu_kernel<float><<<grid, 256, 0, st>>>((const float*)gu, (float*)out, rows, F, limit, alpha);
}

}  // namespace nxdi
