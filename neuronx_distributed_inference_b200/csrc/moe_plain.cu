// Two-matrix experts y = W_down act(W_up x) for activations in bf16 or fp32 and for any sizes: the CUDA-core companion of the grouped
// tcgen05 path (moe_grouped.cu), which needs bf16 and sizes in multiples of 64.  The permutation is the same one (moe_plan_kernel:
// every expert's rows padded to whole 128-row tiles, static row bound, no host synchronisation):
//
//   gather    xp[row] = x[token(row)], zero rows for padding
//   GEMM 1    h = act(xp W_up[e]^T)       64 x 64 output tiles, fp32 accumulation, the expert of a tile from the tile table
//   GEMM 2    y = h W_down[e]^T
//   combine   out[token] = sum_slot affinity * y[pos[token, slot]]     (fp32, fixed slot order)
//
// and for a handful of tokens (decode steps) two weight-streaming kernels without any permutation: one warp per (entry, hidden unit),
// then one warp per (token, output channel) that walks the token's chosen experts.  Compiled WITHOUT fast-math: the fp32 instantiation
// is the exact-arithmetic path.
#include <cuda_bf16.h>

#include <stdexcept>
#include <type_traits>

#include "common.cuh"
#include "seqmix.h"

namespace nxdi {
namespace {

template <typename T> __device__ __forceinline__ float ldx(const T* p);
template <> __device__ __forceinline__ float ldx<float>(const float* p) { return *p; }
template <> __device__ __forceinline__ float ldx<__nv_bfloat16>(const __nv_bfloat16* p) { return __bfloat162float(*p); }
template <typename T> __device__ __forceinline__ void stx(T* p, float v);
template <> __device__ __forceinline__ void stx<float>(float* p, float v) { *p = v; }
template <> __device__ __forceinline__ void stx<__nv_bfloat16>(__nv_bfloat16* p, float v) { *p = __float2bfloat16_rn(v); }

__device__ __forceinline__ float act_apply(int act, float v) {
  switch (act) {
    case 1: return fmaxf(v, 0.f);
    case 2: { const float r = fmaxf(v, 0.f); return r * r; }
    case 3: return v / (1.f + expf(-v));
    case 4: return 0.5f * v * (1.f + tanhf(0.7978845608028654f * (v + 0.044715f * v * v * v)));
    case 5: return 1.f / (1.f + expf(-v));
    default: return v;
  }
}

template <typename T>
__global__ void __launch_bounds__(128) gather_kernel(const T* __restrict__ x, const int* __restrict__ row_entry,
                                                     const int* __restrict__ tile_expert, T* __restrict__ xp, int H, int k) {
  const int r = blockIdx.x;
  if (tile_expert[r >> 7] < 0) return;
  const int ent = row_entry[r];
  T* dst = xp + (size_t)r * H;
  if (ent < 0) {
    for (int c = threadIdx.x; c < H; c += 128) stx(dst + c, 0.f);
    return;
  }
  const T* src = x + (size_t)(ent / k) * H;
  for (int c = threadIdx.x; c < H; c += 128) dst[c] = src[c];
}

// C[r, n] = act(sum_k A[r, k] * W[e, n, k]); block = 64 x 64 outputs, 256 threads x (4 x 4), k in slices of 16
constexpr int PT = 64, PK = 16;
template <typename T>
__global__ void __launch_bounds__(256) grouped_gemm_kernel(const T* __restrict__ A, const T* __restrict__ W, T* __restrict__ C, int N, int K,
                                                           int act, const int* __restrict__ tile_expert) {
  const int r0 = blockIdx.y * PT, n0 = blockIdx.x * PT;
  const int e = tile_expert[r0 >> 7];
  if (e < 0) return;
  __shared__ float As[PK][PT + 1], Ws[PK][PT + 1];
  const T* Wb = W + (size_t)e * N * K;
  const int tx = threadIdx.x & 15, ty = threadIdx.x >> 4;
  float acc[4][4] = {};
  for (int k0 = 0; k0 < K; k0 += PK) {
    for (int i = threadIdx.x; i < PT * PK; i += 256) {
      const int rr = i / PK, kk = i % PK;
      const bool ink = k0 + kk < K;
      As[kk][rr] = ink ? ldx(A + (size_t)(r0 + rr) * K + k0 + kk) : 0.f;
      Ws[kk][rr] = (ink && n0 + rr < N) ? ldx(Wb + (size_t)(n0 + rr) * K + k0 + kk) : 0.f;
    }
    __syncthreads();
#pragma unroll
    for (int kk = 0; kk < PK; ++kk) {
      float a[4], w[4];
#pragma unroll
      for (int i = 0; i < 4; ++i) { a[i] = As[kk][ty * 4 + i]; w[i] = Ws[kk][tx * 4 + i]; }
#pragma unroll
      for (int i = 0; i < 4; ++i)
#pragma unroll
        for (int j = 0; j < 4; ++j) acc[i][j] = fmaf(a[i], w[j], acc[i][j]);
    }
    __syncthreads();
  }
#pragma unroll
  for (int i = 0; i < 4; ++i)
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      const int n = n0 + tx * 4 + j;
      if (n < N) stx(C + (size_t)(r0 + ty * 4 + i) * N + n, act_apply(act, acc[i][j]));
    }
}

template <typename T>
__global__ void __launch_bounds__(128) combine_kernel(const T* __restrict__ y, const float* __restrict__ topk_w, const int* __restrict__ pos,
                                                      T* __restrict__ out, int H, int k) {
  const int tok = blockIdx.x;
  __shared__ int s_pos[64];
  __shared__ float s_w[64];
  if ((int)threadIdx.x < k) {
    s_pos[threadIdx.x] = pos[(size_t)tok * k + threadIdx.x];
    s_w[threadIdx.x] = topk_w[(size_t)tok * k + threadIdx.x];
  }
  __syncthreads();
  for (int c = threadIdx.x; c < H; c += 128) {
    float f = 0.f;
    for (int s = 0; s < k; ++s)
      if (s_pos[s] >= 0) f += s_w[s] * ldx(y + (size_t)s_pos[s] * H + c);
    stx(out + (size_t)tok * H + c, f);
  }
}

// dot product of two dense rows by one warp (every lane gets the sum); 16-byte loads when both rows allow them
template <typename T>
__device__ __forceinline__ float warp_dot(const T* a, const T* b, int n, int lane) {
  constexpr int V = 16 / (int)sizeof(T);
  float s = 0.f;
  if (n % V == 0 && (((uintptr_t)a | (uintptr_t)b) & 15) == 0) {
    for (int c = lane * V; c < n; c += 32 * V) {
      const uint4 ua = *reinterpret_cast<const uint4*>(a + c), ub = __ldg(reinterpret_cast<const uint4*>(b + c));
      if constexpr (V == 4) {
        s = fmaf(__uint_as_float(ua.x), __uint_as_float(ub.x), s); s = fmaf(__uint_as_float(ua.y), __uint_as_float(ub.y), s);
        s = fmaf(__uint_as_float(ua.z), __uint_as_float(ub.z), s); s = fmaf(__uint_as_float(ua.w), __uint_as_float(ub.w), s);
      } else {
        s = fmaf(bf16lo(ua.x), bf16lo(ub.x), s); s = fmaf(bf16hi(ua.x), bf16hi(ub.x), s);
        s = fmaf(bf16lo(ua.y), bf16lo(ub.y), s); s = fmaf(bf16hi(ua.y), bf16hi(ub.y), s);
        s = fmaf(bf16lo(ua.z), bf16lo(ub.z), s); s = fmaf(bf16hi(ua.z), bf16hi(ub.z), s);
        s = fmaf(bf16lo(ua.w), bf16lo(ub.w), s); s = fmaf(bf16hi(ua.w), bf16hi(ub.w), s);
      }
    }
  } else {
    for (int c = lane; c < n; c += 32) s = fmaf(ldx(a + c), ldx(b + c), s);
  }
  return warp_sum(s);
}

// h[entry, i] = act(x[token] . W_up[e, i, :]); one warp per (entry, i)
template <typename T>
__global__ void __launch_bounds__(256) decode_up_kernel(const T* __restrict__ x, const T* __restrict__ w_up, const int* __restrict__ topk_i,
                                                        T* __restrict__ h, int entries, int k, int H, int I, int expert_offset, int e_local,
                                                        int act, int gated) {
  const int lane = threadIdx.x & 31;
  const long long wid = (long long)blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5);
  if (wid >= (long long)entries * I) return;
  const int ent = (int)(wid / I), i = (int)(wid % I);
  const int e = topk_i[ent] - expert_offset;
  if (e < 0 || e >= e_local) return;
  if (gated) {      // w_up holds [gate; up] rows: act(gate . x) * (up . x), each product rounded to the activation type first
    float g = warp_dot(x + (size_t)(ent / k) * H, w_up + ((size_t)e * 2 * I + i) * H, H, lane);
    float u = warp_dot(x + (size_t)(ent / k) * H, w_up + ((size_t)e * 2 * I + I + i) * H, H, lane);
    if constexpr (!std::is_same<T, float>::value) {
      g = __bfloat162float(__float2bfloat16_rn(g));
      u = __bfloat162float(__float2bfloat16_rn(u));
    }
    if (lane == 0) stx(h + (size_t)ent * I + i, act_apply(act, g) * u);
    return;
  }
  const float v = warp_dot(x + (size_t)(ent / k) * H, w_up + ((size_t)e * I + i) * H, H, lane);
  if (lane == 0) stx(h + (size_t)ent * I + i, act_apply(act, v));
}

// out[token, n] = sum_slot affinity * round(h[entry] . W_down[e, n, :]); one warp per (token, n)
template <typename T>
__global__ void __launch_bounds__(256) decode_down_kernel(const T* __restrict__ h, const T* __restrict__ w_down, const float* __restrict__ topk_w,
                                                          const int* __restrict__ topk_i, T* __restrict__ out, int N, int k, int H, int I,
                                                          int expert_offset, int e_local) {
  const int lane = threadIdx.x & 31;
  const long long wid = (long long)blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5);
  if (wid >= (long long)N * H) return;
  const int tok = (int)(wid / H), n = (int)(wid % H);
  float f = 0.f;
  for (int s = 0; s < k; ++s) {
    const int ent = tok * k + s, e = topk_i[ent] - expert_offset;
    if (e < 0 || e >= e_local) continue;
    float v = warp_dot(h + (size_t)ent * I, w_down + ((size_t)e * H + n) * I, I, lane);
    if constexpr (!std::is_same<T, float>::value) v = __bfloat162float(__float2bfloat16_rn(v));     // the expert's output in the activation type
    f += topk_w[ent] * v;
  }
  if (lane == 0) stx(out + (size_t)tok * H + n, f);
}

// ---- fp32 router: logits, sigmoid scores, the k largest, renormalised ----------------------------------------------------------------
// Kernel 1 (logits): block = RT tokens whose rows pass through shared memory as fp32, RKC columns at a time, x 8 warps; a warp forms the
// logits of EG experts for all RT tokens from ONE pass over those experts' weight rows (RT x EG accumulators per lane: EG weight loads
// and RT shared-memory loads feed RT * EG multiply-adds), so the router matrix is read once per RT tokens.  RT = 8 (sixteen tokens per block
// measured slower: fewer resident blocks); EG = 4 for prompt portions, EG = 1 for a handful of tokens, where spreading the experts over
// more blocks matters more than reuse.
// Kernel 2 (selection): one warp per token picks the k largest logits (largest first, lowest index on ties; the sigmoid is monotonic,
// so these are the k largest scores), writes their sigmoid scores and divides them by their sum + eps when eps >= 0.
constexpr int RKC = 1024;      // columns staged per round (4 KB per token), so several blocks share an SM and hide the weight loads
template <typename T, int EG, int RT>
__global__ void __launch_bounds__(256) router_logits_kernel(const T* __restrict__ x, const float* __restrict__ w, float* __restrict__ logits,
                                                            int N, int W, int E) {
  extern __shared__ __align__(16) float rsm[];               // [RT][RKC]
  const int t0 = blockIdx.x * RT, warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int e0 = (blockIdx.y * 8 + warp) * EG;
  const bool active = e0 < E;
  float acc[RT][EG];
#pragma unroll
  for (int t = 0; t < RT; ++t)
#pragma unroll
    for (int g = 0; g < EG; ++g) acc[t][g] = 0.f;
  const float* wr[EG];
#pragma unroll
  for (int g = 0; g < EG; ++g) wr[g] = w + (size_t)min(e0 + g, E - 1) * W;
  for (int k0 = 0; k0 < W; k0 += RKC) {
    const int kc = min(RKC, W - k0);
    if (k0) __syncthreads();
    if (W % 4 == 0) {                     // one 4-wide access per thread and token: 256 threads x 4 = RKC columns
      const int c = threadIdx.x * 4;
#pragma unroll
      for (int t = 0; t < RT; ++t) {
        float4 v = make_float4(0.f, 0.f, 0.f, 0.f);
        if (c < kc && t0 + t < N) {
          const T* src = x + (size_t)(t0 + t) * W + k0 + c;
          if constexpr (std::is_same<T, float>::value) {
            v = *reinterpret_cast<const float4*>(src);
          } else {
            const uint2 r = *reinterpret_cast<const uint2*>(src);
            v = make_float4(bf16lo(r.x), bf16hi(r.x), bf16lo(r.y), bf16hi(r.y));
          }
        }
        *reinterpret_cast<float4*>(rsm + t * RKC + c) = v;
      }
    } else {
      for (int i = threadIdx.x; i < RT * kc; i += 256) {
        const int t = i / kc, c = i % kc;
        rsm[t * RKC + c] = t0 + t < N ? ldx(x + (size_t)(t0 + t) * W + k0 + c) : 0.f;
      }
    }
    __syncthreads();
    if (!active) continue;
    if (W % 4 == 0) {
      for (int c = lane * 4; c < kc; c += 128) {
        float4 wv[EG];
#pragma unroll
        for (int g = 0; g < EG; ++g) wv[g] = __ldg(reinterpret_cast<const float4*>(wr[g] + k0 + c));
#pragma unroll
        for (int t = 0; t < RT; ++t) {
          const float4 xv = *reinterpret_cast<const float4*>(rsm + t * RKC + c);
#pragma unroll
          for (int g = 0; g < EG; ++g)
            acc[t][g] = fmaf(xv.w, wv[g].w, fmaf(xv.z, wv[g].z, fmaf(xv.y, wv[g].y, fmaf(xv.x, wv[g].x, acc[t][g]))));
        }
      }
    } else {
      for (int c = lane; c < kc; c += 32) {
        float wv[EG];
#pragma unroll
        for (int g = 0; g < EG; ++g) wv[g] = __ldg(wr[g] + k0 + c);
#pragma unroll
        for (int t = 0; t < RT; ++t) {
          const float xv = rsm[t * RKC + c];
#pragma unroll
          for (int g = 0; g < EG; ++g) acc[t][g] = fmaf(xv, wv[g], acc[t][g]);
        }
      }
    }
  }
  if (!active) return;
#pragma unroll
  for (int t = 0; t < RT; ++t)
#pragma unroll
    for (int g = 0; g < EG; ++g) {
      const float v = warp_sum(acc[t][g]);
      if (lane == 0 && t0 + t < N && e0 + g < E) logits[(size_t)(t0 + t) * E + e0 + g] = v;
    }
}

__global__ void __launch_bounds__(256) router_select_kernel(const float* __restrict__ logits, float* __restrict__ topk_w, int* __restrict__ topk_i,
                                                            int N, int E, int k, RouterSelect sel) {
  extern __shared__ float zsm[];                             // per warp: [E] scores, [E] choice scores, [groups] group bests
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int tok = blockIdx.x * 8 + warp;
  if (tok >= N) return;
  const int G = sel.groups > 1 ? sel.groups : 0;
  float* sc = zsm + (size_t)warp * (2 * E + G);
  float* ch = sc + E;
  float* gb = ch + E;
  // scores: sigmoid, or softmax over all router outputs
  float mx = -INFINITY;
  for (int e = lane; e < E; e += 32) { const float v = logits[(size_t)tok * E + e]; sc[e] = v; mx = fmaxf(mx, v); }
  if (sel.softmax) {
    mx = warp_max(mx);
    float den = 0.f;
    for (int e = lane; e < E; e += 32) { const float v = expf(sc[e] - mx); sc[e] = v; den += v; }
    den = warp_sum(den);
    for (int e = lane; e < E; e += 32) sc[e] = sc[e] / den;
  } else {
    for (int e = lane; e < E; e += 32) sc[e] = 1.f / (1.f + expf(-sc[e]));
  }
  for (int e = lane; e < E; e += 32) ch[e] = sc[e] + (sel.correction ? sel.correction[e] : 0.f);
  __syncwarp();
  // largest value of an array of n floats, lowest index on ties; every lane gets (value, index)
  auto arg_max = [&](const float* a, int n, float& best, int& bi) {
    best = -INFINITY;
    bi = 0x7fffffff;
    for (int e = lane; e < n; e += 32) {
      const float v = a[e];
      if (v > best || (v == best && e < bi)) { best = v; bi = e; }
    }
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) {
      const float ov = __shfl_xor_sync(0xffffffffu, best, o);
      const int oi = __shfl_xor_sync(0xffffffffu, bi, o);
      if (ov > best || (ov == best && oi < bi)) { best = ov; bi = oi; }
    }
    if (bi >= n) bi = 0;                                     // nothing left to choose from (or not a number): stay inside the array
  };
  if (G) {
    // a group is as good as its best choice score; experts outside the `keep` best groups cannot be chosen
    const int per = E / G;
    for (int g = lane; g < G; g += 32) {
      float m = -INFINITY;
      for (int e = g * per; e < (g + 1) * per; ++e) m = fmaxf(m, ch[e]);
      gb[g] = m;
    }
    __syncwarp();
    for (int j = 0; j < sel.keep; ++j) {
      float best;
      int bg;
      arg_max(gb, G, best, bg);
      if (lane == 0) gb[bg] = NAN;                           // marks the group as kept; NaN never wins a later comparison
      __syncwarp();
    }
    for (int e = lane; e < E; e += 32)
      if (!isnan(gb[e / per])) ch[e] = -INFINITY;            // group not kept
    __syncwarp();
  }
  float sum = 0.f;
  for (int j = 0; j < k; ++j) {
    float best;
    int bi;
    arg_max(ch, E, best, bi);
    const float w = sc[bi];
    sum += w;
    if (lane == 0) {
      topk_w[(size_t)tok * k + j] = w;
      topk_i[(size_t)tok * k + j] = bi;
      ch[bi] = -INFINITY;                                    // taken
    }
    __syncwarp();
  }
  const float mul = (sel.renorm_eps >= 0.f ? 1.f / (sum + sel.renorm_eps) : 1.f) * sel.scale;
  if (mul != 1.f)
    for (int j = lane; j < k; j += 32) topk_w[(size_t)tok * k + j] *= mul;
}

// gated experts: h[r, i] = act(g[r, i]) * g[r, I + i] for the rows of used tiles of the [R, 2 I] first product
template <typename T>
__global__ void __launch_bounds__(256) gate_mul_rows_kernel(const T* __restrict__ gu, T* __restrict__ h, int I, int act,
                                                            const int* __restrict__ tile_expert) {
  const int r = blockIdx.x;
  if (tile_expert[r >> 7] < 0) return;
  const T* row = gu + (size_t)r * 2 * I;
  for (int i = threadIdx.x; i < I; i += 256) stx(h + (size_t)r * I + i, act_apply(act, ldx(row + i)) * ldx(row + I + i));
}

}  // namespace

void router_topk_launch(const void* x, const float* w, float* logits, float* topk_w, int* topk_i, int N, int W, int E, int k,
                        const RouterSelect& sel, bool lp, cudaStream_t st) {
  if (N <= 0) return;
  if (sel.groups > 1 && (E % sel.groups != 0 || sel.keep < 1 || sel.keep > sel.groups)) throw std::runtime_error("router: groups must divide the experts");
  if (k > E) throw std::runtime_error("router: more experts chosen than there are");
  if (E > 4096) throw std::runtime_error("router: more than 4096 experts");
  const bool few = N <= 32;
  const int eg = few ? 1 : 4, rt = 8;
  dim3 grid((N + rt - 1) / rt, (E + 8 * eg - 1) / (8 * eg));
  const size_t smem = sizeof(float) * (size_t)rt * RKC;
  auto go = [&](auto kernel, auto xp) {
    if (smem > 48 * 1024) cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
    kernel<<<grid, 256, smem, st>>>(xp, w, logits, N, W, E);
  };
  if (lp) {
    if (few) go(router_logits_kernel<__nv_bfloat16, 1, 8>, (const __nv_bfloat16*)x); else go(router_logits_kernel<__nv_bfloat16, 4, 8>, (const __nv_bfloat16*)x);
  } else {
    if (few) go(router_logits_kernel<float, 1, 8>, (const float*)x); else go(router_logits_kernel<float, 4, 8>, (const float*)x);
  }
  const size_t sel_smem = sizeof(float) * 8 * (size_t)(2 * E + (sel.groups > 1 ? sel.groups : 0));
  if (sel_smem > 48 * 1024) cudaFuncSetAttribute(router_select_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)sel_smem);
  router_select_kernel<<<(N + 7) / 8, 256, sel_smem, st>>>(logits, topk_w, topk_i, N, E, k, sel);
}

void moe_plain_gather_launch(const void* x, const int* row_entry, const int* tile_expert, void* xp, int R, int H, int k, bool lp, cudaStream_t st) {
  if (R <= 0) return;
  if (lp) gather_kernel<__nv_bfloat16><<<R, 128, 0, st>>>((const __nv_bfloat16*)x, row_entry, tile_expert, (__nv_bfloat16*)xp, H, k);
  else gather_kernel<float><<<R, 128, 0, st>>>((const float*)x, row_entry, tile_expert, (float*)xp, H, k);
}

void moe_plain_gemm_launch(const void* a, const void* w, void* c, int R, int N, int K, int act, const int* tile_expert, bool lp, cudaStream_t st) {
  if (R <= 0 || N <= 0) return;
  if (R % 128 != 0) throw std::runtime_error("moe_plain_gemm: the row bound must be a multiple of 128");
  if (R / PT > 65535) throw std::runtime_error("moe_plain_gemm: too many row tiles");
  dim3 grid((N + PT - 1) / PT, R / PT);
  if (lp) grouped_gemm_kernel<__nv_bfloat16><<<grid, 256, 0, st>>>((const __nv_bfloat16*)a, (const __nv_bfloat16*)w, (__nv_bfloat16*)c, N, K, act, tile_expert);
  else grouped_gemm_kernel<float><<<grid, 256, 0, st>>>((const float*)a, (const float*)w, (float*)c, N, K, act, tile_expert);
}

void moe_plain_combine_launch(const void* y, const float* topk_w, const int* pos, void* out, int N, int H, int k, bool lp, cudaStream_t st) {
  if (N <= 0) return;
  if (k > 64) throw std::runtime_error("moe_plain_combine: top-k > 64");
  if (lp) combine_kernel<__nv_bfloat16><<<N, 128, 0, st>>>((const __nv_bfloat16*)y, topk_w, pos, (__nv_bfloat16*)out, H, k);
  else combine_kernel<float><<<N, 128, 0, st>>>((const float*)y, topk_w, pos, (float*)out, H, k);
}

void moe_plain_gate_mul_launch(const void* gu, void* h, int R, int I, int act, const int* tile_expert, bool lp, cudaStream_t st) {
  if (R <= 0) return;
  if (lp) gate_mul_rows_kernel<__nv_bfloat16><<<R, 256, 0, st>>>((const __nv_bfloat16*)gu, (__nv_bfloat16*)h, I, act, tile_expert);
  else gate_mul_rows_kernel<float><<<R, 256, 0, st>>>((const float*)gu, (float*)h, I, act, tile_expert);
}

void moe_plain_decode_launch(const void* x, const void* w_up, const void* w_down, const float* topk_w, const int* topk_i, void* h, void* out,
                             int N, int k, int H, int I, int expert_offset, int e_local, int act, bool gated, bool lp, cudaStream_t st) {
  if (N <= 0) return;
  const long long w1 = (long long)N * k * I, w2 = (long long)N * H;
  const unsigned g1 = (unsigned)((w1 + 7) / 8), g2 = (unsigned)((w2 + 7) / 8);
  if (lp) {
    decode_up_kernel<__nv_bfloat16><<<g1, 256, 0, st>>>((const __nv_bfloat16*)x, (const __nv_bfloat16*)w_up, topk_i, (__nv_bfloat16*)h, N * k, k, H, I,
                                                        expert_offset, e_local, act, (int)gated);
    decode_down_kernel<__nv_bfloat16><<<g2, 256, 0, st>>>((const __nv_bfloat16*)h, (const __nv_bfloat16*)w_down, topk_w, topk_i, (__nv_bfloat16*)out, N, k,
                                                          H, I, expert_offset, e_local);
  } else {
    decode_up_kernel<float><<<g1, 256, 0, st>>>((const float*)x, (const float*)w_up, topk_i, (float*)h, N * k, k, H, I, expert_offset, e_local, act, (int)gated);
    decode_down_kernel<float><<<g2, 256, 0, st>>>((const float*)h, (const float*)w_down, topk_w, topk_i, (float*)out, N, k, H, I, expert_offset,
                                                  e_local);
  }
}

}  // namespace nxdi
