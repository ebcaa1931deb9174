// Raw-pointer launchers of the ragged sequence-mixer kernels (seqmix.cu).  Conventions shared by all of them: activations are
// [B, T, ...]; row b holds q_len[b] <= T live tokens at positions ctx_len[b] + t; per-sequence state sits in line lines[b] of a state
// tensor and counts as zero when ctx_len[b] == 0.  `lp` selects the activation type: true = bf16, false = fp32.
#pragma once
#include <cuda_runtime.h>
#include <stdint.h>

namespace nxdi {

constexpr int SEQMIX_MAX_TAPS = 8;       // short convolutions: taps per channel
constexpr int SEQMIX_MAX_VDIM = 256;     // attention: value channels per head
constexpr int SEQMIX_MAX_STATE = 256;    // scan: state size per head

void scaled_add_rmsnorm_launch(const float* x, const void* y, bool y_lp, const float* w, float* out, void* out_lp, int rows, int W,
                               float alpha, float eps, float offset, cudaStream_t st);

// fp32 residual stream update and the norm that reads it: s = [x] + [y1] + [y2] + [rms_unit(yn) * wn] + [vec], h = rms_unit(s) * w.
// y1 / y2 / yn share one activation type; every input is optional except that at least one row source is present.
struct StreamAddParams {
  const float* x;                  // [rows, W] or null
  const void *y1, *y2, *yn;        // [rows, W] or null
  const float *wn, *vec, *w;       // [W] or null (w is required when h is wanted)
  float* s;                        // [rows, W]
  void* s_lp;                      // bf16 copy of s, or null
  void* h;                         // normalised rows (bf16 or fp32), or null
  int rows, W;
  float eps;
};
void stream_add_rmsnorm_launch(const StreamAddParams& p, bool y_lp, bool h_lp, cudaStream_t st);

// p points at the latent slice of the projection rows.  rot > 0: the `rot` channels behind the latent are rotated (rotate-half
// layout, cos / sin [B, T, rot / 2]) and stored behind the latent in the cache row of R + rot numbers.  q_rank > 0: channels
// [0, q_rank) of the rows at `q_in` (same strides) are RMS-normalised with q_w into q_out [B, T, q_rank].
void latent_norm_append_launch(const void* p, long long p_sb, long long p_st, const float* w, void* cache, const int* block_table,
                               const int* ctx_len, const int* q_len, int B, int T, int R, int page, int max_blocks, float eps, bool lp,
                               void* rows_out, int rot, const float* cos, const float* sin, const void* q_in, int q_rank, const float* q_w,
                               void* q_out, cudaStream_t st);      // rows_out: [B, T, R + rot] copy of the live rows in token order, or null

// dst[b, t, h, Dd - rot ...] = rotate_half(src[b, t, h, Ds - rot ...]) with cos / sin [B * T, rot / 2]
void rope_half_tail_launch(const void* src, void* dst, const float* cos, const float* sin, long long tokens, int H, int Ds, int Dd, int rot, bool lp,
                           cudaStream_t st);

// s = x + [y1] + [y2]; h = rms_unit(s) * w; out = h + sum_j cw[:, j] * h_(t - K + 1 + j), the rows before a portion from the fp32 state
// line (stream rows, normalised like the new ones; zero when ctx_len == 0).  cw null: out = h.
struct StreamConvParams {
  const float* x;            // [B, T, W]
  const void *y1, *y2;       // [B, T, W] or null, each bf16 or fp32
  int y1_lp, y2_lp;
  const float *w, *cw;       // [W], [W, K] or null
  const float* state;        // [lines, K - 1, W] or null (K == 1)
  const int *lines, *ctx_len, *q_len;
  float* s;                  // [B, T, W]
  void* out;                 // [B, T, W] bf16 or fp32
  int B, T, W, K;
  float eps;
};
void stream_norm_conv_launch(const StreamConvParams& p, bool out_lp, cudaStream_t st);

// y[tok, :] += x[tok, :] * sum_j topk_w[tok, j] [topk_i[tok, j] >= num_experts] (fp32 sum, in place)
void identity_expert_add_launch(void* y, const void* x, const float* topk_w, const int* topk_i, int N, int H, int k, int num_experts, bool lp,
                                cudaStream_t st);

// x [rows, H, D] *= sigmoid(gate[row, h]) in place; gate rows are g_stride elements apart; D a multiple of 16 bytes
void head_gate_mul_launch(void* x, const void* gate, long long g_stride, long long rows, int H, int D, bool lp, cudaStream_t st);

// act codes: 1 relu, 2 relu^2, 3 silu, 4 tanh-gelu, 5 sigmoid, 6 erf-gelu.  on_other: out = gate * act(other) instead of act(gate) * other.
// g_stride: elements between rows of `gate` (C when dense).
void gated_act_mul_launch(const void* gate, long long g_stride, const void* other, long long o_stride, void* out, long long rows, int C, int act,
                          bool on_other, bool lp, cudaStream_t st);
void unary_act_launch(const void* x, void* out, long long n, int act, bool lp, cudaStream_t st);

// Two-matrix experts y = W_down act(W_up x) on a device-side permutation (moe_plain.cu); T = bf16 or fp32, any sizes.
void moe_plain_gather_launch(const void* x, const int* row_entry, const int* tile_expert, void* xp, int R, int H, int k, bool lp, cudaStream_t st);
void moe_plain_gemm_launch(const void* a, const void* w, void* c, int R, int N, int K, int act, const int* tile_expert, bool lp, cudaStream_t st);
void moe_plain_combine_launch(const void* y, const float* topk_w, const int* pos, void* out, int N, int H, int k, bool lp, cudaStream_t st);
// gated: w_up holds [gate; up] rows ([E, 2 I, H]) and the hidden row is act(gate . x) * (up . x)
void moe_plain_decode_launch(const void* x, const void* w_up, const void* w_down, const float* topk_w, const int* topk_i, void* h, void* out,
                             int N, int k, int H, int I, int expert_offset, int e_local, int act, bool gated, bool lp, cudaStream_t st);
// h[r, i] = act(gu[r, i]) * gu[r, I + i] for the rows of used 128-row tiles
void moe_plain_gate_mul_launch(const void* gu, void* h, int R, int I, int act, const int* tile_expert, bool lp, cudaStream_t st);

// fp32 router: logits = x W^T (x bf16 or fp32, W fp32 [E, W]) on CUDA cores with the rows in shared memory, then per token the
// scores (sigmoid, or softmax over all E) of the k experts with the largest score + correction among the `keep` best of `groups` equal
// groups of neighbours, divided by their sum + renorm_eps when renorm_eps >= 0, times scale.  `logits` [N, E] is written and read.
struct RouterSelect {
  int softmax;               // 0: sigmoid scores
  const float* correction;   // [E] or null: added to the scores for the choice only
  int groups, keep;          // groups <= 1: no group limit
  float renorm_eps, scale;
};
void router_topk_launch(const void* x, const float* w, float* logits, float* topk_w, int* topk_i, int N, int W, int E, int k,
                        const RouterSelect& sel, bool lp, cudaStream_t st);

void short_conv_launch(const void* u, long long u_sb, long long u_st, const float* w, const float* bias, const void* state,
                       const int* lines, const int* ctx_len, const int* q_len, float* y, int B, int T, int C, int K, bool silu, bool lp,
                       cudaStream_t st);

void short_conv_update_launch(const void* u, long long u_sb, long long u_st, void* state, const int* lines, const int* ctx_len,
                              const int* q_len, int B, int T, int C, int K, bool lp, cudaStream_t st);

struct ConvQkParams {
  const void* p;            // [B, T, >= Cq + Ck + Cv] projections, row strides below
  long long p_sb, p_st;
  const float* conv_w;      // [Cq + Ck + Cv, K]
  const void* state;        // [lines, K - 1, Cq + Ck + Cv]
  const int *lines, *ctx_len, *q_len;
  const float *q_norm_w, *k_norm_w;
  const float *cos, *sin;   // [B, T, R / 2]
  void* q_out;              // [B, T, n_q, D]
  void *k_cache, *v_cache;  // [blocks, page, n_kv, D | Dv]
  const int* block_table;   // [B, max_blocks]
  int B, T, K, n_q, n_kv, D, Dv, R, page, max_blocks;
  float eps;
};
void conv_qknorm_rope_append_launch(const ConvQkParams& p, bool lp, cudaStream_t st);

struct WindowAttnParams {
  const void* q;            // [B, T, Hq, D]
  const void *k_cache, *v_cache;
  const int *block_table, *ctx_len, *q_len;
  const void* gate;         // [B, T, Hq * Dv] with row strides below, or null
  long long g_sb, g_st;
  void* out;                // [B, T, Hq * Dv]
  int B, T, Hq, G, D, Dv, page, max_blocks, window, keep_first;
  float scale, softcap;
  const float* sinks;       // [Hq] or null: exp(sinks[h]) joins the softmax denominator of head h (no key, no value)
  int gate_per_head;        // 1: gate is [B, T, Hq], one sigmoid factor per head instead of one per output channel
  int chunk;                // > 0: key j is visible from position p only when j / chunk == p / chunk (instead of a window)
  const float* slopes;      // [Hq] or null: slopes[h] * (p - j) is taken off the score of head h
  const float* head_scale;  // [Hq] or null: the score of head h is multiplied by head_scale[h] as well (a learned temperature per head)
  long long v_rs;           // elements between the value rows of neighbouring (token, kv head) pairs; Dv <= v_rs (values that are a
                            // prefix of a wider cache row: v_cache = k_cache, v_rs = D)
};
void paged_window_attention_launch(const WindowAttnParams& p, bool lp, cudaStream_t st);

struct SsdScanParams {
  const float* xBC;         // [B, T, inner + 2 G N] after convolution and SiLU
  const void *dt_raw, *z;   // strided views of the in-projection, activation type
  long long dt_sb, dt_st, z_sb, z_st;
  const float *A_log, *dt_bias, *D_skip;
  float* state;             // [lines, nh, N, P]
  const int *lines, *ctx_len, *q_len;
  float* y;                 // [B, T, inner] = (S^T C + D x) * silu(z)
  int B, T, nh, P, N, G;
};
void ssd_scan_launch(const SsdScanParams& p, bool lp, cudaStream_t st);

// Update of an fp32 residual stream whose sublayers are normalised on both sides, and the norm the next sublayer reads:
//   y = a_scale * f_a(a) + b_scale * f_b(b), f(v) = rms_unit(v) * weight when the weight is given, else v   (b optional)
//   s = x + mult * ls * norm(y) * post_w   (s = x when a is null);   h = norm(s) * next_w   (when next_w is given)
// norm: layer norm without bias when center, RMS norm otherwise.  All arithmetic fp32; a / b share one activation type.
struct SandwichParams {
  const float* x;                  // [rows, W]
  const void *a, *b;               // [rows, W] or null
  const float *a_w, *b_w;          // [W] or null
  const float *post_w, *ls;        // [W] or null
  const float* next_w;             // [W] or null
  float* s;                        // [rows, W]
  void* h;                         // [rows, W] bf16 or fp32, or null
  int rows, W, center;
  float a_scale, b_scale, mult, eps;
};
void stream_sandwich_norm_launch(const SandwichParams& p, bool y_lp, bool h_lp, cudaStream_t st);

// Per-head RMS norm (before or after the rotation, weights [D] shared by the heads or null) + rotate-half rotation of the first R
// channels of every q / k head + paged cache write.  value_from_key: the raw k slice doubles as the value (no v slice, Dv == D).
struct HeadNormRopeParams {
  const void* p;            // [B, T, >= Cq + Ck (+ Cv)] projections q | k | v, row strides below
  long long p_sb, p_st;
  const float *q_w, *k_w;   // [D] or null
  const float *cos, *sin;   // [B, T, R / 2] or null
  void* q_out;              // [B, T, n_q, D]
  void *k_cache, *v_cache;  // [blocks, page, n_kv, D | Dv]
  const int *block_table, *ctx_len, *q_len;
  int B, T, n_q, n_kv, D, Dv, R, page, max_blocks;
  int norm_at;              // 0 none, 1 before the rotation, 2 after it
  int value_from_key;
  float eps;
};
void head_norm_rope_append_launch(const HeadNormRopeParams& p, bool lp, cudaStream_t st);

// Gated delta rule with a carried fp32 state M [lines, nh, D, Dv]: q / k scaled to unit length (q also by D^-1/2), b = sigmoid(beta_raw),
// log decay = -exp(A_log) * softplus(a_raw + dt_bias); per step M *= decay, e = b * (v - M' k), M += outer(k, e), y = M' q.
struct DeltaScanParams {
  const float* qkv;         // [B, T, 2 n_qk D + nh Dv] after convolution and activation
  const void *beta_raw, *a_raw;      // [B, T, nh] strided views of the in-projection, activation type
  long long beta_sb, beta_st, a_sb, a_st;
  const float *A_log, *dt_bias;
  float* state;             // [lines, nh, D, Dv]
  const int *lines, *ctx_len, *q_len;
  float* o;                 // [B, T, nh * Dv]
  int B, T, nh, n_qk, D, Dv;
  float unit_eps;
};
void gated_delta_scan_launch(const DeltaScanParams& p, bool lp, cudaStream_t st);

// out[row, h, :] = rms_unit(y[row, h, :]) * w[:] * act(gate[row, h, :]); w [Dv] is shared by the heads; gate rows g_stride elements apart
void head_rmsnorm_gate_launch(const float* y, const float* w, const void* gate, long long g_stride, void* out, long long rows, int H, int Dv,
                              float eps, int act, bool gate_lp, bool out_lp, cudaStream_t st);

void group_rmsnorm_launch(const float* y, const float* w, void* out, bool out_lp, int rows, int W, int groups, float eps, cudaStream_t st);

void clamped_glu_launch(const void* gu, void* out, long long rows, int F, float limit, float alpha, bool lp, cudaStream_t st);

}  // namespace nxdi
