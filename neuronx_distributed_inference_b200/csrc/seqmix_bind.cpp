// pybind11 surface of the ragged sequence-mixer kernels (seqmix.cu); registered into the extension module by bindings.cpp.
#include <torch/extension.h>
#include <ATen/cuda/CUDAContext.h>
#include <c10/cuda/CUDAGuard.h>

#include "api.h"
#include "seqmix.h"

namespace nxdi {
namespace {

using OptT = c10::optional<at::Tensor>;
inline cudaStream_t stream() { return at::cuda::getCurrentCUDAStream(); }
inline bool is_f32(const at::Tensor& t) { return t.scalar_type() == at::kFloat; }
inline bool is_lp(const at::Tensor& t) { return t.scalar_type() == at::kBFloat16; }
inline void check_act(const at::Tensor& t, const char* what) {
  TORCH_CHECK(t.is_cuda() && (is_f32(t) || is_lp(t)), what, ": CUDA tensor of bfloat16 or float32");
}
inline void check_f32(const at::Tensor& t, const char* what) {
  TORCH_CHECK(t.is_cuda() && is_f32(t) && t.is_contiguous(), what, ": contiguous float32 CUDA tensor");
}
inline void check_i32(const at::Tensor& t, int64_t n, const char* what) {
  TORCH_CHECK(t.is_cuda() && t.scalar_type() == at::kInt && t.is_contiguous() && t.numel() >= n, what, ": contiguous int32 CUDA tensor");
}
// [B, T, C] view whose last axis is dense and whose rows are evenly strided
inline void check_rows(const at::Tensor& t, const char* what) {
  TORCH_CHECK(t.dim() == 3 && t.stride(2) == 1, what, ": [B, T, C] with a dense last axis");
}

std::tuple<at::Tensor, at::Tensor> scaled_add_rmsnorm(const at::Tensor& x, const OptT& y, const OptT& w, double alpha, double eps,
                                                      double offset, bool want_lp) {
  check_f32(x, "scaled_add_rmsnorm x");
  TORCH_CHECK(x.dim() == 2);
  if (y.has_value()) {
    check_act(*y, "scaled_add_rmsnorm y");
    TORCH_CHECK(y->is_contiguous() && y->sizes() == x.sizes());
  }
  if (w.has_value()) {
    check_f32(*w, "scaled_add_rmsnorm weight");
    TORCH_CHECK(w->numel() == x.size(1));
  }
  c10::cuda::CUDAGuard guard(x.device());
  auto out = at::empty_like(x);
  at::Tensor lp = want_lp ? at::empty(x.sizes(), x.options().dtype(at::kBFloat16)) : at::Tensor();
  scaled_add_rmsnorm_launch(x.data_ptr<float>(), y.has_value() ? y->data_ptr() : nullptr, y.has_value() && is_lp(*y),
                            w.has_value() ? w->data_ptr<float>() : nullptr, out.data_ptr<float>(), want_lp ? lp.data_ptr() : nullptr,
                            (int)x.size(0), (int)x.size(1), (float)alpha, (float)eps, (float)offset, stream());
  return {out, want_lp ? lp : out};
}

void check_conv(const at::Tensor& u, const at::Tensor& w, const at::Tensor& state, const at::Tensor& lines, const at::Tensor& ctx,
                const at::Tensor& qlen) {
  check_act(u, "short_conv input");
  check_rows(u, "short_conv input");
  check_f32(w, "short_conv weight");
  const int64_t B = u.size(0), C = u.size(2), K = w.size(1);
  TORCH_CHECK(w.dim() == 2 && w.size(0) == C && K >= 1 && K <= SEQMIX_MAX_TAPS, "short_conv: weight [C, taps], taps <= ", SEQMIX_MAX_TAPS);
  TORCH_CHECK(state.is_cuda() && state.scalar_type() == u.scalar_type() && state.is_contiguous() && state.dim() == 3 &&
              state.size(1) == K - 1 && state.size(2) == C, "short_conv: state [lines, taps - 1, C] of the input's type");
  check_i32(lines, B, "lines");
  check_i32(ctx, B, "ctx_len");
  check_i32(qlen, B, "q_len");
}

at::Tensor short_conv(const at::Tensor& u, const at::Tensor& w, const OptT& bias, const at::Tensor& state, const at::Tensor& lines,
                      const at::Tensor& ctx, const at::Tensor& qlen, bool silu) {
  check_conv(u, w, state, lines, ctx, qlen);
  if (bias.has_value()) check_f32(*bias, "short_conv bias");
  c10::cuda::CUDAGuard guard(u.device());
  auto y = at::zeros({u.size(0), u.size(1), u.size(2)}, u.options().dtype(at::kFloat));
  short_conv_launch(u.data_ptr(), u.stride(0), u.stride(1), w.data_ptr<float>(), bias.has_value() ? bias->data_ptr<float>() : nullptr,
                    state.data_ptr(), lines.data_ptr<int>(), ctx.data_ptr<int>(), qlen.data_ptr<int>(), y.data_ptr<float>(),
                    (int)u.size(0), (int)u.size(1), (int)u.size(2), (int)w.size(1), silu, is_lp(u), stream());
  return y;
}

void short_conv_update(const at::Tensor& u, at::Tensor state, const at::Tensor& lines, const at::Tensor& ctx, const at::Tensor& qlen) {
  check_act(u, "short_conv_update input");
  check_rows(u, "short_conv_update input");
  const int64_t B = u.size(0), C = u.size(2), K = state.size(1) + 1;
  TORCH_CHECK(state.is_cuda() && state.scalar_type() == u.scalar_type() && state.is_contiguous() && state.dim() == 3 && state.size(2) == C &&
              K <= SEQMIX_MAX_TAPS);
  check_i32(lines, B, "lines");
  check_i32(ctx, B, "ctx_len");
  check_i32(qlen, B, "q_len");
  c10::cuda::CUDAGuard guard(u.device());
  short_conv_update_launch(u.data_ptr(), u.stride(0), u.stride(1), state.data_ptr(), lines.data_ptr<int>(), ctx.data_ptr<int>(),
                           qlen.data_ptr<int>(), (int)B, (int)u.size(1), (int)C, (int)K, is_lp(u), stream());
}

at::Tensor conv_qknorm_rope_append(const at::Tensor& p, const at::Tensor& conv_w, const at::Tensor& state, const at::Tensor& lines,
                                   const at::Tensor& ctx, const at::Tensor& qlen, const OptT& q_norm_w, const OptT& k_norm_w, double eps,
                                   int64_t n_q, int64_t n_kv, int64_t D, int64_t Dv, const OptT& cos, const OptT& sin,
                                   at::Tensor k_cache, at::Tensor v_cache, const OptT& block_table) {
  check_act(p, "conv_qknorm_rope_append projections");
  check_rows(p, "conv_qknorm_rope_append projections");
  const int64_t B = p.size(0), T = p.size(1), C = n_q * D + n_kv * (D + Dv), K = conv_w.size(1);
  TORCH_CHECK(p.size(2) >= C && D % 2 == 0, "conv_qknorm_rope_append: projection narrower than q | k | v, or odd head size");
  check_f32(conv_w, "conv weight");
  TORCH_CHECK(conv_w.dim() == 2 && conv_w.size(0) == C && K >= 1 && K <= SEQMIX_MAX_TAPS);
  TORCH_CHECK(state.is_cuda() && state.scalar_type() == p.scalar_type() && state.is_contiguous() && state.dim() == 3 &&
              state.size(1) == K - 1 && state.size(2) == C, "conv_qknorm_rope_append: state [lines, taps - 1, q | k | v channels]");
  check_i32(lines, B, "lines");
  check_i32(ctx, B, "ctx_len");
  check_i32(qlen, B, "q_len");
  if (q_norm_w.has_value()) {
    check_f32(*q_norm_w, "q norm weight");
    TORCH_CHECK(q_norm_w->numel() == n_q * D);
  }
  int64_t R = 0;
  if (cos.has_value()) {      // no tables: no rotation
    TORCH_CHECK(sin.has_value());
    check_f32(*cos, "cos");
    check_f32(*sin, "sin");
    TORCH_CHECK(cos->dim() == 3 && cos->size(0) == B && cos->size(1) == T && sin->sizes() == cos->sizes());
    R = 2 * cos->size(2);
  }
  TORCH_CHECK(R <= D, "rotated channels exceed the head size");
  ConvQkParams a{};
  if (n_kv > 0) {
    TORCH_CHECK(block_table.has_value());
    if (k_norm_w.has_value()) {
      check_f32(*k_norm_w, "k norm weight");
      TORCH_CHECK(k_norm_w->numel() == n_kv * D);
      a.k_norm_w = k_norm_w->data_ptr<float>();
    }
    TORCH_CHECK(k_cache.is_cuda() && k_cache.scalar_type() == p.scalar_type() && k_cache.is_contiguous() && k_cache.dim() == 4 &&
                k_cache.size(2) == n_kv && k_cache.size(3) == D, "k cache [blocks, page, kv heads, D] of the activation type");
    TORCH_CHECK(v_cache.is_cuda() && v_cache.scalar_type() == p.scalar_type() && v_cache.is_contiguous() && v_cache.dim() == 4 &&
                v_cache.size(0) == k_cache.size(0) && v_cache.size(1) == k_cache.size(1) && v_cache.size(2) == n_kv && v_cache.size(3) == Dv);
    TORCH_CHECK(block_table->is_cuda() && block_table->scalar_type() == at::kInt && block_table->is_contiguous() && block_table->dim() == 2 &&
                block_table->size(0) == B);
    a.k_cache = k_cache.data_ptr();
    a.v_cache = v_cache.data_ptr();
    a.block_table = block_table->data_ptr<int>();
    a.page = (int)k_cache.size(1);
    a.max_blocks = (int)block_table->size(1);
  }
  c10::cuda::CUDAGuard guard(p.device());
  auto q = at::zeros({B, T, n_q, D}, p.options());
  a.p = p.data_ptr(); a.p_sb = p.stride(0); a.p_st = p.stride(1);
  a.conv_w = conv_w.data_ptr<float>(); a.state = state.data_ptr();
  a.lines = lines.data_ptr<int>(); a.ctx_len = ctx.data_ptr<int>(); a.q_len = qlen.data_ptr<int>();
  a.q_norm_w = q_norm_w.has_value() ? q_norm_w->data_ptr<float>() : nullptr;
  a.cos = cos.has_value() ? cos->data_ptr<float>() : nullptr;
  a.sin = sin.has_value() ? sin->data_ptr<float>() : nullptr;
  a.q_out = q.data_ptr();
  a.B = (int)B; a.T = (int)T; a.K = (int)K; a.n_q = (int)n_q; a.n_kv = (int)n_kv; a.D = (int)D; a.Dv = (int)Dv; a.R = (int)R;
  a.eps = (float)eps;
  conv_qknorm_rope_append_launch(a, is_lp(p), stream());
  return q;
}

at::Tensor paged_window_attention(const at::Tensor& q, const at::Tensor& k_cache, const at::Tensor& v_cache, const at::Tensor& block_table,
                                  const at::Tensor& ctx, const at::Tensor& qlen, double scale, double softcap, int64_t window,
                                  int64_t keep_first, const OptT& gate, const OptT& sinks, bool gate_per_head, int64_t chunk, const OptT& slopes,
                                  int64_t value_dim, const OptT& head_scale) {
  check_act(q, "paged_window_attention q");
  TORCH_CHECK(q.dim() == 4 && q.is_contiguous());
  const int64_t B = q.size(0), T = q.size(1), Hq = q.size(2), D = q.size(3);
  TORCH_CHECK(k_cache.is_cuda() && k_cache.scalar_type() == q.scalar_type() && k_cache.is_contiguous() && k_cache.dim() == 4 && k_cache.size(3) == D);
  TORCH_CHECK(v_cache.is_cuda() && v_cache.scalar_type() == q.scalar_type() && v_cache.is_contiguous() && v_cache.dim() == 4 &&
              v_cache.size(0) == k_cache.size(0) && v_cache.size(1) == k_cache.size(1) && v_cache.size(2) == k_cache.size(2));
  // value_dim: the value of a key is the first value_dim channels of its row in v_cache
  const int64_t G = k_cache.size(2), Dv = value_dim;
  TORCH_CHECK(Dv >= 1 && Dv <= v_cache.size(3) && chunk >= 0 && !(chunk > 0 && window > 0), "paged_window_attention: value size / mask");
  TORCH_CHECK(Hq % G == 0 && Dv <= SEQMIX_MAX_VDIM, "paged_window_attention: heads must divide, value size <= ", SEQMIX_MAX_VDIM);
  TORCH_CHECK(block_table.is_cuda() && block_table.scalar_type() == at::kInt && block_table.is_contiguous() && block_table.dim() == 2 &&
              block_table.size(0) == B);
  check_i32(ctx, B, "ctx_len");
  check_i32(qlen, B, "q_len");
  WindowAttnParams a{};
  if (gate.has_value()) {
    check_rows(*gate, "gate");
    TORCH_CHECK(gate->is_cuda() && gate->scalar_type() == q.scalar_type() && gate->size(0) == B && gate->size(1) == T &&
                gate->size(2) == (gate_per_head ? Hq : Hq * Dv), "gate: [B, T, heads * value size], or [B, T, heads] with gate_per_head");
    a.gate = gate->data_ptr(); a.g_sb = gate->stride(0); a.g_st = gate->stride(1);
    a.gate_per_head = gate_per_head ? 1 : 0;
  }
  if (sinks.has_value()) {
    check_f32(*sinks, "sinks");
    TORCH_CHECK(sinks->numel() == Hq, "sinks: one per query head");
    a.sinks = sinks->data_ptr<float>();
  }
  if (slopes.has_value()) {
    check_f32(*slopes, "slopes");
    TORCH_CHECK(slopes->numel() == Hq, "slopes: one per query head");
    a.slopes = slopes->data_ptr<float>();
  }
  if (head_scale.has_value()) {
    check_f32(*head_scale, "head_scale");
    TORCH_CHECK(head_scale->numel() == Hq, "head_scale: one per query head");
    a.head_scale = head_scale->data_ptr<float>();
  }
  a.chunk = (int)chunk;
  a.v_rs = v_cache.size(3);
  c10::cuda::CUDAGuard guard(q.device());
  auto out = at::zeros({B, T, Hq * Dv}, q.options());
  a.q = q.data_ptr(); a.k_cache = k_cache.data_ptr(); a.v_cache = v_cache.data_ptr();
  a.block_table = block_table.data_ptr<int>(); a.ctx_len = ctx.data_ptr<int>(); a.q_len = qlen.data_ptr<int>();
  a.out = out.data_ptr();
  a.B = (int)B; a.T = (int)T; a.Hq = (int)Hq; a.G = (int)G; a.D = (int)D; a.Dv = (int)Dv; a.page = (int)k_cache.size(1);
  a.max_blocks = (int)block_table.size(1); a.window = (int)window; a.keep_first = (int)keep_first;
  a.scale = (float)scale; a.softcap = (float)softcap;
  paged_window_attention_launch(a, is_lp(q), stream());
  return out;
}

at::Tensor ssd_scan(const at::Tensor& xBC, const at::Tensor& dt_raw, const at::Tensor& z, const at::Tensor& A_log, const at::Tensor& dt_bias,
                    const at::Tensor& D_skip, at::Tensor state, const at::Tensor& lines, const at::Tensor& ctx, const at::Tensor& qlen,
                    int64_t nh, int64_t P, int64_t N, int64_t G) {
  check_f32(xBC, "ssd_scan xBC");
  const int64_t B = xBC.size(0), T = xBC.size(1), inner = nh * P;
  TORCH_CHECK(xBC.dim() == 3 && xBC.size(2) == inner + 2 * G * N && nh % G == 0 && N <= SEQMIX_MAX_STATE, "ssd_scan: xBC [B, T, inner + 2 G N], N <= ",
              SEQMIX_MAX_STATE);
  check_act(dt_raw, "ssd_scan dt");
  check_rows(dt_raw, "ssd_scan dt");
  check_rows(z, "ssd_scan z");
  TORCH_CHECK(z.is_cuda() && z.scalar_type() == dt_raw.scalar_type() && dt_raw.size(0) == B && dt_raw.size(1) == T && dt_raw.size(2) == nh &&
              z.size(0) == B && z.size(1) == T && z.size(2) == inner);
  check_f32(A_log, "A_log"); check_f32(dt_bias, "dt_bias"); check_f32(D_skip, "D");
  TORCH_CHECK(A_log.numel() == nh && dt_bias.numel() == nh && D_skip.numel() == nh);
  check_f32(state, "ssd_scan state");
  TORCH_CHECK(state.dim() == 4 && state.size(1) == nh && state.size(2) == N && state.size(3) == P, "ssd_scan: state [lines, heads, N, head_dim]");
  check_i32(lines, B, "lines"); check_i32(ctx, B, "ctx_len"); check_i32(qlen, B, "q_len");
  c10::cuda::CUDAGuard guard(xBC.device());
  auto y = at::zeros({B, T, inner}, xBC.options());
  SsdScanParams a{};
  a.xBC = xBC.data_ptr<float>(); a.dt_raw = dt_raw.data_ptr(); a.z = z.data_ptr();
  a.dt_sb = dt_raw.stride(0); a.dt_st = dt_raw.stride(1); a.z_sb = z.stride(0); a.z_st = z.stride(1);
  a.A_log = A_log.data_ptr<float>(); a.dt_bias = dt_bias.data_ptr<float>(); a.D_skip = D_skip.data_ptr<float>();
  a.state = state.data_ptr<float>(); a.lines = lines.data_ptr<int>(); a.ctx_len = ctx.data_ptr<int>(); a.q_len = qlen.data_ptr<int>();
  a.y = y.data_ptr<float>();
  a.B = (int)B; a.T = (int)T; a.nh = (int)nh; a.P = (int)P; a.N = (int)N; a.G = (int)G;
  ssd_scan_launch(a, is_lp(dt_raw), stream());
  return y;
}

at::Tensor group_rmsnorm(const at::Tensor& y, const at::Tensor& w, int64_t groups, double eps, bool out_lp) {
  check_f32(y, "group_rmsnorm input");
  check_f32(w, "group_rmsnorm weight");
  TORCH_CHECK(y.dim() == 2 && groups >= 1 && y.size(1) % groups == 0 && w.numel() == y.size(1));
  c10::cuda::CUDAGuard guard(y.device());
  auto out = at::empty(y.sizes(), y.options().dtype(out_lp ? at::kBFloat16 : at::kFloat));
  group_rmsnorm_launch(y.data_ptr<float>(), w.data_ptr<float>(), out.data_ptr(), out_lp, (int)y.size(0), (int)y.size(1), (int)groups, (float)eps,
                       stream());
  return out;
}

at::Tensor clamped_glu(const at::Tensor& gu, double limit, double alpha) {
  check_act(gu, "clamped_glu input");
  TORCH_CHECK(gu.dim() == 2 && gu.is_contiguous() && gu.size(1) % 2 == 0);
  c10::cuda::CUDAGuard guard(gu.device());
  auto out = at::empty({gu.size(0), gu.size(1) / 2}, gu.options());
  clamped_glu_launch(gu.data_ptr(), out.data_ptr(), gu.size(0), (int)(gu.size(1) / 2), (float)limit, (float)alpha, is_lp(gu), stream());
  return out;
}

std::tuple<at::Tensor, OptT, OptT> stream_add_rmsnorm(const OptT& x, const OptT& y1, const OptT& y2, const OptT& yn, const OptT& wn,
                                                      const OptT& vec, const OptT& w, double eps, bool h_lp, bool want_s_lp) {
  const at::Tensor* first = x.has_value() ? &*x : (y1.has_value() ? &*y1 : (yn.has_value() ? &*yn : nullptr));
  TORCH_CHECK(first != nullptr && first->dim() == 2, "stream_add_rmsnorm: at least one [rows, W] input");
  const int64_t rows = first->size(0), W = first->size(1);
  if (x.has_value()) {
    check_f32(*x, "stream_add_rmsnorm x");
    TORCH_CHECK(x->sizes() == first->sizes());
  }
  bool y_lp = false, seen = false;
  for (const OptT* y : {&y1, &y2, &yn}) {
    if (!y->has_value()) continue;
    check_act(**y, "stream_add_rmsnorm addend");
    TORCH_CHECK((*y)->is_contiguous() && (*y)->sizes() == first->sizes());
    TORCH_CHECK(!seen || y_lp == is_lp(**y), "stream_add_rmsnorm: addends of one type");
    y_lp = is_lp(**y);
    seen = true;
  }
  for (const OptT* v : {&wn, &vec, &w}) {
    if (!v->has_value()) continue;
    check_f32(**v, "stream_add_rmsnorm vector");
    TORCH_CHECK((*v)->numel() == W);
  }
  c10::cuda::CUDAGuard guard(first->device());
  auto f32 = first->options().dtype(at::kFloat);
  auto s = at::empty({rows, W}, f32);
  OptT s_lp, h;
  if (want_s_lp) s_lp = at::empty({rows, W}, f32.dtype(at::kBFloat16));
  if (w.has_value()) h = at::empty({rows, W}, f32.dtype(h_lp ? at::kBFloat16 : at::kFloat));
  StreamAddParams a{};
  a.x = x.has_value() ? x->data_ptr<float>() : nullptr;
  a.y1 = y1.has_value() ? y1->data_ptr() : nullptr;
  a.y2 = y2.has_value() ? y2->data_ptr() : nullptr;
  a.yn = yn.has_value() ? yn->data_ptr() : nullptr;
  a.wn = wn.has_value() ? wn->data_ptr<float>() : nullptr;
  a.vec = vec.has_value() ? vec->data_ptr<float>() : nullptr;
  a.w = w.has_value() ? w->data_ptr<float>() : nullptr;
  a.s = s.data_ptr<float>();
  a.s_lp = s_lp.has_value() ? s_lp->data_ptr() : nullptr;
  a.h = h.has_value() ? h->data_ptr() : nullptr;
  a.rows = (int)rows; a.W = (int)W; a.eps = (float)eps;
  stream_add_rmsnorm_launch(a, y_lp, h_lp, stream());
  return {s, s_lp, h};
}

std::tuple<OptT, OptT> latent_norm_append(const at::Tensor& p, int64_t offset, int64_t rank, const at::Tensor& w, double eps, at::Tensor cache,
                                          const at::Tensor& block_table, const at::Tensor& ctx, const at::Tensor& qlen, bool emit_rows, int64_t rot,
                                          const OptT& cos, const OptT& sin, int64_t q_rank, const OptT& q_w) {
  check_act(p, "latent_norm_append input");
  check_rows(p, "latent_norm_append input");
  const int64_t B = p.size(0), T = p.size(1);
  TORCH_CHECK(offset >= 0 && rank >= 1 && rot >= 0 && rot % 2 == 0 && offset + rank + rot <= p.size(2), "latent_norm_append: slice outside the row");
  if (rot > 0) {
    TORCH_CHECK(cos.has_value() && sin.has_value());
    check_f32(*cos, "cos");
    check_f32(*sin, "sin");
    TORCH_CHECK(cos->numel() == B * T * (rot / 2) && sin->numel() == cos->numel(), "cos / sin [B, T, rot / 2]");
  }
  if (q_rank > 0) {
    TORCH_CHECK(q_w.has_value() && q_rank <= p.size(2));
    check_f32(*q_w, "query latent norm weight");
    TORCH_CHECK(q_w->numel() == q_rank);
  }
  check_f32(w, "latent norm weight");
  TORCH_CHECK(w.numel() == rank);
  TORCH_CHECK(cache.is_cuda() && cache.scalar_type() == p.scalar_type() && cache.is_contiguous() && cache.dim() == 4 && cache.size(2) == 1 &&
              cache.size(3) == rank + rot, "latent cache [blocks, page, 1, rank + rotated part] of the activation type");
  TORCH_CHECK(block_table.is_cuda() && block_table.scalar_type() == at::kInt && block_table.is_contiguous() && block_table.dim() == 2 &&
              block_table.size(0) == B);
  check_i32(ctx, B, "ctx_len");
  check_i32(qlen, B, "q_len");
  c10::cuda::CUDAGuard guard(p.device());
  const char* base = (const char*)p.data_ptr() + offset * p.element_size();
  OptT rows, cq;
  if (emit_rows) rows = at::zeros({B, T, 1, rank + rot}, p.options());      // rows past q_len stay zero
  if (q_rank > 0) cq = at::zeros({B, T, q_rank}, p.options());
  latent_norm_append_launch(base, p.stride(0), p.stride(1), w.data_ptr<float>(), cache.data_ptr(), block_table.data_ptr<int>(), ctx.data_ptr<int>(),
                            qlen.data_ptr<int>(), (int)B, (int)T, (int)rank, (int)cache.size(1), (int)block_table.size(1), (float)eps, is_lp(p),
                            rows.has_value() ? rows->data_ptr() : nullptr, (int)rot, rot > 0 ? cos->data_ptr<float>() : nullptr,
                            rot > 0 ? sin->data_ptr<float>() : nullptr, p.data_ptr(), (int)q_rank, q_rank > 0 ? q_w->data_ptr<float>() : nullptr,
                            cq.has_value() ? cq->data_ptr() : nullptr, stream());
  return {rows, cq};
}

void head_gate_mul(at::Tensor x, const at::Tensor& gate) {
  check_act(x, "head_gate_mul x");
  check_rows(gate, "head_gate_mul gate");
  TORCH_CHECK(x.dim() == 4 && x.is_contiguous() && gate.is_cuda() && gate.scalar_type() == x.scalar_type() && gate.size(0) == x.size(0) &&
              gate.size(1) == x.size(1) && gate.size(2) == x.size(2) && gate.stride(0) == gate.size(1) * gate.stride(1),
              "head_gate_mul: x [B, T, H, D] contiguous, gate [B, T, H] with evenly strided rows");
  const int64_t V = is_lp(x) ? 8 : 4;
  TORCH_CHECK(x.size(3) % V == 0 && ((uintptr_t)x.data_ptr() & 15) == 0, "head_gate_mul: head size in multiples of 16 bytes");
  c10::cuda::CUDAGuard guard(x.device());
  head_gate_mul_launch(x.data_ptr(), gate.data_ptr(), gate.stride(1), x.size(0) * x.size(1), (int)x.size(2), (int)x.size(3), is_lp(x), stream());
}

at::Tensor gated_act_mul(const at::Tensor& gate, const at::Tensor& other, int64_t act, bool on_other) {
  check_act(gate, "gated_act_mul gate");
  TORCH_CHECK(gate.dim() == 2 && gate.is_contiguous() && other.is_cuda() && other.scalar_type() == gate.scalar_type() && other.dim() == 2 &&
              other.sizes() == gate.sizes() && other.stride(1) == 1, "gated_act_mul: [rows, C] inputs of one type, the second with a row stride");
  c10::cuda::CUDAGuard guard(gate.device());
  auto out = at::empty_like(gate);
  gated_act_mul_launch(gate.data_ptr(), gate.stride(0), other.data_ptr(), other.stride(0), out.data_ptr(), gate.size(0), (int)gate.size(1), (int)act,
                       on_other, is_lp(gate), stream());
  return out;
}

at::Tensor unary_act(const at::Tensor& x, int64_t act) {
  check_act(x, "unary_act input");
  TORCH_CHECK(x.is_contiguous());
  c10::cuda::CUDAGuard guard(x.device());
  auto out = at::empty_like(x);
  unary_act_launch(x.data_ptr(), out.data_ptr(), x.numel(), (int)act, is_lp(x), stream());
  return out;
}

// Routed two-matrix experts: x [N, H], w_up [E, I, H], w_down [E, H, I] (activation type), topk_w fp32 / topk_i int32 [N, k].
// `tc`: bf16 with H and I in multiples of 64 -> grouped tcgen05 GEMMs, the activation as an elementwise pass between them.
at::Tensor moe_plain(const at::Tensor& x, const at::Tensor& w_up, const at::Tensor& w_down, const at::Tensor& topk_w, const at::Tensor& topk_i,
                     int64_t expert_offset, int64_t act, bool tc, bool gated) {
  check_act(x, "moe_plain x");
  TORCH_CHECK(x.dim() == 2 && x.is_contiguous() && w_up.dim() == 3 && w_down.dim() == 3 && w_up.is_contiguous() && w_down.is_contiguous() &&
              w_up.scalar_type() == x.scalar_type() && w_down.scalar_type() == x.scalar_type() && w_up.is_cuda() && w_down.is_cuda());
  // gated: w_up holds [gate; up] rows, [E, 2 I, H], and the hidden row is act(gate) * up
  const int N = (int)x.size(0), H = (int)x.size(1), E = (int)w_up.size(0), I = (int)w_down.size(2), k = (int)topk_i.size(1);
  TORCH_CHECK(w_up.size(1) == (gated ? 2 : 1) * I && w_up.size(2) == H && w_down.size(0) == E && w_down.size(1) == H && !(gated && tc),
              "moe_plain: w_up [E, I, H] ([E, 2 I, H] gated), w_down [E, H, I]");
  TORCH_CHECK(topk_w.is_cuda() && topk_w.scalar_type() == at::kFloat && topk_i.is_cuda() && topk_i.scalar_type() == at::kInt && topk_w.is_contiguous() &&
              topk_i.is_contiguous() && topk_w.numel() == (int64_t)N * k && topk_i.size(0) == N && k <= 64 && E <= 512);
  const bool lp = is_lp(x);
  TORCH_CHECK(!tc || (lp && H % 64 == 0 && I % 64 == 0), "moe_plain: the tensor-core path needs bf16 and sizes in multiples of 64");
  c10::cuda::CUDAGuard guard(x.device());
  auto st = stream();
  auto out = at::empty({N, H}, x.options());
  if (N * k <= 32) {        // decode steps: weight-streaming kernels, no permutation
    auto h = at::empty({(int64_t)N * k, I}, x.options());
    moe_plain_decode_launch(x.data_ptr(), w_up.data_ptr(), w_down.data_ptr(), topk_w.data_ptr<float>(), topk_i.data_ptr<int>(), h.data_ptr(),
                            out.data_ptr(), N, k, H, I, (int)expert_offset, E, (int)act, gated, lp, st);
    return out;
  }
  const int64_t R = (((int64_t)N * k + (int64_t)E * 127) + 127) / 128 * 128;   // static bound: graph-stable shapes
  auto iopt = x.options().dtype(at::kInt);
  auto pos = at::empty({(int64_t)N * k}, iopt);
  auto row_entry = at::empty({R}, iopt);
  auto tile_expert = at::empty({R / 128}, iopt);
  auto xp = at::empty({R, H}, x.options());
  auto h = at::empty({R, I}, x.options());
  auto y = at::empty({R, H}, x.options());
  moe_plan_launch(topk_i.data_ptr<int>(), N * k, (int)expert_offset, E, (int)R, pos.data_ptr<int>(), row_entry.data_ptr<int>(),
                  tile_expert.data_ptr<int>(), st);
  if (tc) {
    moe_gather_launch(x.data_ptr(), topk_w.data_ptr<float>(), row_entry.data_ptr<int>(), tile_expert.data_ptr<int>(), xp.data_ptr(), (int)R, H, k, 0, st);
    gemm_grouped_launch(xp.data_ptr(), w_up.data_ptr(), nullptr, h.data_ptr(), (int)R, I, H, E, 0, tile_expert.data_ptr<int>(), nullptr, nullptr, st);
    unary_act_launch(h.data_ptr(), h.data_ptr(), (long long)R * I, (int)act, true, st);      // rows of unused tiles hold junk; nothing reads them
    gemm_grouped_launch(h.data_ptr(), w_down.data_ptr(), nullptr, y.data_ptr(), (int)R, H, I, E, 0, tile_expert.data_ptr<int>(), nullptr, nullptr, st);
    moe_combine_launch(y.data_ptr(), topk_w.data_ptr<float>(), pos.data_ptr<int>(), out.data_ptr(), N, H, k, 0, st);
    return out;
  }
  moe_plain_gather_launch(x.data_ptr(), row_entry.data_ptr<int>(), tile_expert.data_ptr<int>(), xp.data_ptr(), (int)R, H, k, lp, st);
  if (gated) {
    auto gu = at::empty({R, 2 * (int64_t)I}, x.options());
    moe_plain_gemm_launch(xp.data_ptr(), w_up.data_ptr(), gu.data_ptr(), (int)R, 2 * I, H, 0, tile_expert.data_ptr<int>(), lp, st);
    moe_plain_gate_mul_launch(gu.data_ptr(), h.data_ptr(), (int)R, I, (int)act, tile_expert.data_ptr<int>(), lp, st);
  } else {
    moe_plain_gemm_launch(xp.data_ptr(), w_up.data_ptr(), h.data_ptr(), (int)R, I, H, (int)act, tile_expert.data_ptr<int>(), lp, st);
  }
  moe_plain_gemm_launch(h.data_ptr(), w_down.data_ptr(), y.data_ptr(), (int)R, H, I, 0, tile_expert.data_ptr<int>(), lp, st);
  moe_plain_combine_launch(y.data_ptr(), topk_w.data_ptr<float>(), pos.data_ptr<int>(), out.data_ptr(), N, H, k, lp, st);
  return out;
}

std::tuple<at::Tensor, at::Tensor, at::Tensor> router_topk(const at::Tensor& x, const at::Tensor& w, int64_t k, double renorm_eps, bool softmax,
                                                           const OptT& correction, int64_t groups, int64_t keep, double scale) {
  check_act(x, "router input");
  check_f32(w, "router weight");
  TORCH_CHECK(x.dim() == 2 && x.is_contiguous() && w.dim() == 2 && w.size(1) == x.size(1) && k >= 1 && k <= w.size(0));
  const int N = (int)x.size(0), W = (int)x.size(1), E = (int)w.size(0);
  c10::cuda::CUDAGuard guard(x.device());
  auto f32 = x.options().dtype(at::kFloat);
  auto logits = at::empty({N, E}, f32);
  auto tw = at::empty({N, k}, f32);
  auto ti = at::empty({N, k}, x.options().dtype(at::kInt));
  RouterSelect sel{};
  sel.softmax = softmax ? 1 : 0;
  if (correction.has_value()) {
    check_f32(*correction, "router score correction");
    TORCH_CHECK(correction->numel() == E);
    sel.correction = correction->data_ptr<float>();
  }
  sel.groups = (int)groups; sel.keep = (int)keep; sel.renorm_eps = (float)renorm_eps; sel.scale = (float)scale;
  router_topk_launch(x.data_ptr(), w.data_ptr<float>(), logits.data_ptr<float>(), tw.data_ptr<float>(), ti.data_ptr<int>(), N, W, E, (int)k, sel,
                     is_lp(x), stream());
  return {logits, tw, ti};
}

void rope_half_tail(const at::Tensor& src, at::Tensor dst, int64_t rot, const at::Tensor& cos, const at::Tensor& sin) {
  check_act(src, "rope_half_tail source");
  TORCH_CHECK(src.dim() == 4 && dst.dim() == 4 && src.is_contiguous() && dst.is_contiguous() && dst.is_cuda() && dst.scalar_type() == src.scalar_type() &&
              src.size(0) == dst.size(0) && src.size(1) == dst.size(1) && src.size(2) == dst.size(2) && rot % 2 == 0 && rot <= src.size(3) &&
              rot <= dst.size(3), "rope_half_tail: [B, T, H, D] tensors of one type");
  check_f32(cos, "cos");
  check_f32(sin, "sin");
  const int64_t tokens = src.size(0) * src.size(1);
  TORCH_CHECK(cos.numel() == tokens * (rot / 2) && sin.numel() == cos.numel(), "cos / sin [B, T, rot / 2]");
  c10::cuda::CUDAGuard guard(src.device());
  rope_half_tail_launch(src.data_ptr(), dst.data_ptr(), cos.data_ptr<float>(), sin.data_ptr<float>(), tokens, (int)src.size(2), (int)src.size(3),
                        (int)dst.size(3), (int)rot, is_lp(src), stream());
}

std::tuple<at::Tensor, at::Tensor> stream_norm_conv(const at::Tensor& x, const OptT& y1, const OptT& y2, const at::Tensor& w, const OptT& cw,
                                                    const OptT& state, const OptT& lines, const at::Tensor& ctx, const at::Tensor& qlen, double eps,
                                                    bool out_lp) {
  check_f32(x, "stream_norm_conv x");
  TORCH_CHECK(x.dim() == 3, "stream_norm_conv: x [B, T, W]");
  const int64_t B = x.size(0), T = x.size(1), W = x.size(2);
  StreamConvParams a{};
  for (const OptT* y : {&y1, &y2}) {
    if (!y->has_value()) continue;
    check_act(**y, "stream_norm_conv addend");
    TORCH_CHECK((*y)->is_contiguous() && (*y)->sizes() == x.sizes());
  }
  if (y1.has_value()) { a.y1 = y1->data_ptr(); a.y1_lp = is_lp(*y1); }
  if (y2.has_value()) { a.y2 = y2->data_ptr(); a.y2_lp = is_lp(*y2); }
  check_f32(w, "stream_norm_conv norm weight");
  TORCH_CHECK(w.numel() == W);
  a.K = 1;
  if (cw.has_value()) {
    check_f32(*cw, "stream_norm_conv taps");
    TORCH_CHECK(cw->dim() == 2 && cw->size(0) == W && cw->size(1) >= 1 && cw->size(1) <= SEQMIX_MAX_TAPS, "taps [W, K], K <= ", SEQMIX_MAX_TAPS);
    a.K = (int)cw->size(1);
    a.cw = cw->data_ptr<float>();
    if (a.K > 1) {
      TORCH_CHECK(state.has_value() && lines.has_value());
      check_f32(*state, "stream_norm_conv state");
      TORCH_CHECK(state->dim() == 3 && state->size(1) == a.K - 1 && state->size(2) == W, "state [lines, K - 1, W] float32");
      check_i32(*lines, B, "lines");
      a.state = state->data_ptr<float>();
      a.lines = lines->data_ptr<int>();
    }
  }
  check_i32(ctx, B, "ctx_len");
  check_i32(qlen, B, "q_len");
  c10::cuda::CUDAGuard guard(x.device());
  auto s = at::empty_like(x);                                                        // the kernel writes rows past q_len as zeros
  auto out = at::empty(x.sizes(), x.options().dtype(out_lp ? at::kBFloat16 : at::kFloat));
  a.x = x.data_ptr<float>(); a.w = w.data_ptr<float>();
  a.ctx_len = ctx.data_ptr<int>(); a.q_len = qlen.data_ptr<int>();
  a.s = s.data_ptr<float>(); a.out = out.data_ptr();
  a.B = (int)B; a.T = (int)T; a.W = (int)W; a.eps = (float)eps;
  stream_norm_conv_launch(a, out_lp, stream());
  return {s, out};
}

void identity_expert_add(at::Tensor y, const at::Tensor& x, const at::Tensor& topk_w, const at::Tensor& topk_i, int64_t num_experts) {
  check_act(y, "identity_expert_add y");
  TORCH_CHECK(y.dim() == 2 && y.is_contiguous() && x.is_cuda() && x.is_contiguous() && x.scalar_type() == y.scalar_type() && x.sizes() == y.sizes());
  const int64_t N = y.size(0), k = topk_i.size(1);
  TORCH_CHECK(topk_w.is_cuda() && topk_w.scalar_type() == at::kFloat && topk_w.is_contiguous() && topk_w.numel() == N * k && topk_i.is_cuda() &&
              topk_i.scalar_type() == at::kInt && topk_i.is_contiguous() && topk_i.size(0) == N);
  c10::cuda::CUDAGuard guard(y.device());
  identity_expert_add_launch(y.data_ptr(), x.data_ptr(), topk_w.data_ptr<float>(), topk_i.data_ptr<int>(), (int)N, (int)y.size(1), (int)k,
                             (int)num_experts, is_lp(y), stream());
}

}  // namespace


inline const float* opt_f32(const OptT& t, int64_t n, const char* what) {
  if (!t.has_value()) return nullptr;
  check_f32(*t, what);
  TORCH_CHECK(t->numel() == n, what, ": ", n, " numbers");
  return t->data_ptr<float>();
}

std::tuple<at::Tensor, OptT> stream_sandwich_norm(const at::Tensor& x, const OptT& a, const OptT& b, const OptT& a_w, const OptT& b_w, double a_scale,
                                                  double b_scale, const OptT& post_w, const OptT& ls, double mult, const OptT& next_w, double eps,
                                                  bool center, bool h_lp) {
  check_f32(x, "stream_sandwich_norm x");
  TORCH_CHECK(x.dim() == 2);
  const int64_t rows = x.size(0), W = x.size(1);
  TORCH_CHECK(W * 4 <= 200 * 1024, "stream_sandwich_norm: rows of at most 51200 numbers");
  TORCH_CHECK(a.has_value() || !b.has_value(), "stream_sandwich_norm: b without a");
  bool y_lp = false;
  for (const OptT* t : {&a, &b}) {
    if (!t->has_value()) continue;
    check_act(**t, "stream_sandwich_norm a / b");
    TORCH_CHECK((*t)->is_contiguous() && (*t)->sizes() == x.sizes(), "stream_sandwich_norm: a / b like x, contiguous");
    y_lp = is_lp(**t);
  }
  TORCH_CHECK(!(a.has_value() && b.has_value()) || a->scalar_type() == b->scalar_type(), "stream_sandwich_norm: a and b of one type");
  SandwichParams p{};
  p.x = x.data_ptr<float>();
  p.a = a.has_value() ? a->data_ptr() : nullptr;
  p.b = b.has_value() ? b->data_ptr() : nullptr;
  p.a_w = opt_f32(a_w, W, "a weight"); p.b_w = opt_f32(b_w, W, "b weight");
  p.post_w = opt_f32(post_w, W, "post weight"); p.ls = opt_f32(ls, W, "layer scale"); p.next_w = opt_f32(next_w, W, "next weight");
  c10::cuda::CUDAGuard guard(x.device());
  auto s = at::empty_like(x);
  OptT h;
  if (next_w.has_value()) h = at::empty(x.sizes(), x.options().dtype(h_lp ? at::kBFloat16 : at::kFloat));
  p.s = s.data_ptr<float>();
  p.h = h.has_value() ? h->data_ptr() : nullptr;
  p.rows = (int)rows; p.W = (int)W; p.center = center ? 1 : 0;
  p.a_scale = (float)a_scale; p.b_scale = (float)b_scale; p.mult = (float)mult; p.eps = (float)eps;
  stream_sandwich_norm_launch(p, y_lp, h_lp, stream());
  return {s, h};
}

at::Tensor head_norm_rope_append(const at::Tensor& pr, int64_t n_q, int64_t n_kv, int64_t D, int64_t Dv, const OptT& cos, const OptT& sin,
                                 const OptT& q_w, const OptT& k_w, int64_t norm_at, double eps, bool value_from_key, at::Tensor k_cache,
                                 at::Tensor v_cache, const at::Tensor& block_table, const at::Tensor& ctx, const at::Tensor& qlen) {
  check_act(pr, "head_norm_rope_append rows");
  check_rows(pr, "head_norm_rope_append rows");
  const int64_t B = pr.size(0), T = pr.size(1);
  const int64_t need = n_q * D + n_kv * D + (value_from_key ? 0 : n_kv * Dv);
  TORCH_CHECK(pr.size(2) >= need && D >= 1 && D <= 256 && Dv >= 1 && (!value_from_key || Dv == D), "head_norm_rope_append: q | k | v slices, head size <= 256");
  TORCH_CHECK(norm_at >= 0 && norm_at <= 2);
  TORCH_CHECK(k_cache.is_cuda() && k_cache.scalar_type() == pr.scalar_type() && k_cache.is_contiguous() && k_cache.dim() == 4 &&
              k_cache.size(2) == n_kv && k_cache.size(3) == D, "head_norm_rope_append: key cache [blocks, page, kv heads, D]");
  TORCH_CHECK(v_cache.is_cuda() && v_cache.scalar_type() == pr.scalar_type() && v_cache.is_contiguous() && v_cache.dim() == 4 &&
              v_cache.size(0) == k_cache.size(0) && v_cache.size(1) == k_cache.size(1) && v_cache.size(2) == n_kv && v_cache.size(3) == Dv,
              "head_norm_rope_append: value cache [blocks, page, kv heads, Dv]");
  TORCH_CHECK(block_table.is_cuda() && block_table.scalar_type() == at::kInt && block_table.is_contiguous() && block_table.dim() == 2 &&
              block_table.size(0) == B);
  check_i32(ctx, B, "ctx_len");
  check_i32(qlen, B, "q_len");
  HeadNormRopeParams p{};
  if (cos.has_value()) {
    TORCH_CHECK(sin.has_value());
    check_f32(*cos, "cos"); check_f32(*sin, "sin");
    TORCH_CHECK(cos->dim() == 3 && cos->size(0) == B && cos->size(1) == T && cos->sizes() == sin->sizes() && 2 * cos->size(2) <= D,
                "cos / sin: [B, T, R / 2] with R <= D");
    p.cos = cos->data_ptr<float>(); p.sin = sin->data_ptr<float>(); p.R = (int)(2 * cos->size(2));
  }
  p.q_w = opt_f32(q_w, D, "q norm weight"); p.k_w = opt_f32(k_w, D, "k norm weight");
  c10::cuda::CUDAGuard guard(pr.device());
  auto q = at::zeros({B, T, n_q, D}, pr.options());
  p.p = pr.data_ptr(); p.p_sb = pr.stride(0); p.p_st = pr.stride(1);
  p.q_out = q.data_ptr(); p.k_cache = k_cache.data_ptr(); p.v_cache = v_cache.data_ptr();
  p.block_table = block_table.data_ptr<int>(); p.ctx_len = ctx.data_ptr<int>(); p.q_len = qlen.data_ptr<int>();
  p.B = (int)B; p.T = (int)T; p.n_q = (int)n_q; p.n_kv = (int)n_kv; p.D = (int)D; p.Dv = (int)Dv; p.page = (int)k_cache.size(1);
  p.max_blocks = (int)block_table.size(1); p.norm_at = (int)norm_at; p.value_from_key = value_from_key ? 1 : 0; p.eps = (float)eps;
  head_norm_rope_append_launch(p, is_lp(pr), stream());
  return q;
}

at::Tensor gated_delta_scan(const at::Tensor& qkv, const at::Tensor& beta_raw, const at::Tensor& a_raw, const at::Tensor& A_log,
                            const at::Tensor& dt_bias, at::Tensor state, const at::Tensor& lines, const at::Tensor& ctx, const at::Tensor& qlen,
                            int64_t nh, int64_t n_qk, int64_t D, int64_t Dv, double unit_eps) {
  check_f32(qkv, "gated_delta_scan q | k | v");
  TORCH_CHECK(qkv.dim() == 3 && qkv.size(2) == 2 * n_qk * D + nh * Dv && nh % n_qk == 0 && D >= 1 && D <= 256, "gated_delta_scan: sizes (D <= 256)");
  const int64_t B = qkv.size(0), T = qkv.size(1);
  for (const at::Tensor* t : {&beta_raw, &a_raw}) {
    check_act(*t, "gated_delta_scan beta / a");
    check_rows(*t, "gated_delta_scan beta / a");
    TORCH_CHECK(t->size(0) == B && t->size(1) == T && t->size(2) == nh);
  }
  TORCH_CHECK(beta_raw.scalar_type() == a_raw.scalar_type());
  check_f32(A_log, "A_log"); check_f32(dt_bias, "dt_bias");
  TORCH_CHECK(A_log.numel() == nh && dt_bias.numel() == nh);
  check_f32(state, "gated_delta_scan state");
  TORCH_CHECK(state.dim() == 4 && state.size(1) == nh && state.size(2) == D && state.size(3) == Dv, "gated_delta_scan: state [lines, heads, D, Dv]");
  check_i32(lines, B, "lines"); check_i32(ctx, B, "ctx_len"); check_i32(qlen, B, "q_len");
  c10::cuda::CUDAGuard guard(qkv.device());
  auto o = at::zeros({B, T, nh * Dv}, qkv.options());
  DeltaScanParams p{};
  p.qkv = qkv.data_ptr<float>();
  p.beta_raw = beta_raw.data_ptr(); p.beta_sb = beta_raw.stride(0); p.beta_st = beta_raw.stride(1);
  p.a_raw = a_raw.data_ptr(); p.a_sb = a_raw.stride(0); p.a_st = a_raw.stride(1);
  p.A_log = A_log.data_ptr<float>(); p.dt_bias = dt_bias.data_ptr<float>(); p.state = state.data_ptr<float>();
  p.lines = lines.data_ptr<int>(); p.ctx_len = ctx.data_ptr<int>(); p.q_len = qlen.data_ptr<int>();
  p.o = o.data_ptr<float>();
  p.B = (int)B; p.T = (int)T; p.nh = (int)nh; p.n_qk = (int)n_qk; p.D = (int)D; p.Dv = (int)Dv; p.unit_eps = (float)unit_eps;
  gated_delta_scan_launch(p, is_lp(beta_raw), stream());
  return o;
}

at::Tensor head_rmsnorm_gate(const at::Tensor& y, const at::Tensor& w, int64_t heads, double eps, const at::Tensor& gate, int64_t act, bool out_lp) {
  check_f32(y, "head_rmsnorm_gate y");
  check_f32(w, "head_rmsnorm_gate weight");
  TORCH_CHECK(y.dim() == 2 && y.size(1) % heads == 0);
  const int64_t rows = y.size(0), Dv = y.size(1) / heads;
  TORCH_CHECK(w.numel() == Dv && Dv <= SEQMIX_MAX_VDIM, "head_rmsnorm_gate: weight [Dv], Dv <= ", SEQMIX_MAX_VDIM);
  check_act(gate, "head_rmsnorm_gate gate");
  TORCH_CHECK(gate.dim() == 2 && gate.size(0) == rows && gate.size(1) == y.size(1) && gate.stride(1) == 1, "head_rmsnorm_gate: gate [rows, heads * Dv]");
  c10::cuda::CUDAGuard guard(y.device());
  auto out = at::empty(y.sizes(), y.options().dtype(out_lp ? at::kBFloat16 : at::kFloat));
  head_rmsnorm_gate_launch(y.data_ptr<float>(), w.data_ptr<float>(), gate.data_ptr(), gate.stride(0), out.data_ptr(), rows, (int)heads, (int)Dv,
                           (float)eps, (int)act, is_lp(gate), out_lp, stream());
  return out;
}


void register_seqmix(pybind11::module_& m) {
  m.def("stream_sandwich_norm", &stream_sandwich_norm);
  m.def("head_norm_rope_append", &head_norm_rope_append);
  m.def("gated_delta_scan", &gated_delta_scan);
  m.def("head_rmsnorm_gate", &head_rmsnorm_gate);
  m.def("router_topk", &router_topk);
  m.def("rope_half_tail", &rope_half_tail);
  m.def("stream_norm_conv", &stream_norm_conv);
  m.def("identity_expert_add", &identity_expert_add);
  m.def("stream_add_rmsnorm", &stream_add_rmsnorm);
  m.def("latent_norm_append", &latent_norm_append);
  m.def("head_gate_mul", &head_gate_mul);
  m.def("gated_act_mul", &gated_act_mul);
  m.def("unary_act", &unary_act);
  m.def("moe_plain", &moe_plain);
  m.def("scaled_add_rmsnorm", &scaled_add_rmsnorm);
  m.def("short_conv", &short_conv);
  m.def("short_conv_update", &short_conv_update);
  m.def("conv_qknorm_rope_append", &conv_qknorm_rope_append);
  m.def("paged_window_attention", &paged_window_attention);
  m.def("ssd_scan", &ssd_scan);
  m.def("group_rmsnorm", &group_rmsnorm);
  m.def("clamped_glu", &clamped_glu);
}

}  // namespace nxdi
