// torch.ops.sglb.* — thin adapters from at::Tensor to the raw-pointer kernel API (kernels/api.h).
// Loaded with torch.ops.load_library(sglang_b200/_C.so).  Every adapter bumps a launch counter so bench.py can
// report how many of OUR kernels ran inside the timed region (CUDA-graph replays are accounted in Python).
#include <ATen/cuda/CUDAContext.h>
#include <c10/cuda/CUDAGuard.h>
#include <torch/library.h>
#include <torch/types.h>

#include <atomic>

#include "kernels/api.h"

namespace {

std::atomic<int64_t> g_launches{0};
inline void count(int n = 1) { g_launches.fetch_add(n, std::memory_order_relaxed); }
inline cudaStream_t cur_stream() { return at::cuda::getCurrentCUDAStream().stream(); }
int num_sms() {
  static int n = 0;
  if (!n) {
    int dev = 0;
    cudaGetDevice(&dev);
    cudaDeviceGetAttribute(&n, cudaDevAttrMultiProcessorCount, dev);
  }
  return n;
}
#define CHECK_CUDA(t) TORCH_CHECK((t).is_cuda(), #t " must be a CUDA tensor")
#define CHECK_BF16(t) TORCH_CHECK((t).scalar_type() == at::kBFloat16, #t " must be bfloat16")
#define CHECK_I32(t) TORCH_CHECK((t).scalar_type() == at::kInt, #t " must be int32")
#define CHECK_LAST_CONTIG(t) TORCH_CHECK((t).stride(-1) == 1, #t " must be contiguous in the last dim")
template <typename T>
const T* opt_ptr(const c10::optional<at::Tensor>& t) { return t.has_value() ? t->data_ptr<T>() : nullptr; }
template <typename T>
T* opt_mptr(const c10::optional<at::Tensor>& t) { return t.has_value() ? t->data_ptr<T>() : nullptr; }

int64_t launch_count() { return g_launches.load(); }
void reset_launch_count() { g_launches.store(0); }

void rmsnorm(at::Tensor x, c10::optional<at::Tensor> residual, const at::Tensor& w, at::Tensor out, double eps, bool gemma) {
  CHECK_CUDA(x); CHECK_BF16(x); CHECK_BF16(w); CHECK_BF16(out); CHECK_LAST_CONTIG(x); CHECK_LAST_CONTIG(out);
  TORCH_CHECK(x.dim() == 2 && out.dim() == 2);
  if (residual.has_value()) { CHECK_BF16(*residual); TORCH_CHECK(residual->is_contiguous()); }
  c10::cuda::CUDAGuard g(x.device());
  sglb::rmsnorm(x.data_ptr(), residual.has_value() ? residual->data_ptr() : nullptr, w.data_ptr(), out.data_ptr(),
                (int)x.size(0), (int)x.size(1), (int)x.stride(0), (int)out.stride(0), (float)eps, gemma, cur_stream());
  count();
}

void act_and_mul(const at::Tensor& x, at::Tensor out, int64_t act) {
  CHECK_CUDA(x); CHECK_BF16(x); CHECK_BF16(out); CHECK_LAST_CONTIG(x); TORCH_CHECK(out.is_contiguous());
  c10::cuda::CUDAGuard g(x.device());
  sglb::act_and_mul(x.data_ptr(), out.data_ptr(), (int)x.size(0), (int)out.size(1), (int)x.stride(0), (int)act, cur_stream());
  count();
}

void rope_kv_write(at::Tensor q, const at::Tensor& k, const at::Tensor& v, const at::Tensor& positions,
                   const at::Tensor& cos_sin, at::Tensor k_cache, at::Tensor v_cache, const at::Tensor& out_loc, bool neox,
                   double k_scale, double v_scale, int64_t nslabs, int64_t slab_stride) {
  CHECK_CUDA(q); CHECK_BF16(q); CHECK_BF16(k); CHECK_BF16(v); CHECK_I32(positions); CHECK_I32(out_loc);
  TORCH_CHECK(q.dim() == 3 && k.dim() == 3 && v.dim() == 3, "q/k/v must be [T, H, D]");
  TORCH_CHECK(cos_sin.scalar_type() == at::kFloat && cos_sin.is_contiguous());
  TORCH_CHECK(q.stride(2) == 1 && q.stride(1) == q.size(2) && k.stride(1) == k.size(2) && v.stride(1) == v.size(2));
  const bool fp8 = k_cache.scalar_type() == at::kFloat8_e4m3fn;
  TORCH_CHECK(fp8 || k_cache.scalar_type() == at::kBFloat16, "kv cache must be bf16 or fp8_e4m3");
  TORCH_CHECK(k_cache.is_contiguous() && v_cache.is_contiguous());
  c10::cuda::CUDAGuard g(q.device());
  sglb::rope_kv_write(q.data_ptr(), k.data_ptr(), v.data_ptr(), positions.data_ptr<int>(), cos_sin.data_ptr<float>(),
                      k_cache.data_ptr(), v_cache.data_ptr(), out_loc.data_ptr<int>(), (int)q.size(0), (int)q.size(1),
                      (int)k.size(1), (int)q.size(2), (int)cos_sin.size(1), (int)q.stride(0), (int)k.stride(0),
                      (int)v.stride(0), neox, fp8, (float)k_scale, (float)v_scale, (int)std::max<int64_t>(1, nslabs), (long long)slab_stride,
                      cur_stream());
  count();
}

void apply_pt_delta(at::Tensor page_table, const at::Tensor& rows, const at::Tensor& cols, const at::Tensor& vals,
                    c10::optional<at::Tensor> n, int64_t n_max) {
  CHECK_CUDA(page_table); CHECK_I32(page_table); CHECK_I32(rows); CHECK_I32(cols); CHECK_I32(vals);
  if (n_max <= 0) return;
  c10::cuda::CUDAGuard g(page_table.device());
  sglb::apply_pt_delta(page_table.data_ptr<int>(), (int)page_table.stride(0), rows.data_ptr<int>(), cols.data_ptr<int>(),
                       vals.data_ptr<int>(), opt_ptr<int>(n), (int)n_max, cur_stream());
  count();
}

void embedding(const at::Tensor& weight, const at::Tensor& ids, c10::optional<at::Tensor> gather_idx, at::Tensor out,
               int64_t vocab_start) {
  CHECK_CUDA(weight); CHECK_BF16(weight); CHECK_I32(ids); CHECK_BF16(out);
  TORCH_CHECK(weight.is_contiguous() && out.is_contiguous());
  c10::cuda::CUDAGuard g(weight.device());
  sglb::embedding(weight.data_ptr(), ids.data_ptr<int>(), opt_ptr<int>(gather_idx), out.data_ptr(), (int)out.size(0),
                  (int)weight.size(1), (int)weight.size(0), (int)vocab_start, cur_stream());
  count();
}

void gather_rows(const at::Tensor& x, const at::Tensor& idx, at::Tensor out) {
  CHECK_CUDA(x); CHECK_BF16(x); CHECK_I32(idx); CHECK_LAST_CONTIG(x); TORCH_CHECK(out.is_contiguous());
  c10::cuda::CUDAGuard g(x.device());
  sglb::gather_rows(x.data_ptr(), idx.data_ptr<int>(), out.data_ptr(), (int)idx.size(0), (int)x.size(1), (int)x.stride(0),
                    cur_stream());
  count();
}

// impl: 0 = tcgen05, 1 = SIMT reference
void attn_fwd(const at::Tensor& q, const at::Tensor& k_cache, const at::Tensor& v_cache, at::Tensor out,
              c10::optional<at::Tensor> lse, c10::optional<at::Tensor> part_o, c10::optional<at::Tensor> part_lse,
              const at::Tensor& page_table, const at::Tensor& req_slots, const at::Tensor& seq_lens,
              c10::optional<at::Tensor> cu_q, c10::optional<at::Tensor> tok2req, int64_t max_q_len, int64_t page_size,
              int64_t num_splits, double scale, bool causal, int64_t window, double logit_cap, double k_scale,
              double v_scale, int64_t impl, c10::optional<at::Tensor> tree_anc, c10::optional<at::Tensor> slopes,
              c10::optional<at::Tensor> log_rates, int64_t keep_first) {
  CHECK_CUDA(q); CHECK_BF16(q); CHECK_BF16(out); CHECK_I32(page_table); CHECK_I32(req_slots); CHECK_I32(seq_lens);
  TORCH_CHECK(q.dim() == 3 && q.stride(2) == 1 && q.stride(1) == q.size(2), "q must be [T, Hq, D] with packed heads");
  TORCH_CHECK(k_cache.dim() == 3 && v_cache.dim() == 3, "k_cache must be [slots, Hkv, D]");
  // the tcgen05 kernels read the caches through tensor maps: a layer may use the leading Hkv * D columns of wider pool rows
  const bool tc_impl = impl == 0 || impl == 2;
  const bool rows_ok = k_cache.stride(2) == 1 && k_cache.stride(1) == k_cache.size(2) && v_cache.strides() == k_cache.strides() &&
                       k_cache.stride(0) >= k_cache.size(1) * k_cache.size(2);
  TORCH_CHECK(out.is_contiguous() && (tc_impl ? rows_ok : (k_cache.is_contiguous() && v_cache.is_contiguous())), "attn_fwd: cache layout");
  const int kv_stride = (int)k_cache.stride(0);
  const int T = (int)q.size(0), Hq = (int)q.size(1), D = (int)q.size(2), Hkv = (int)k_cache.size(1);
  const int B = (int)req_slots.size(0);
  const bool fp8 = k_cache.scalar_type() == at::kFloat8_e4m3fn;
  c10::cuda::CUDAGuard g(q.device());
  if (slopes.has_value())      // per-head distance bias (tcgen05 kernels only)
    TORCH_CHECK((impl == 0 || impl == 2) && slopes->scalar_type() == at::kFloat && slopes->is_contiguous() && slopes->numel() == Hq && causal,
                "attn_fwd: slopes must be fp32 [Hq] on the tcgen05 kernels, causal");
  if (log_rates.has_value())   // logarithmic form of the distance bias: slopes[h] * ln(1 + log_rates[h] * distance)
    TORCH_CHECK(slopes.has_value() && log_rates->scalar_type() == at::kFloat && log_rates->is_contiguous() && log_rates->numel() == Hq && logit_cap <= 0.0,
                "attn_fwd: log_rates must be fp32 [Hq], given with slopes and without a soft cap");
  if (keep_first > 0)          // kept first tokens of a window (tcgen05 kernels only)
    TORCH_CHECK((impl == 0 || impl == 2) && causal && !tree_anc.has_value(), "attn_fwd: kept first tokens need the tcgen05 kernels, causal");
  if (impl == 0 || impl == 2) {
    TORCH_CHECK(!fp8, "tcgen05 attention: fp8 KV cache not yet supported (use impl=1)");
    if (num_splits > 1) TORCH_CHECK(part_o.has_value() && part_lse.has_value(), "split-KV needs workspaces");
    // persistent kernels take work items from an atomic counter (one zero-initialised [next, done] pair per device, re-armed by the kernel)
    static at::Tensor sched[16];
    const int di = q.get_device();
    TORCH_CHECK(di >= 0 && di < 16);
    if (!sched[di].defined()) {
      cudaStreamCaptureStatus cst = cudaStreamCaptureStatusNone;
      cudaStreamIsCapturing(cur_stream(), &cst);
      TORCH_CHECK(cst == cudaStreamCaptureStatusNone, "attn_fwd: first call on this device is inside a CUDA-graph capture (warm up eagerly first)");
      sched[di] = at::zeros({2}, q.options().dtype(at::kInt));
    }
    int* sched_ptr = sched[di].data_ptr<int>();
    // decode (one query token per request): keys-as-M kernel (attention_decode.cu) unless SGLB_ATTN_DECODE=v2 asks for the query-major one
    static const bool decode_v3 = [] { const char* e = getenv("SGLB_ATTN_DECODE"); return !(e && std::string(e) == "v2"); }();
    if (tree_anc.has_value())
      TORCH_CHECK(cu_q.has_value() && tree_anc->scalar_type() == at::kInt && tree_anc->is_contiguous() && tree_anc->numel() == T,
                  "tree_anc must be int32 [T] (ancestor bits per query token)");
    if (!cu_q.has_value() && decode_v3 && sglb::attn_decode_tc_supported(Hq, Hkv, D, (int)page_size)) {
      TORCH_CHECK(T == B, "decode attention expects one query token per request");
      sglb::attn_decode_tc(q.data_ptr(), k_cache.data_ptr(), v_cache.data_ptr(), out.data_ptr(), opt_mptr<float>(lse), opt_mptr<float>(part_o),
                           opt_mptr<float>(part_lse), page_table.data_ptr<int>(), (int)page_table.stride(0), req_slots.data_ptr<int>(),
                           seq_lens.data_ptr<int>(), B, (int)q.stride(0), Hq, Hkv, D, (int)k_cache.size(0), (int)page_size, (int)num_splits,
                           (float)scale, (int)window, (float)logit_cap, sched_ptr, num_sms(), cur_stream(), opt_ptr<float>(slopes), opt_ptr<float>(log_rates),
                           (int)keep_first, kv_stride);
      count(num_splits > 1 ? 2 : 1);
      return;
    }
    if (impl != 2) sched_ptr = nullptr;      // impl 0: classic (non-persistent) launch of the query-major kernel
    sglb::attn_fwd_tc(q.data_ptr(), k_cache.data_ptr(), v_cache.data_ptr(), out.data_ptr(), opt_mptr<float>(lse),
                      opt_mptr<float>(part_o), opt_mptr<float>(part_lse), page_table.data_ptr<int>(),
                      (int)page_table.stride(0), req_slots.data_ptr<int>(), seq_lens.data_ptr<int>(), opt_ptr<int>(cu_q), B, T,
                      (int)q.stride(0), (int)max_q_len, Hq, Hkv, D, (int)k_cache.size(0), (int)page_size, (int)num_splits,
                      (float)scale, causal ? 1 : 0, (int)window, (float)logit_cap, sched_ptr, num_sms(), cur_stream(),
                      tree_anc.has_value() ? reinterpret_cast<const unsigned*>(tree_anc->data_ptr<int>()) : nullptr, opt_ptr<float>(slopes),
                      opt_ptr<float>(log_rates), (int)keep_first, kv_stride);
    count(num_splits > 1 ? 2 : 1);
  } else {
    TORCH_CHECK(!tree_anc.has_value(), "tree masks need the tcgen05 attention (impl 0 / 2)");
    sglb::attn_fwd_simt(q.data_ptr(), k_cache.data_ptr(), v_cache.data_ptr(), out.data_ptr(), opt_mptr<float>(lse),
                        page_table.data_ptr<int>(), (int)page_table.stride(0), req_slots.data_ptr<int>(),
                        seq_lens.data_ptr<int>(), opt_ptr<int>(cu_q), opt_ptr<int>(tok2req), T, (int)q.stride(0), Hq, Hkv, D,
                        (int)page_size, (float)scale, causal ? 1 : 0, (int)window, (float)logit_cap, fp8, (float)k_scale,
                        (float)v_scale, cur_stream());
    count();
  }
}

// Mamba: causal depthwise conv1d over a ragged batch with the rolling per-request state (decode when cu_q is None)
void causal_conv1d(const at::Tensor& x, const at::Tensor& w, c10::optional<at::Tensor> bias, at::Tensor conv_state, c10::optional<at::Tensor> cu_q,
                   const at::Tensor& req_slots, const at::Tensor& seq_lens, int64_t max_q_len, bool silu, at::Tensor u) {
  CHECK_CUDA(x); CHECK_CUDA(conv_state); CHECK_I32(req_slots); CHECK_I32(seq_lens);
  TORCH_CHECK(x.dim() == 2 && x.stride(1) == 1 && w.dim() == 2 && w.is_contiguous() && conv_state.dim() == 3 && conv_state.is_contiguous());
  const bool bf16 = x.scalar_type() == at::kBFloat16;
  TORCH_CHECK((bf16 || x.scalar_type() == at::kFloat) && w.scalar_type() == x.scalar_type() && conv_state.scalar_type() == x.scalar_type(),
              "causal_conv1d: x / weight / state must share bf16 or fp32");
  const int C = (int)x.size(1), K = (int)w.size(1);
  TORCH_CHECK(w.size(0) == C && conv_state.size(1) == C && conv_state.size(2) == K - 1 && u.scalar_type() == at::kFloat && u.stride(1) == 1 &&
              u.size(0) == x.size(0) && u.size(1) == C);
  if (bias.has_value()) TORCH_CHECK(bias->scalar_type() == x.scalar_type() && bias->numel() == C);
  c10::cuda::CUDAGuard g(x.device());
  sglb::causal_conv1d(x.data_ptr(), (int)x.stride(0), w.data_ptr(), bias.has_value() ? bias->data_ptr() : nullptr, conv_state.data_ptr(),
                      opt_ptr<int>(cu_q), req_slots.data_ptr<int>(), seq_lens.data_ptr<int>(), (int)req_slots.size(0), (int)max_q_len, C, K, silu, bf16,
                      u.data_ptr<float>(), (int)u.stride(0), cur_stream());
  count(2);
}

// Mamba-2 decode: S = S * exp(dt A) + dt x B ; y = <S, C> + D x   (state fp32 [slots, H, P, N], one token per request)
void selective_state_update(at::Tensor state, const at::Tensor& req_slots, const at::Tensor& x, const at::Tensor& dt, const at::Tensor& A,
                            const at::Tensor& Bm, const at::Tensor& Cm, c10::optional<at::Tensor> D, at::Tensor y) {
  CHECK_CUDA(state); CHECK_I32(req_slots);
  TORCH_CHECK(state.dim() == 4 && state.is_contiguous() && state.scalar_type() == at::kFloat);
  const int H = (int)state.size(1), P = (int)state.size(2), N = (int)state.size(3), B = (int)req_slots.size(0);
  for (const at::Tensor* t : std::initializer_list<const at::Tensor*>{&x, &dt, &A, &Bm, &Cm, &y})
    TORCH_CHECK(t->scalar_type() == at::kFloat && t->is_cuda(), "selective_state_update: fp32 CUDA tensors");
  TORCH_CHECK(x.dim() == 2 && x.stride(1) == 1 && x.size(0) == B && x.size(1) == H * P && dt.is_contiguous() && dt.numel() == B * H && A.numel() == H);
  TORCH_CHECK(Bm.dim() == 2 && Bm.stride(1) == 1 && Cm.dim() == 2 && Cm.stride(1) == 1 && Bm.stride(0) == Cm.stride(0) && Bm.size(1) % N == 0);
  TORCH_CHECK((reinterpret_cast<uintptr_t>(Bm.data_ptr()) & 15) == 0 && (reinterpret_cast<uintptr_t>(Cm.data_ptr()) & 15) == 0 && Bm.stride(0) % 4 == 0,
              "selective_state_update: B / C rows must be 16-byte aligned");
  const int G = (int)(Bm.size(1) / N);
  TORCH_CHECK(y.is_contiguous() && y.numel() == (int64_t)B * H * P);
  c10::cuda::CUDAGuard g(state.device());
  sglb::selective_state_update(state.data_ptr<float>(), req_slots.data_ptr<int>(), x.data_ptr<float>(), (int)x.stride(0), dt.data_ptr<float>(),
                               A.data_ptr<float>(), Bm.data_ptr<float>(), Cm.data_ptr<float>(), (int)Bm.stride(0),
                               D.has_value() ? D->data_ptr<float>() : nullptr, B, H, P, N, G, y.data_ptr<float>(), cur_stream());
  count();
}

// gated delta rule decode step (Qwen3-Next): u = conv output rows [q (Hk*Dk) | k (Hk*Dk) | v (Hv*Dv)], state fp32 [slots, Hv, Dk, Dv]
void gated_delta_update(at::Tensor state, const at::Tensor& req_slots, const at::Tensor& u, const at::Tensor& g, const at::Tensor& beta, int64_t Hk,
                        at::Tensor out) {
  CHECK_CUDA(state); CHECK_I32(req_slots);
  TORCH_CHECK(state.dim() == 4 && state.is_contiguous() && state.scalar_type() == at::kFloat && u.scalar_type() == at::kFloat && u.dim() == 2 &&
              u.stride(1) == 1 && g.scalar_type() == at::kFloat && beta.scalar_type() == at::kFloat && g.is_contiguous() && beta.is_contiguous() &&
              out.scalar_type() == at::kFloat && out.is_contiguous());
  const int Hv = (int)state.size(1), Dk = (int)state.size(2), Dv = (int)state.size(3), B = (int)req_slots.size(0);
  TORCH_CHECK(Hk > 0 && Hv % Hk == 0 && u.size(0) == B && u.size(1) == 2 * Hk * Dk + (int64_t)Hv * Dv && g.numel() == (int64_t)B * Hv &&
              out.numel() == (int64_t)B * Hv * Dv);
  c10::cuda::CUDAGuard guard(state.device());
  const bool ok = sglb::gated_delta_update(state.data_ptr<float>(), req_slots.data_ptr<int>(), u.data_ptr<float>(), (int)u.stride(0), (int)(Hk * Dk),
                                           (int)(2 * Hk * Dk), g.data_ptr<float>(), beta.data_ptr<float>(), B, Hv, (int)(Hv / Hk), Dk, Dv,
                                           out.data_ptr<float>(), cur_stream());
  TORCH_CHECK(ok, "gated_delta_update: key dim must be 64 or 128 and value dim <= 256");
  count();
}

void add_rmsnorm_f32(at::Tensor residual, c10::optional<at::Tensor> delta, const at::Tensor& w, at::Tensor out, double eps, bool zero_centred) {
  CHECK_CUDA(residual);
  TORCH_CHECK(residual.scalar_type() == at::kFloat && residual.dim() == 2 && residual.is_contiguous() && out.is_contiguous() && w.is_contiguous());
  TORCH_CHECK(out.scalar_type() == w.scalar_type() && (out.scalar_type() == at::kFloat || out.scalar_type() == at::kBFloat16));
  TORCH_CHECK(out.numel() == residual.numel() && (w.numel() == residual.size(1) || w.numel() == 1));          // one element: one gain for all
  bool dbf = false;
  if (delta.has_value()) {
    TORCH_CHECK(delta->is_contiguous() && delta->numel() == residual.numel() && (delta->scalar_type() == at::kFloat || delta->scalar_type() == at::kBFloat16));
    dbf = delta->scalar_type() == at::kBFloat16;
  }
  c10::cuda::CUDAGuard g(residual.device());
  sglb::add_rmsnorm_f32(residual.data_ptr<float>(), delta.has_value() ? delta->data_ptr() : nullptr, dbf, w.data_ptr(), out.data_ptr(),
                        out.scalar_type() == at::kBFloat16, (int)residual.size(0), (int)residual.size(1), (float)eps, zero_centred,
                        w.numel() == 1 && residual.size(1) != 1 ? 0 : 1, cur_stream());
  count();
}

void clamped_glu(const at::Tensor& gu, at::Tensor out, double limit, double alpha) {
  CHECK_CUDA(gu);
  TORCH_CHECK(gu.dim() == 2 && gu.is_contiguous() && out.is_contiguous() && gu.scalar_type() == out.scalar_type() && gu.size(1) % 2 == 0 &&
              out.numel() * 2 == gu.numel() && (gu.scalar_type() == at::kFloat || gu.scalar_type() == at::kBFloat16));
  c10::cuda::CUDAGuard g(gu.device());
  sglb::clamped_glu(gu.data_ptr(), out.data_ptr(), gu.scalar_type() == at::kBFloat16, (int)gu.size(0), (int)(gu.size(1) / 2), (float)limit,
                    (float)alpha, cur_stream());
  count();
}

void gated_delta_rule(const at::Tensor& u, int64_t Hk, int64_t Dk, int64_t H, int64_t Dv, const at::Tensor& a_raw, const at::Tensor& A_log,
                      const at::Tensor& dt_bias, const at::Tensor& b_raw, at::Tensor state, const at::Tensor& req_slots, const at::Tensor& seq_lens,
                      c10::optional<at::Tensor> cu_q, c10::optional<at::Tensor> gate_raw, c10::optional<at::Tensor> norm_w, double eps,
                      bool gate_silu, bool per_channel, at::Tensor out) {
  CHECK_CUDA(u); CHECK_I32(req_slots); CHECK_I32(seq_lens);
  auto f32c = [](const at::Tensor& t) { return t.scalar_type() == at::kFloat && t.is_contiguous(); };
  TORCH_CHECK(f32c(u) && f32c(a_raw) && f32c(A_log) && f32c(dt_bias) && f32c(b_raw) && f32c(state) && f32c(out) && u.dim() == 2);
  const int64_t T = u.size(0);
  const int B = (int)req_slots.size(0);
  TORCH_CHECK(Hk > 0 && H % Hk == 0 && u.size(1) == 2 * Hk * Dk + H * Dv && state.dim() == 4 && state.size(1) == H && state.size(2) == Dk &&
              state.size(3) == Dv && out.numel() == T * H * Dv && b_raw.numel() == T * H && A_log.numel() == H);
  const int64_t nd = per_channel ? H * Dk : H;
  TORCH_CHECK(a_raw.numel() == T * nd && dt_bias.numel() == nd, "gated_delta_rule: decay input must be [T, H] or (per channel) [T, H * Dk]");
  TORCH_CHECK(gate_raw.has_value() == norm_w.has_value());
  if (gate_raw.has_value()) TORCH_CHECK(f32c(*gate_raw) && f32c(*norm_w) && gate_raw->numel() == T * H * Dv && norm_w->numel() == Dv);
  if (cu_q.has_value()) { CHECK_I32(*cu_q); TORCH_CHECK(cu_q->numel() == B + 1); } else TORCH_CHECK(T == B);
  if (T == 0) return;
  c10::cuda::CUDAGuard g(u.device());
  const bool ok = sglb::gated_delta_rule(u.data_ptr<float>(), (int)u.stride(0), (int)Hk, (int)Dk, (int)H, (int)Dv, a_raw.data_ptr<float>(), per_channel,
                                         A_log.data_ptr<float>(), dt_bias.data_ptr<float>(), b_raw.data_ptr<float>(), opt_ptr<float>(gate_raw),
                                         opt_ptr<float>(norm_w), (float)eps, gate_silu, state.data_ptr<float>(), req_slots.data_ptr<int>(),
                                         seq_lens.data_ptr<int>(), opt_ptr<int>(cu_q), B, out.data_ptr<float>(), cur_stream());
  TORCH_CHECK(ok, "gated_delta_rule: head shape (key dim ", Dk, ", value dim ", Dv, ") does not fit one CTA per head");
  count();
}

// ---- bigram embedding / sandwich norms / Mamba-2 scan / biased window attention / identity-expert router
static bool bf16_or_f32(const at::Tensor& t) { return t.scalar_type() == at::kBFloat16 || t.scalar_type() == at::kFloat; }

void bigram_embedding(const at::Tensor& embed, c10::optional<at::Tensor> bigram, const at::Tensor& ids, c10::optional<at::Tensor> prev_tokens,
                      c10::optional<at::Tensor> cu_q, const at::Tensor& req_slots, const at::Tensor& seq_lens, int64_t max_q_len, double scale,
                      int64_t mul_prev, int64_t mul_cur, int64_t buckets, at::Tensor out) {
  CHECK_CUDA(embed); CHECK_I32(ids); CHECK_I32(req_slots); CHECK_I32(seq_lens);
  TORCH_CHECK(bf16_or_f32(embed) && embed.dim() == 2 && embed.is_contiguous() && ids.is_contiguous() && out.scalar_type() == at::kFloat &&
              out.is_contiguous() && out.size(0) == ids.size(0) && out.size(1) == embed.size(1));
  const int B = (int)req_slots.size(0);
  if (cu_q.has_value()) { CHECK_I32(*cu_q); TORCH_CHECK(cu_q->numel() == B + 1); } else TORCH_CHECK(ids.size(0) == B);
  if (bigram.has_value()) {
    TORCH_CHECK(bigram->scalar_type() == embed.scalar_type() && bigram->is_contiguous() && bigram->size(1) == embed.size(1) && buckets > 0 &&
                bigram->size(0) > buckets && prev_tokens.has_value() && prev_tokens->scalar_type() == at::kInt && prev_tokens->is_contiguous());
  }
  if (ids.size(0) == 0) return;
  c10::cuda::CUDAGuard g(embed.device());
  sglb::bigram_embedding(embed.data_ptr(), bigram.has_value() ? bigram->data_ptr() : nullptr, embed.scalar_type() == at::kBFloat16, ids.data_ptr<int>(),
                         bigram.has_value() ? prev_tokens->data_ptr<int>() : nullptr, opt_ptr<int>(cu_q), req_slots.data_ptr<int>(),
                         seq_lens.data_ptr<int>(), B, cu_q.has_value() ? (int)max_q_len : 1, (int)embed.size(1), (int)embed.size(0), (float)scale,
                         (long long)mul_prev, (long long)mul_cur, (int)buckets, out.data_ptr<float>(), cur_stream());
  count();
}

void postnorm_add_rmsnorm_f32(at::Tensor residual, const at::Tensor& delta, const at::Tensor& post_w, const at::Tensor& w, at::Tensor out, double eps,
                              bool zero_centred) {
  CHECK_CUDA(residual);
  TORCH_CHECK(residual.scalar_type() == at::kFloat && residual.dim() == 2 && residual.is_contiguous() && out.is_contiguous() && w.is_contiguous() &&
              post_w.is_contiguous() && delta.is_contiguous() && bf16_or_f32(out) && bf16_or_f32(delta));
  TORCH_CHECK(out.scalar_type() == w.scalar_type() && out.scalar_type() == post_w.scalar_type() && out.numel() == residual.numel() &&
              delta.numel() == residual.numel() && (w.numel() == residual.size(1) || w.numel() == 1) &&
              (post_w.numel() == residual.size(1) || post_w.numel() == 1));
  c10::cuda::CUDAGuard g(residual.device());
  sglb::postnorm_add_rmsnorm_f32(residual.data_ptr<float>(), delta.data_ptr(), delta.scalar_type() == at::kBFloat16, post_w.data_ptr(), w.data_ptr(),
                                 out.data_ptr(), out.scalar_type() == at::kBFloat16, (int)residual.size(0), (int)residual.size(1), (float)eps, zero_centred,
                                 post_w.numel() == 1 && residual.size(1) != 1 ? 0 : 1, w.numel() == 1 && residual.size(1) != 1 ? 0 : 1, cur_stream());
  count();
}

void grouped_rmsnorm(const at::Tensor& x, const at::Tensor& w, int64_t groups, double eps, at::Tensor out, c10::optional<at::Tensor> gate, double out_scale) {
  CHECK_CUDA(x);
  TORCH_CHECK(x.scalar_type() == at::kFloat && x.dim() == 2 && x.is_contiguous() && out.dim() == 2 && out.stride(1) == 1 && w.is_contiguous() &&
              bf16_or_f32(out) && out.scalar_type() == w.scalar_type() && out.size(0) == x.size(0) && out.size(1) == x.size(1) && w.numel() == x.size(1));
  if (gate.has_value())
    TORCH_CHECK(gate->scalar_type() == out.scalar_type() && gate->dim() == 2 && gate->stride(1) == 1 && gate->size(0) == x.size(0) &&
                gate->size(1) == x.size(1));
  if (x.size(0) == 0) return;
  c10::cuda::CUDAGuard g(x.device());
  sglb::grouped_rmsnorm(x.data_ptr<float>(), w.data_ptr(), out.data_ptr(), out.scalar_type() == at::kBFloat16, (int)x.size(0), (int)x.size(1), (int)groups,
                        (float)eps, gate.has_value() ? gate->data_ptr() : nullptr, gate.has_value() ? (int)gate->stride(0) : 0, (int)out.stride(0),
                        (float)out_scale, cur_stream());
  count();
}

void mamba2_scan(const at::Tensor& u, c10::optional<at::Tensor> z, c10::optional<at::Tensor> dt_raw, c10::optional<at::Tensor> dt_bias,
                 c10::optional<at::Tensor> A_log, c10::optional<at::Tensor> D, at::Tensor state, const at::Tensor& req_slots, const at::Tensor& seq_lens,
                 c10::optional<at::Tensor> cu_q, int64_t H, int64_t P, int64_t N, int64_t G, at::Tensor out, c10::optional<at::Tensor> decay,
                 c10::optional<at::Tensor> gates) {
  CHECK_CUDA(u); CHECK_I32(req_slots); CHECK_I32(seq_lens);
  auto f32c = [](const at::Tensor& t) { return t.scalar_type() == at::kFloat && t.is_contiguous(); };
  TORCH_CHECK(f32c(u) && f32c(state) && f32c(out) && u.dim() == 2 && u.size(1) >= H * P + 2 * G * N);
  bool in_bf16 = false;
  const bool fixed = decay.has_value() || gates.has_value();
  if (gates.has_value()) {          // every token brings its decay and step: no step-size inputs
    TORCH_CHECK(!decay.has_value() && f32c(*gates) && gates->dim() == 3 && gates->size(0) == u.size(0) && gates->size(1) == H && gates->size(2) >= 2);
    if (z.has_value()) in_bf16 = z->scalar_type() == at::kBFloat16;
  } else if (decay.has_value()) {          // constant decay per head, step size 1: no step-size inputs
    TORCH_CHECK(f32c(*decay) && decay->numel() == H);
    if (z.has_value()) in_bf16 = z->scalar_type() == at::kBFloat16;
  } else {
    TORCH_CHECK(dt_raw.has_value() && dt_bias.has_value() && A_log.has_value() && f32c(*dt_bias) && f32c(*A_log) && dt_bias->numel() == H && A_log->numel() == H);
    TORCH_CHECK(bf16_or_f32(*dt_raw) && dt_raw->dim() == 2 && dt_raw->stride(1) == 1 && dt_raw->size(1) >= H && dt_raw->size(0) == u.size(0));
    in_bf16 = dt_raw->scalar_type() == at::kBFloat16;
    if (z.has_value()) TORCH_CHECK(z->scalar_type() == dt_raw->scalar_type());
  }
  if (z.has_value()) TORCH_CHECK(bf16_or_f32(*z) && z->dim() == 2 && z->stride(1) == 1 && z->size(1) >= H * P && z->size(0) == u.size(0));
  if (D.has_value()) TORCH_CHECK(f32c(*D) && D->numel() == H);
  TORCH_CHECK(state.dim() == 4 && state.size(1) == H && state.size(2) == N && state.size(3) == P && out.size(0) == u.size(0) &&
              out.numel() == u.size(0) * H * P);
  const int B = (int)req_slots.size(0);
  if (cu_q.has_value()) { CHECK_I32(*cu_q); TORCH_CHECK(cu_q->numel() == B + 1); } else TORCH_CHECK(u.size(0) == B);
  if (u.size(0) == 0) return;
  c10::cuda::CUDAGuard g(u.device());
  sglb::mamba2_scan(u.data_ptr<float>(), (int)u.stride(0), z.has_value() ? z->data_ptr() : nullptr, z.has_value() ? (int)z->stride(0) : 0,
                    fixed ? nullptr : dt_raw->data_ptr(), fixed ? 0 : (int)dt_raw->stride(0), in_bf16,
                    fixed ? nullptr : dt_bias->data_ptr<float>(), fixed ? nullptr : A_log->data_ptr<float>(), opt_ptr<float>(D),
                    state.data_ptr<float>(), req_slots.data_ptr<int>(), seq_lens.data_ptr<int>(), opt_ptr<int>(cu_q), B, (int)H, (int)P, (int)N, (int)G,
                    out.data_ptr<float>(), opt_ptr<float>(decay), opt_ptr<float>(gates), gates.has_value() ? (int)gates->size(2) : 0, cur_stream());
  count();
}

void qk_norm_cache_write(const at::Tensor& qkv, int64_t H, int64_t G, int64_t D, int64_t Dv, const at::Tensor& positions, double eps, double temp_coef,
                         int64_t temp_every, at::Tensor k_cache, at::Tensor v_cache, const at::Tensor& loc, bool normalise, at::Tensor q_out, int64_t pad) {
  CHECK_CUDA(qkv); CHECK_I32(positions); CHECK_I32(loc);
  TORCH_CHECK(bf16_or_f32(qkv) && qkv.dim() == 2 && qkv.stride(1) == 1 && qkv.size(1) == (H + G) * D + G * Dv);
  TORCH_CHECK(k_cache.scalar_type() == qkv.scalar_type() && v_cache.scalar_type() == qkv.scalar_type() && q_out.scalar_type() == qkv.scalar_type() &&
              q_out.is_contiguous() && q_out.numel() == qkv.size(0) * H * (pad > 0 ? pad : D) && (pad == 0 || (pad >= D && pad >= Dv)));
  TORCH_CHECK(k_cache.dim() == 3 && k_cache.size(1) == 1 && k_cache.stride(2) == 1 && v_cache.stride(2) == 1 && k_cache.stride(0) == v_cache.stride(0) &&
              k_cache.size(2) >= G * (pad > 0 ? pad : D) && v_cache.size(2) >= G * (pad > 0 ? pad : Dv) && temp_every >= 1 && positions.numel() == qkv.size(0) && loc.numel() == qkv.size(0));
  if (qkv.size(0) == 0) return;
  c10::cuda::CUDAGuard g(qkv.device());
  sglb::qk_norm_cache_write(qkv.data_ptr(), (int)qkv.stride(0), qkv.scalar_type() == at::kBFloat16, (int)qkv.size(0), (int)H, (int)G, (int)D, (int)Dv,
                            positions.data_ptr<int>(), (float)eps, (float)temp_coef, (int)temp_every, k_cache.data_ptr(), v_cache.data_ptr(),
                            (size_t)k_cache.stride(0), loc.data_ptr<int>(), normalise, q_out.data_ptr(), (int)pad, cur_stream());
  count();
}

void window_attention(const at::Tensor& q, const at::Tensor& k_cache, const at::Tensor& v_cache, int64_t G, int64_t Dv, const at::Tensor& page_table,
                      const at::Tensor& req_slots, const at::Tensor& seq_lens, c10::optional<at::Tensor> cu_q, int64_t max_q_len, int64_t page_size,
                      double scale, double softcap, int64_t window, c10::optional<at::Tensor> slopes, c10::optional<at::Tensor> sinks, at::Tensor out,
                      int64_t dim, int64_t pad, int64_t keep_first, c10::optional<at::Tensor> log_rates, c10::optional<at::Tensor> gate, double out_scale) {
  CHECK_CUDA(q); CHECK_I32(page_table); CHECK_I32(req_slots); CHECK_I32(seq_lens);
  // out: [T, H, Dv] contiguous, or a [T, H * Dv] block of columns of a wider buffer
  TORCH_CHECK(bf16_or_f32(q) && q.dim() == 3 && q.is_contiguous() && out.scalar_type() == q.scalar_type() && out.numel() == q.size(0) * q.size(1) * Dv &&
              (out.is_contiguous() || (out.dim() == 2 && out.stride(1) == 1 && out.size(1) == q.size(1) * Dv)));
  const int ldo = out.dim() == 2 ? (int)out.stride(0) : (int)(q.size(1) * Dv);
  // pad > 0: q [T, H, pad] and every key / value head occupy ``pad`` columns of which the first ``dim`` / ``Dv`` count
  const int64_t H = q.size(1), D = pad > 0 ? dim : q.size(2);
  TORCH_CHECK(pad == 0 || (q.size(2) == pad && D >= 1 && D <= pad && Dv <= pad));
  TORCH_CHECK(k_cache.scalar_type() == q.scalar_type() && v_cache.scalar_type() == q.scalar_type() && k_cache.dim() == 3 && k_cache.size(1) == 1 &&
              k_cache.stride(2) == 1 && v_cache.stride(2) == 1 && k_cache.stride(0) == v_cache.stride(0) && k_cache.size(2) >= G * (pad > 0 ? pad : D) &&
              v_cache.size(2) >= G * (pad > 0 ? pad : Dv) && page_table.dim() == 2 && page_table.stride(1) == 1 && G >= 1 && H % G == 0);
  const int B = (int)req_slots.size(0);
  if (cu_q.has_value()) { CHECK_I32(*cu_q); TORCH_CHECK(cu_q->numel() == B + 1); } else TORCH_CHECK(q.size(0) == B);
  if (sinks.has_value()) TORCH_CHECK(sinks->scalar_type() == at::kFloat && sinks->is_contiguous() && sinks->numel() == H);
  if (slopes.has_value()) TORCH_CHECK(slopes->scalar_type() == at::kFloat && slopes->is_contiguous() && slopes->numel() == H);
  if (log_rates.has_value()) TORCH_CHECK(slopes.has_value() && log_rates->scalar_type() == at::kFloat && log_rates->is_contiguous() && log_rates->numel() == H);
  bool gate_per_head = false;
  if (gate.has_value()) {
    TORCH_CHECK(gate->scalar_type() == q.scalar_type() && gate->dim() == 2 && gate->stride(1) == 1 && gate->size(0) == q.size(0) &&
                (gate->size(1) == H || gate->size(1) == H * Dv));
    gate_per_head = gate->size(1) == H && Dv != 1;
  }
  if (q.size(0) == 0) return;
  c10::cuda::CUDAGuard g(q.device());
  sglb::window_attention(q.data_ptr(), k_cache.data_ptr(), v_cache.data_ptr(), q.scalar_type() == at::kBFloat16, (size_t)k_cache.stride(0), (int)H, (int)G,
                         (int)D, (int)Dv, page_table.data_ptr<int>(), (int)page_table.stride(0), (int)page_size, req_slots.data_ptr<int>(),
                         seq_lens.data_ptr<int>(), opt_ptr<int>(cu_q), B, cu_q.has_value() ? (int)max_q_len : 1, (float)scale, (float)softcap, (int)window,
                         opt_ptr<float>(slopes), opt_ptr<float>(sinks), out.data_ptr(), (int)pad, (int)keep_first, opt_ptr<float>(log_rates),
                         gate.has_value() ? gate->data_ptr() : nullptr, gate.has_value() ? (int)gate->stride(0) : 0, gate_per_head, ldo, (float)out_scale,
                         cur_stream());
  count();
}

void mamba1_scan(const at::Tensor& u, const at::Tensor& dt_raw, c10::optional<at::Tensor> dt_bias, const at::Tensor& A_log, const at::Tensor& Bm,
                 const at::Tensor& Cm, c10::optional<at::Tensor> D, c10::optional<at::Tensor> z, at::Tensor state, const at::Tensor& req_slots,
                 const at::Tensor& seq_lens, c10::optional<at::Tensor> cu_q, at::Tensor out) {
  CHECK_CUDA(u); CHECK_I32(req_slots); CHECK_I32(seq_lens);
  auto f32c = [](const at::Tensor& t) { return t.scalar_type() == at::kFloat && t.is_contiguous(); };
  const int64_t T = u.size(0), C = u.size(1), N = A_log.size(1);
  TORCH_CHECK(f32c(u) && f32c(A_log) && f32c(state) && u.dim() == 2 && A_log.dim() == 2 && A_log.size(0) == C && out.is_contiguous() && bf16_or_f32(out) &&
              out.numel() == u.numel());
  TORCH_CHECK(dt_raw.scalar_type() == at::kFloat && dt_raw.dim() == 2 && dt_raw.stride(1) == 1 && dt_raw.size(0) == T && dt_raw.size(1) == C);
  TORCH_CHECK(bf16_or_f32(Bm) && Bm.scalar_type() == Cm.scalar_type() && Bm.dim() == 2 && Cm.dim() == 2 && Bm.stride(1) == 1 && Cm.stride(1) == 1 &&
              Bm.stride(0) == Cm.stride(0) && Bm.size(0) == T && Cm.size(0) == T && Bm.size(1) == N && Cm.size(1) == N);
  if (dt_bias.has_value()) TORCH_CHECK(f32c(*dt_bias) && dt_bias->numel() == C);
  if (D.has_value()) TORCH_CHECK(f32c(*D) && D->numel() == C);
  if (z.has_value()) TORCH_CHECK(bf16_or_f32(*z) && z->dim() == 2 && z->stride(1) == 1 && z->size(0) == T && z->size(1) == C);
  TORCH_CHECK(state.numel() == state.size(0) * C * N);
  const int B = (int)req_slots.size(0);
  if (cu_q.has_value()) { CHECK_I32(*cu_q); TORCH_CHECK(cu_q->numel() == B + 1); } else TORCH_CHECK(T == B);
  if (T == 0) return;
  c10::cuda::CUDAGuard g(u.device());
  sglb::mamba1_scan(u.data_ptr<float>(), dt_raw.data_ptr<float>(), (int)dt_raw.stride(0), opt_ptr<float>(dt_bias), A_log.data_ptr<float>(), Bm.data_ptr(),
                    Cm.data_ptr(), (int)Bm.stride(0), Bm.scalar_type() == at::kBFloat16, opt_ptr<float>(D), z.has_value() ? z->data_ptr() : nullptr,
                    z.has_value() ? (int)z->stride(0) : 0, z.has_value() && z->scalar_type() == at::kBFloat16, state.data_ptr<float>(),
                    req_slots.data_ptr<int>(), seq_lens.data_ptr<int>(), opt_ptr<int>(cu_q), B, (int)C, (int)N, out.data_ptr(),
                    out.scalar_type() == at::kBFloat16, cur_stream());
  count();
}

void attention_prepare(const at::Tensor& qkv, int64_t H, int64_t G, int64_t D, int64_t Dv, const at::Tensor& positions, at::Tensor k_cache, at::Tensor v_cache,
                       const at::Tensor& loc, c10::optional<at::Tensor> q_norm_w, c10::optional<at::Tensor> k_norm_w, double eps,
                       c10::optional<at::Tensor> inv_freq, c10::optional<at::Tensor> v_first, double v_lambda, at::Tensor q_out, int64_t pad,
                       c10::optional<at::Tensor> v_inv_freq, bool v_interleaved) {
  CHECK_CUDA(qkv); CHECK_I32(positions); CHECK_I32(loc);
  const int64_t T = qkv.size(0);
  TORCH_CHECK(bf16_or_f32(qkv) && qkv.dim() == 2 && qkv.stride(1) == 1 && qkv.size(1) >= H * D + G * D + G * Dv && H % G == 0);
  TORCH_CHECK(pad == 0 || (D <= pad && Dv <= pad));
  const int64_t hs = pad > 0 ? pad : D, hv = pad > 0 ? pad : Dv;
  TORCH_CHECK(q_out.is_contiguous() && q_out.scalar_type() == qkv.scalar_type() && q_out.numel() == T * H * hs);
  TORCH_CHECK(k_cache.scalar_type() == qkv.scalar_type() && v_cache.scalar_type() == qkv.scalar_type() && k_cache.dim() == 3 && k_cache.size(1) == 1 &&
              k_cache.stride(2) == 1 && v_cache.stride(2) == 1 && k_cache.stride(0) == v_cache.stride(0) && k_cache.size(2) >= G * hs &&
              v_cache.size(2) >= G * hv && positions.numel() == T && loc.numel() == T);
  TORCH_CHECK(q_norm_w.has_value() == k_norm_w.has_value());
  if (q_norm_w.has_value())
    TORCH_CHECK(q_norm_w->scalar_type() == qkv.scalar_type() && k_norm_w->scalar_type() == qkv.scalar_type() && q_norm_w->is_contiguous() &&
                k_norm_w->is_contiguous() && q_norm_w->numel() == H * D && k_norm_w->numel() == G * D);
  int half = 0;
  if (inv_freq.has_value()) {
    TORCH_CHECK(inv_freq->scalar_type() == at::kFloat && inv_freq->is_contiguous() && 2 * inv_freq->numel() <= D);
    half = (int)inv_freq->numel();
  }
  if (v_first.has_value())
    TORCH_CHECK(v_first->scalar_type() == qkv.scalar_type() && v_first->dim() == 2 && v_first->stride(1) == 1 && v_first->size(0) == T &&
                v_first->size(1) == G * Dv);
  if (v_inv_freq.has_value())
    TORCH_CHECK(v_inv_freq->scalar_type() == at::kFloat && v_inv_freq->is_contiguous() && Dv % 2 == 0 && v_inv_freq->numel() == Dv / 2);
  if (T == 0) return;
  c10::cuda::CUDAGuard g(qkv.device());
  sglb::attention_prepare(qkv.data_ptr(), (int)qkv.stride(0), qkv.scalar_type() == at::kBFloat16, (int)T, (int)H, (int)G, (int)D, (int)Dv,
                          positions.data_ptr<int>(), q_norm_w.has_value() ? q_norm_w->data_ptr() : nullptr, k_norm_w.has_value() ? k_norm_w->data_ptr() : nullptr,
                          (float)eps, half > 0 ? inv_freq->data_ptr<float>() : nullptr, half, v_first.has_value() ? v_first->data_ptr() : nullptr,
                          v_first.has_value() ? (int)v_first->stride(0) : 0, (float)v_lambda, k_cache.data_ptr(), v_cache.data_ptr(), (size_t)k_cache.stride(0),
                          loc.data_ptr<int>(), q_out.data_ptr(), (int)pad, opt_ptr<float>(v_inv_freq), v_interleaved, cur_stream());
  count();
}

void sigmoid_gate(const at::Tensor& o, const at::Tensor& gate, int64_t Dv, double out_scale, at::Tensor out) {
  CHECK_CUDA(o);
  const int64_t T = o.size(0), H = o.size(1);
  TORCH_CHECK(bf16_or_f32(o) && o.dim() == 3 && o.is_contiguous() && Dv >= 1 && Dv <= o.size(2) && out.scalar_type() == o.scalar_type() && out.dim() == 2 &&
              out.stride(1) == 1 && out.size(0) == T && out.size(1) == H * Dv);
  TORCH_CHECK(gate.scalar_type() == o.scalar_type() && gate.dim() == 2 && gate.stride(1) == 1 && gate.size(0) == T && (gate.size(1) == H || gate.size(1) == H * Dv));
  if (T == 0) return;
  c10::cuda::CUDAGuard g(o.device());
  sglb::sigmoid_gate(o.data_ptr(), (int)o.size(2), gate.data_ptr(), (int)gate.stride(0), gate.size(1) == H && Dv != 1, o.scalar_type() == at::kBFloat16, (int)T,
                     (int)H, (int)Dv, (float)out_scale, out.data_ptr(), (int)out.stride(0), cur_stream());
  count();
}

void activation(const at::Tensor& x, int64_t act, at::Tensor out, c10::optional<at::Tensor> mul) {
  CHECK_CUDA(x);
  TORCH_CHECK(bf16_or_f32(x) && bf16_or_f32(out) && x.dim() == 2 && x.stride(1) == 1 && out.is_contiguous() && out.numel() == x.numel() && (act == 0 || act == 2));
  if (mul.has_value())
    TORCH_CHECK(mul->scalar_type() == x.scalar_type() && mul->dim() == 2 && mul->stride(1) == 1 && mul->size(0) == x.size(0) && mul->size(1) == x.size(1));
  if (x.numel() == 0) return;
  c10::cuda::CUDAGuard g(x.device());
  sglb::activation(x.data_ptr(), (int)x.stride(0), x.scalar_type() == at::kBFloat16, out.data_ptr(), out.scalar_type() == at::kBFloat16, (int)x.size(0),
                   (int)x.size(1), (int)act, mul.has_value() ? mul->data_ptr() : nullptr, mul.has_value() ? (int)mul->stride(0) : 0, cur_stream());
  count();
}

void attention_sink_gate(const at::Tensor& o, const at::Tensor& lse, const at::Tensor& sinks, int64_t Dv, at::Tensor out) {
  CHECK_CUDA(o); CHECK_BF16(o); CHECK_BF16(out);
  TORCH_CHECK(o.dim() == 3 && o.is_contiguous() && out.is_contiguous() && Dv >= 1 && Dv <= o.size(2) && out.numel() == o.size(0) * o.size(1) * Dv);
  TORCH_CHECK(lse.scalar_type() == at::kFloat && lse.is_contiguous() && lse.numel() == o.size(0) * o.size(1) && sinks.scalar_type() == at::kFloat &&
              sinks.is_contiguous() && sinks.numel() == o.size(1));
  if (o.size(0) == 0) return;
  c10::cuda::CUDAGuard g(o.device());
  sglb::attention_sink_gate(o.data_ptr(), (int)o.size(2), lse.data_ptr<float>(), sinks.data_ptr<float>(), (int)(o.size(0) * o.size(1)), (int)o.size(1), (int)Dv,
                            out.data_ptr(), cur_stream());
  count();
}

void moe_softmax_bias_route(const at::Tensor& logits, c10::optional<at::Tensor> corr, int64_t n_real, at::Tensor w, at::Tensor ids, at::Tensor ident) {
  CHECK_CUDA(logits); CHECK_I32(ids);
  TORCH_CHECK(logits.scalar_type() == at::kFloat && logits.dim() == 2 && logits.stride(1) == 1 && w.scalar_type() == at::kFloat && w.is_contiguous() &&
              ids.is_contiguous() && ident.scalar_type() == at::kFloat && ident.is_contiguous() && w.size(0) == logits.size(0) && ids.sizes() == w.sizes() &&
              ident.numel() == logits.size(0));
  if (corr.has_value()) TORCH_CHECK(corr->scalar_type() == at::kFloat && corr->is_contiguous() && corr->numel() == logits.size(1));
  if (logits.size(0) == 0) return;
  c10::cuda::CUDAGuard g(logits.device());
  sglb::moe_softmax_bias_route(logits.data_ptr<float>(), (int)logits.stride(0), opt_ptr<float>(corr), (int)logits.size(0), (int)logits.size(1),
                               (int)w.size(1), (int)n_real, w.data_ptr<float>(), ids.data_ptr<int>(), ident.data_ptr<float>(), cur_stream());
  count();
}

void moe_identity_shared_combine(at::Tensor y, const at::Tensor& h, c10::optional<at::Tensor> ident, c10::optional<at::Tensor> shared,
                                 c10::optional<at::Tensor> gate) {
  CHECK_CUDA(y);
  TORCH_CHECK(bf16_or_f32(y) && y.dim() == 2 && y.is_contiguous() && h.is_contiguous() && h.scalar_type() == y.scalar_type() && h.numel() == y.numel());
  if (ident.has_value()) TORCH_CHECK(ident->scalar_type() == at::kFloat && ident->is_contiguous() && ident->numel() == y.size(0));
  if (shared.has_value())
    TORCH_CHECK(shared->scalar_type() == y.scalar_type() && shared->is_contiguous() && shared->numel() == y.numel() &&
                (!gate.has_value() || (gate->scalar_type() == at::kFloat && gate->is_contiguous() && gate->numel() == y.size(0))));
  if (y.size(0) == 0 || (!ident.has_value() && !shared.has_value())) return;
  c10::cuda::CUDAGuard g(y.device());
  sglb::moe_identity_shared_combine(y.data_ptr(), h.data_ptr(), opt_ptr<float>(ident), shared.has_value() ? shared->data_ptr() : nullptr,
                                    shared.has_value() && gate.has_value() ? gate->data_ptr<float>() : nullptr, y.scalar_type() == at::kBFloat16, (int)y.size(0),
                                    (int)y.size(1),
                                    cur_stream());
  count();
}

void latent_attention(const at::Tensor& q, const at::Tensor& cache, int64_t rank, const at::Tensor& page_table, const at::Tensor& req_slots,
                      const at::Tensor& seq_lens, c10::optional<at::Tensor> cu_q, int64_t max_q_len, int64_t max_kv_len, int64_t page_size, double scale,
                      int64_t window, c10::optional<at::Tensor> sinks, at::Tensor out, int64_t v_rank) {
  CHECK_CUDA(q); CHECK_I32(page_table); CHECK_I32(req_slots); CHECK_I32(seq_lens);
  if (v_rank <= 0) v_rank = rank;
  TORCH_CHECK(q.scalar_type() == at::kFloat && q.dim() == 3 && q.is_contiguous() && out.scalar_type() == at::kFloat && out.is_contiguous() &&
              v_rank <= rank && out.numel() == q.size(0) * q.size(1) * v_rank && q.size(2) == rank);
  TORCH_CHECK((cache.scalar_type() == at::kFloat || cache.scalar_type() == at::kBFloat16) && cache.dim() == 3 && cache.size(1) == 1 &&
              cache.stride(2) == 1 && cache.size(2) >= rank && page_table.dim() == 2 && page_table.stride(1) == 1);
  const int B = (int)req_slots.size(0);
  if (cu_q.has_value()) { CHECK_I32(*cu_q); TORCH_CHECK(cu_q->numel() == B + 1); } else TORCH_CHECK(q.size(0) == B);
  if (sinks.has_value()) TORCH_CHECK(sinks->scalar_type() == at::kFloat && sinks->is_contiguous() && sinks->numel() == q.size(1));
  if (q.size(0) == 0) return;
  c10::cuda::CUDAGuard g(q.device());
  // decode splits the keys of a request over CTAs: room for up to 32 partial results per (request, head)
  const bool decode = !cu_q.has_value() || max_q_len == 1;
  at::Tensor ws;
  size_t ws_floats = 0;
  if (decode) {
    const int64_t ns = std::max<int64_t>(1, std::min<int64_t>(32, 296 / std::max<int64_t>(1, B)));
    ws_floats = (size_t)(B * ns * q.size(1) * (rank + 2));
    ws = at::empty({(int64_t)ws_floats}, q.options());
  }
  sglb::latent_attention(q.data_ptr<float>(), cache.data_ptr(), cache.scalar_type() == at::kBFloat16, (int)cache.stride(0), (int)rank,
                         page_table.data_ptr<int>(), (int)page_table.stride(0), (int)page_size, req_slots.data_ptr<int>(), seq_lens.data_ptr<int>(),
                         opt_ptr<int>(cu_q), B, (int)max_q_len, (int)max_kv_len, (int)q.size(1), (float)scale, (int)window, opt_ptr<float>(sinks),
                         out.data_ptr<float>(), decode ? ws.data_ptr<float>() : nullptr, ws_floats, (int)v_rank, cur_stream());
  count(decode ? 2 : 1);
}

void latent_prepare(const at::Tensor& x, int64_t q_rank, c10::optional<at::Tensor> q_norm_w, int64_t rank, int64_t rot_dim, const at::Tensor& kv_norm_w,
                    double eps, const at::Tensor& positions, c10::optional<at::Tensor> inv_freq, double mult, at::Tensor cache, const at::Tensor& loc,
                    c10::optional<at::Tensor> cq) {
  CHECK_CUDA(x); CHECK_I32(positions); CHECK_I32(loc);
  const int64_t T = x.size(0);
  TORCH_CHECK(bf16_or_f32(x) && x.dim() == 2 && x.stride(1) == 1 && q_rank >= 0 && rank >= 1 && rot_dim >= 0 && rot_dim % 2 == 0 &&
              x.size(1) >= q_rank + rank + rot_dim);
  TORCH_CHECK(cache.scalar_type() == x.scalar_type() && cache.dim() == 3 && cache.size(1) == 1 && cache.stride(2) == 1 && cache.size(2) >= rank + rot_dim &&
              positions.numel() == T && loc.numel() == T);
  TORCH_CHECK(kv_norm_w.scalar_type() == x.scalar_type() && kv_norm_w.is_contiguous() && kv_norm_w.numel() == rank);
  if (q_rank > 0)
    TORCH_CHECK(q_norm_w.has_value() && cq.has_value() && q_norm_w->scalar_type() == x.scalar_type() && q_norm_w->is_contiguous() &&
                q_norm_w->numel() == q_rank && cq->scalar_type() == x.scalar_type() && cq->is_contiguous() && cq->numel() == T * q_rank);
  if (inv_freq.has_value()) TORCH_CHECK(inv_freq->scalar_type() == at::kFloat && inv_freq->is_contiguous() && 2 * inv_freq->numel() == rot_dim);
  if (T == 0) return;
  c10::cuda::CUDAGuard g(x.device());
  sglb::latent_prepare(x.data_ptr(), (int)x.stride(0), x.scalar_type() == at::kBFloat16, (int)T, (int)q_rank, q_rank > 0 ? q_norm_w->data_ptr() : nullptr,
                       (int)rank, (int)rot_dim, kv_norm_w.data_ptr(), (float)eps, positions.data_ptr<int>(), opt_ptr<float>(inv_freq), (float)mult,
                       cache.data_ptr(), (size_t)cache.stride(0), loc.data_ptr<int>(), q_rank > 0 ? cq->data_ptr() : nullptr, cur_stream());
  count();
}

void latent_query(const at::Tensor& q, const at::Tensor& q_abs, int64_t dim, int64_t rot_dim, const at::Tensor& positions, c10::optional<at::Tensor> inv_freq,
                  double mult, at::Tensor out) {
  CHECK_CUDA(q); CHECK_I32(positions);
  TORCH_CHECK(bf16_or_f32(q) && q.dim() == 3 && q.is_contiguous() && q.size(2) == dim + rot_dim && rot_dim % 2 == 0);
  const int64_t T = q.size(0), H = q.size(1);
  TORCH_CHECK(q_abs.scalar_type() == at::kFloat && q_abs.dim() == 3 && q_abs.is_contiguous() && q_abs.size(0) == H && q_abs.size(1) == T);
  const int64_t R = q_abs.size(2);
  TORCH_CHECK(out.scalar_type() == at::kFloat && out.is_contiguous() && out.numel() == T * H * (R + rot_dim) && positions.numel() == T);
  if (inv_freq.has_value()) TORCH_CHECK(inv_freq->scalar_type() == at::kFloat && inv_freq->is_contiguous() && 2 * inv_freq->numel() == rot_dim);
  if (T == 0) return;
  c10::cuda::CUDAGuard g(q.device());
  sglb::latent_query(q.data_ptr(), q.scalar_type() == at::kBFloat16, q_abs.data_ptr<float>(), (int)T, (int)H, (int)dim, (int)rot_dim, (int)R,
                     positions.data_ptr<int>(), opt_ptr<float>(inv_freq), (float)mult, out.data_ptr<float>(), cur_stream());
  count();
}

void rotate_heads(const at::Tensor& o, const at::Tensor& positions, const at::Tensor& inv_freq, int64_t Dv, bool interleaved, bool inverse,
                  c10::optional<at::Tensor> lse, c10::optional<at::Tensor> sinks, at::Tensor out) {
  CHECK_CUDA(o); CHECK_I32(positions);
  const int64_t T = o.size(0), H = o.size(1);
  TORCH_CHECK(bf16_or_f32(o) && o.dim() == 3 && o.is_contiguous() && Dv >= 2 && Dv % 2 == 0 && Dv <= o.size(2) && out.scalar_type() == o.scalar_type() &&
              out.is_contiguous() && out.numel() == T * H * Dv && positions.numel() == T && out.data_ptr() != o.data_ptr());
  TORCH_CHECK(inv_freq.scalar_type() == at::kFloat && inv_freq.is_contiguous() && 2 * inv_freq.numel() == Dv);
  TORCH_CHECK(lse.has_value() == sinks.has_value());
  if (lse.has_value())
    TORCH_CHECK(lse->scalar_type() == at::kFloat && lse->is_contiguous() && lse->numel() == T * H && sinks->scalar_type() == at::kFloat &&
                sinks->is_contiguous() && sinks->numel() == H);
  if (T == 0) return;
  c10::cuda::CUDAGuard g(o.device());
  sglb::rotate_heads(o.data_ptr(), (int)o.size(2), o.scalar_type() == at::kBFloat16, positions.data_ptr<int>(), inv_freq.data_ptr<float>(), (int)T, (int)H,
                     (int)Dv, interleaved, inverse, opt_ptr<float>(lse), opt_ptr<float>(sinks), out.data_ptr(), cur_stream());
  count();
}

void parallel_add_rmsnorm_f32(at::Tensor residual, c10::optional<at::Tensor> d1, c10::optional<at::Tensor> d2, c10::optional<at::Tensor> d3, const at::Tensor& w1,
                              c10::optional<at::Tensor> w2, at::Tensor out1, c10::optional<at::Tensor> out2, double eps, bool zero_centred) {
  CHECK_CUDA(residual);
  TORCH_CHECK(residual.scalar_type() == at::kFloat && residual.dim() == 2 && residual.is_contiguous() && bf16_or_f32(out1) && out1.is_contiguous() &&
              out1.numel() == residual.numel() && w1.scalar_type() == out1.scalar_type() && w1.is_contiguous() && w1.numel() == residual.size(1));
  TORCH_CHECK(w2.has_value() == out2.has_value());
  if (w2.has_value())
    TORCH_CHECK(w2->scalar_type() == out1.scalar_type() && w2->is_contiguous() && w2->numel() == residual.size(1) && out2->scalar_type() == out1.scalar_type() &&
                out2->is_contiguous() && out2->numel() == residual.numel());
  TORCH_CHECK(d1.has_value() || !d2.has_value());
  bool dbf = out1.scalar_type() == at::kBFloat16;
  if (d1.has_value()) {
    TORCH_CHECK(bf16_or_f32(*d1) && d1->is_contiguous() && d1->numel() == residual.numel());
    dbf = d1->scalar_type() == at::kBFloat16;
  }
  if (d2.has_value()) TORCH_CHECK(d2->scalar_type() == d1->scalar_type() && d2->is_contiguous() && d2->numel() == residual.numel());
  if (d3.has_value()) TORCH_CHECK(d3->scalar_type() == at::kFloat && d3->is_contiguous() && d3->numel() == residual.numel());
  if (residual.size(0) == 0) return;
  c10::cuda::CUDAGuard g(residual.device());
  sglb::parallel_add_rmsnorm_f32(residual.data_ptr<float>(), d1.has_value() ? d1->data_ptr() : nullptr, d2.has_value() ? d2->data_ptr() : nullptr, dbf,
                                 opt_ptr<float>(d3), w1.data_ptr(), w2.has_value() ? w2->data_ptr() : nullptr, out1.data_ptr(),
                                 out2.has_value() ? out2->data_ptr() : nullptr, out1.scalar_type() == at::kBFloat16, (int)residual.size(0),
                                 (int)residual.size(1), (float)eps, zero_centred, cur_stream());
  count();
}

void mlstm_prepare(const at::Tensor& proj, const at::Tensor& gates_raw, int64_t H, int64_t D, int64_t Dv, double cap, at::Tensor mstate,
                   const at::Tensor& req_slots, const at::Tensor& seq_lens, c10::optional<at::Tensor> cu_q, at::Tensor u, at::Tensor gates) {
  CHECK_CUDA(proj); CHECK_I32(req_slots); CHECK_I32(seq_lens);
  const int64_t T = proj.size(0);
  auto f32c = [](const at::Tensor& t) { return t.scalar_type() == at::kFloat && t.is_contiguous(); };
  TORCH_CHECK(bf16_or_f32(proj) && proj.dim() == 2 && proj.stride(1) == 1 && proj.size(1) >= 2 * H * D + H * Dv);
  TORCH_CHECK(f32c(gates_raw) && gates_raw.numel() == T * 2 * H && f32c(mstate) && mstate.dim() == 2 && mstate.size(1) == H && f32c(u) &&
              u.numel() == T * (H * (Dv + 1) + 2 * H * D) && f32c(gates) && gates.numel() == T * H * 3);
  const int B = (int)req_slots.size(0);
  if (cu_q.has_value()) { CHECK_I32(*cu_q); TORCH_CHECK(cu_q->numel() == B + 1); } else TORCH_CHECK(T == B);
  if (T == 0) return;
  c10::cuda::CUDAGuard g(proj.device());
  sglb::mlstm_prepare(proj.data_ptr(), (int)proj.stride(0), proj.scalar_type() == at::kBFloat16, gates_raw.data_ptr<float>(), (int)T, B, (int)H, (int)D,
                      (int)Dv, (float)cap, mstate.data_ptr<float>(), req_slots.data_ptr<int>(), seq_lens.data_ptr<int>(), opt_ptr<int>(cu_q),
                      u.data_ptr<float>(), gates.data_ptr<float>(), cur_stream());
  count();
}

void mlstm_readout(const at::Tensor& y, const at::Tensor& gates, int64_t H, int64_t Dv, const at::Tensor& norm_w, double eps, c10::optional<at::Tensor> gate,
                   at::Tensor out) {
  CHECK_CUDA(y);
  const int64_t T = y.size(0);
  TORCH_CHECK(y.scalar_type() == at::kFloat && y.is_contiguous() && y.numel() == T * H * (Dv + 1) && gates.scalar_type() == at::kFloat &&
              gates.is_contiguous() && gates.numel() == T * H * 3);
  TORCH_CHECK(bf16_or_f32(out) && out.is_contiguous() && out.numel() == T * H * Dv && norm_w.scalar_type() == out.scalar_type() && norm_w.is_contiguous() &&
              norm_w.numel() == H * Dv);
  if (gate.has_value())
    TORCH_CHECK(gate->scalar_type() == out.scalar_type() && gate->dim() == 2 && gate->stride(1) == 1 && gate->size(0) == T && gate->size(1) == H * Dv);
  if (T == 0) return;
  c10::cuda::CUDAGuard g(y.device());
  sglb::mlstm_readout(y.data_ptr<float>(), gates.data_ptr<float>(), (int)T, (int)H, (int)Dv, norm_w.data_ptr(), (float)eps,
                      gate.has_value() ? gate->data_ptr() : nullptr, gate.has_value() ? (int)gate->stride(0) : 0, out.data_ptr(),
                      out.scalar_type() == at::kBFloat16, cur_stream());
  count();
}

void causal_softmax(const at::Tensor& scores, int64_t tq, int64_t first, double scale, at::Tensor out) {
  CHECK_CUDA(scores);
  TORCH_CHECK(scores.scalar_type() == at::kFloat && scores.dim() == 2 && scores.is_contiguous() && bf16_or_f32(out) && out.is_contiguous() &&
              out.numel() == scores.numel() && tq >= 1 && scores.size(0) % tq == 0 && first >= 0);
  if (scores.numel() == 0) return;
  c10::cuda::CUDAGuard g(scores.device());
  sglb::causal_softmax(scores.data_ptr<float>(), out.data_ptr(), out.scalar_type() == at::kBFloat16, (int)scores.size(0), (int)tq, (int)scores.size(1), (int)first,
                       (float)scale, cur_stream());
  count();
}

// bench tool: per-role cycle accounting of the decode attention kernel into buf [ctas * 30] (int64); an empty tensor turns it off
void attn_decode_prof(const at::Tensor& buf) {
  if (buf.numel() == 0) { sglb::attn_decode_set_prof(nullptr); return; }
  CHECK_CUDA(buf); TORCH_CHECK(buf.scalar_type() == at::kLong && buf.is_contiguous() && buf.numel() >= 148 * 40);
  sglb::attn_decode_set_prof((long long*)buf.data_ptr<int64_t>());
}

// out[M, N(/2 for silu_mul)] = a[M, K] @ w[N, K]^T (+bias | silu*mul)
void gemm(const at::Tensor& a, const at::Tensor& w, at::Tensor out, c10::optional<at::Tensor> bias, int64_t epilogue,
          int64_t bn) {
  CHECK_CUDA(a); CHECK_BF16(a); CHECK_BF16(w); CHECK_BF16(out); CHECK_LAST_CONTIG(a); CHECK_LAST_CONTIG(w); CHECK_LAST_CONTIG(out);
  TORCH_CHECK(a.dim() == 2 && w.dim() == 2 && out.dim() == 2 && a.size(1) == w.size(1));
  TORCH_CHECK((reinterpret_cast<uintptr_t>(a.data_ptr()) & 15) == 0 && (reinterpret_cast<uintptr_t>(w.data_ptr()) & 15) == 0 &&
              (reinterpret_cast<uintptr_t>(out.data_ptr()) & 15) == 0, "gemm operands must be 16-byte aligned");
  c10::cuda::CUDAGuard g(a.device());
  sglb::gemm_bf16_tc(a.data_ptr(), w.data_ptr(), out.data_ptr(), bias.has_value() ? bias->data_ptr() : nullptr,
                     (int)a.size(0), (int)w.size(0), (int)a.size(1), (int)a.stride(0), (int)w.stride(0), (int)out.stride(0),
                     (int)epilogue, (int)bn, num_sms(), cur_stream());
  count();
}
int64_t gemm_pick_bn(int64_t M, int64_t N, int64_t K) { return sglb::gemm_pick_bn((int)M, (int)N, (int)K, num_sms()); }

void sample(const at::Tensor& logits, const at::Tensor& temperature, const at::Tensor& top_k, const at::Tensor& top_p,
            const at::Tensor& min_p, c10::optional<at::Tensor> seeds, c10::optional<at::Tensor> out_slots,
            c10::optional<at::Tensor> next_token_buf, at::Tensor out_tokens, c10::optional<at::Tensor> out_logprobs,
            int64_t global_seed, c10::optional<at::Tensor> step_ptr, int64_t step) {
  CHECK_CUDA(logits); CHECK_LAST_CONTIG(logits); CHECK_I32(top_k); CHECK_I32(out_tokens);
  TORCH_CHECK(logits.dim() == 2);
  const bool bf16 = logits.scalar_type() == at::kBFloat16;
  TORCH_CHECK(bf16 || logits.scalar_type() == at::kFloat, "logits must be bf16 or fp32");
  if (seeds.has_value())
    TORCH_CHECK(seeds->dim() == 2 && seeds->size(0) == logits.size(0) && seeds->size(1) == 2 && seeds->is_contiguous() &&
                seeds->scalar_type() == at::kLong, "seeds must be int64 [B, 2] = (seed, output position | -1)");
  c10::cuda::CUDAGuard g(logits.device());
  sglb::sample(logits.data_ptr(), bf16, (int)logits.size(0), (int)logits.size(1), (int)logits.stride(0),
               temperature.data_ptr<float>(), top_k.data_ptr<int>(), top_p.data_ptr<float>(), min_p.data_ptr<float>(),
               seeds.has_value() ? (const long long*)seeds->data_ptr<int64_t>() : nullptr, opt_ptr<int>(out_slots),
               opt_mptr<int>(next_token_buf), out_tokens.data_ptr<int>(), opt_mptr<float>(out_logprobs),
               (unsigned long long)global_seed, step_ptr.has_value() ? (const long long*)step_ptr->data_ptr<int64_t>() : nullptr,
               (long long)step, cur_stream());
  count();
}

void greedy_shard(const at::Tensor& logits, int64_t v_valid, int64_t v_offset, int64_t rank, int64_t tp, at::Tensor buf) {
  CHECK_CUDA(logits); CHECK_LAST_CONTIG(logits); CHECK_CUDA(buf);
  TORCH_CHECK(logits.dim() == 2 && buf.dim() == 3 && buf.size(0) == tp && buf.size(2) == 4 && buf.is_contiguous() &&
              buf.scalar_type() == at::kBFloat16 && buf.size(1) >= logits.size(0), "greedy_shard: buf must be bf16 [tp, Bpad >= B, 4]");
  const bool bf16 = logits.scalar_type() == at::kBFloat16;
  TORCH_CHECK(bf16 || logits.scalar_type() == at::kFloat, "logits must be bf16 or fp32");
  TORCH_CHECK(v_valid >= 0 && v_valid <= logits.size(1) && v_offset + v_valid < (1 << 24) && rank >= 0 && rank < tp);
  c10::cuda::CUDAGuard g(logits.device());
  sglb::greedy_shard(logits.data_ptr(), bf16, (int)logits.size(0), (int)logits.stride(0), (int)v_valid, (int)v_offset, (int)rank, (int)tp,
                     (int)buf.size(1), buf.data_ptr(), cur_stream());
  count();
}
void greedy_merge(const at::Tensor& buf, int64_t B, c10::optional<at::Tensor> out_slots, c10::optional<at::Tensor> next_token_buf,
                  at::Tensor out_tokens) {
  CHECK_CUDA(buf); CHECK_I32(out_tokens);
  TORCH_CHECK(buf.dim() == 3 && buf.size(2) == 4 && buf.is_contiguous() && buf.scalar_type() == at::kBFloat16 && B <= buf.size(1) &&
              out_tokens.numel() >= B);
  c10::cuda::CUDAGuard g(buf.device());
  sglb::greedy_merge(buf.data_ptr(), (int)buf.size(0), (int)buf.size(1), (int)B, opt_ptr<int>(out_slots), opt_mptr<int>(next_token_buf),
                     out_tokens.data_ptr<int>(), cur_stream());
  count();
}

void apply_token_bitmask(at::Tensor logits, const at::Tensor& bitmask, c10::optional<at::Tensor> row_idx) {
  CHECK_CUDA(logits); CHECK_I32(bitmask); TORCH_CHECK(bitmask.is_contiguous() && logits.dim() == 2);
  const bool bf16 = logits.scalar_type() == at::kBFloat16;
  c10::cuda::CUDAGuard g(logits.device());
  sglb::apply_token_bitmask(logits.data_ptr(), bf16, bitmask.data_ptr<int>(), opt_ptr<int>(row_idx), (int)bitmask.size(0),
                            (int)logits.size(1), (int)logits.stride(0), cur_stream());
  count();
}

void apply_penalties(at::Tensor logits, const at::Tensor& counts, c10::optional<at::Tensor> prompt_mask, const at::Tensor& freq,
                     const at::Tensor& pres, const at::Tensor& rep) {
  CHECK_CUDA(logits); TORCH_CHECK(logits.scalar_type() == at::kFloat && logits.dim() == 2); CHECK_I32(counts);
  c10::cuda::CUDAGuard g(logits.device());
  sglb::apply_penalties(logits.data_ptr<float>(), counts.data_ptr<int>(),
                        prompt_mask.has_value() ? prompt_mask->data_ptr<uint8_t>() : nullptr, freq.data_ptr<float>(),
                        pres.data_ptr<float>(), rep.data_ptr<float>(), (int)logits.size(0), (int)logits.size(1),
                        (int)logits.stride(0), cur_stream());
  count();
}

void bump_counts(at::Tensor counts, const at::Tensor& tokens) {
  CHECK_CUDA(counts); CHECK_I32(counts); CHECK_I32(tokens);
  c10::cuda::CUDAGuard g(counts.device());
  sglb::bump_counts(counts.data_ptr<int>(), tokens.data_ptr<int>(), (int)tokens.size(0), (int)counts.size(1), cur_stream());
  count();
}

void nvl_allreduce(const at::Tensor& buf_ptrs, const at::Tensor& flag_ptrs, int64_t mc_ptr, int64_t slot_off, int64_t rank,
                   int64_t world, at::Tensor out, at::Tensor epoch, at::Tensor done, int64_t channel, int64_t algo) {
  CHECK_CUDA(out); CHECK_BF16(out); TORCH_CHECK(out.is_contiguous() && !buf_ptrs.is_cuda() && !flag_ptrs.is_cuda());
  c10::cuda::CUDAGuard g(out.device());
  sglb::nvl_allreduce(buf_ptrs.data_ptr<int64_t>(), flag_ptrs.data_ptr<int64_t>(), mc_ptr, slot_off, (int)rank, (int)world,
                      out.data_ptr(), (int)out.numel(), reinterpret_cast<uint32_t*>(epoch.data_ptr<int>()),
                      reinterpret_cast<uint32_t*>(done.data_ptr<int>()), (int)channel, (int)algo, num_sms(), cur_stream());
  count();
}

void nvl_ar_add_rmsnorm(const at::Tensor& buf_ptrs, const at::Tensor& flag_ptrs, int64_t mc_ptr, int64_t slot_off, int64_t rank,
                        int64_t world, c10::optional<at::Tensor> residual, const at::Tensor& w, at::Tensor out, double eps, bool gemma,
                        at::Tensor epoch, at::Tensor done, int64_t channel) {
  CHECK_CUDA(out); CHECK_BF16(out); CHECK_BF16(w); TORCH_CHECK(out.is_contiguous() && out.dim() == 2);
  if (residual.has_value()) TORCH_CHECK(residual->is_contiguous());
  c10::cuda::CUDAGuard g(out.device());
  sglb::nvl_ar_add_rmsnorm(buf_ptrs.data_ptr<int64_t>(), flag_ptrs.data_ptr<int64_t>(), mc_ptr, slot_off, (int)rank, (int)world,
                           residual.has_value() ? residual->data_ptr() : nullptr, w.data_ptr(), out.data_ptr(), (int)out.size(0),
                           (int)out.size(1), (float)eps, gemma, reinterpret_cast<uint32_t*>(epoch.data_ptr<int>()),
                           reinterpret_cast<uint32_t*>(done.data_ptr<int>()), (int)channel, num_sms(), cur_stream());
  count();
}

// large-T variant: reduce-scatter + residual add + RMSNorm + all-gather; the normalised rows land in the result region (slot_off + out_off)
// of EVERY rank's arena, the residual stream stays row-sharded (row t belongs to rank t % world)
void nvl_rs_add_rmsnorm_ag(const at::Tensor& buf_ptrs, const at::Tensor& flag_ptrs, int64_t mc_ptr, int64_t slot_off, int64_t out_off, int64_t rank,
                           int64_t world, c10::optional<at::Tensor> residual, const at::Tensor& w, int64_t T, int64_t H, double eps, bool gemma,
                           at::Tensor epoch, at::Tensor done, int64_t channel) {
  CHECK_CUDA(w); CHECK_BF16(w);
  if (residual.has_value()) TORCH_CHECK(residual->is_contiguous() && residual->scalar_type() == at::kBFloat16 && residual->numel() == T * H);
  c10::cuda::CUDAGuard g(w.device());
  sglb::nvl_rs_add_rmsnorm_ag(buf_ptrs.data_ptr<int64_t>(), flag_ptrs.data_ptr<int64_t>(), mc_ptr, slot_off, out_off, (int)rank, (int)world,
                              residual.has_value() ? residual->data_ptr() : nullptr, w.data_ptr(), (int)T, (int)H, (float)eps, gemma,
                              reinterpret_cast<uint32_t*>(epoch.data_ptr<int>()), reinterpret_cast<uint32_t*>(done.data_ptr<int>()), (int)channel,
                              num_sms(), cur_stream());
  count();
}

// fused GEMM + all-reduce producer: a[M,K] @ w[N,K]^T pushed into slot [rank] of every peer's arena
void gemm_push(const at::Tensor& a, const at::Tensor& w, const at::Tensor& peer_slot_ptrs, const at::Tensor& peer_flag_ptrs,
               int64_t rank, int64_t world, at::Tensor epoch, at::Tensor done, int64_t bn) {
  CHECK_CUDA(a); CHECK_BF16(a); CHECK_BF16(w); CHECK_LAST_CONTIG(a); CHECK_LAST_CONTIG(w);
  TORCH_CHECK(a.dim() == 2 && w.dim() == 2 && a.size(1) == w.size(1) && !peer_slot_ptrs.is_cuda() && !peer_flag_ptrs.is_cuda());
  c10::cuda::CUDAGuard g(a.device());
  sglb::gemm_bf16_tc_push(a.data_ptr(), w.data_ptr(), (int)a.size(0), (int)w.size(0), (int)a.size(1), (int)a.stride(0), (int)w.stride(0),
                          peer_slot_ptrs.data_ptr<int64_t>(), peer_flag_ptrs.data_ptr<int64_t>(), (int)rank, (int)world,
                          reinterpret_cast<const uint32_t*>(epoch.data_ptr<int>()), reinterpret_cast<uint32_t*>(done.data_ptr<int>()),
                          (int)bn, num_sms(), cur_stream());
  count();
}

void nvl_local_reduce_add_rmsnorm(const at::Tensor& slot, int64_t flags_ptr, c10::optional<at::Tensor> residual, const at::Tensor& w,
                                  at::Tensor out, int64_t world, int64_t nslabs, double eps, bool gemma, at::Tensor epoch, at::Tensor done) {
  CHECK_CUDA(out); CHECK_BF16(out); CHECK_BF16(w); CHECK_BF16(slot); TORCH_CHECK(out.is_contiguous() && out.dim() == 2);
  c10::cuda::CUDAGuard g(out.device());
  sglb::nvl_local_reduce_add_rmsnorm(slot.data_ptr(), reinterpret_cast<uint32_t*>(flags_ptr),
                                     residual.has_value() ? residual->data_ptr() : nullptr, w.data_ptr(), out.data_ptr(),
                                     (int)out.size(0), (int)out.size(1), (int)world, (int)nslabs, (float)eps, gemma,
                                     reinterpret_cast<uint32_t*>(epoch.data_ptr<int>()), reinterpret_cast<uint32_t*>(done.data_ptr<int>()),
                                     num_sms(), cur_stream());
  count();
}

// HiCache page mover: dev_buf [planes, slots, ...] <-> pinned host_buf; page indices as int32 DEVICE tensors; strides in bytes
void kv_transfer_pages(at::Tensor dev_buf, at::Tensor host_buf, const at::Tensor& dev_pages, const at::Tensor& host_pages, int64_t planes,
                       int64_t dev_plane_stride, int64_t host_plane_stride, int64_t host_page_stride, int64_t chunk_bytes, bool to_host) {
  CHECK_CUDA(dev_buf); CHECK_I32(dev_pages); CHECK_I32(host_pages);
  TORCH_CHECK(!host_buf.is_cuda() && host_buf.is_pinned(), "kv_transfer_pages: the host pool must be pinned memory");
  TORCH_CHECK(dev_pages.is_cuda() && host_pages.is_cuda() && dev_pages.numel() == host_pages.numel());
  c10::cuda::CUDAGuard g(dev_buf.device());
  void* hptr = nullptr;
  TORCH_CHECK(cudaHostGetDevicePointer(&hptr, host_buf.data_ptr(), 0) == cudaSuccess, "kv_transfer_pages: host pool is not device-mapped");
  sglb::kv_transfer_pages(dev_buf.data_ptr(), hptr, dev_pages.data_ptr<int>(), host_pages.data_ptr<int>(), (int)dev_pages.numel(), (int)planes,
                          dev_plane_stride, host_plane_stride, host_page_stride, (int)chunk_bytes, to_host, cur_stream());
  count();
}

// y[perm[i], :] += B[slot] (A[slot] x[perm[i], :])  for the tokens listed in the tile table (see kernels/lora.cu)
void lora_sgmv(const at::Tensor& x, const at::Tensor& a_pool, const at::Tensor& b_pool, const at::Tensor& tile_slot,
               const at::Tensor& tile_start, const at::Tensor& tile_cnt, const at::Tensor& perm, at::Tensor h, at::Tensor y, int64_t b1, int64_t b2) {
  CHECK_CUDA(x); CHECK_BF16(x); CHECK_BF16(y); CHECK_BF16(a_pool); CHECK_BF16(b_pool); CHECK_LAST_CONTIG(x); CHECK_LAST_CONTIG(y);
  CHECK_I32(tile_slot); CHECK_I32(tile_start); CHECK_I32(tile_cnt); CHECK_I32(perm);
  TORCH_CHECK(a_pool.dim() == 4 && b_pool.dim() == 3 && a_pool.is_contiguous() && b_pool.is_contiguous() && x.dim() == 2 && y.dim() == 2);
  TORCH_CHECK(h.scalar_type() == at::kFloat && h.is_contiguous());
  const int n_sub = (int)a_pool.size(1), R = (int)a_pool.size(2), K = (int)a_pool.size(3), N = (int)b_pool.size(1);
  TORCH_CHECK(x.size(1) == K && y.size(1) == N && b_pool.size(2) == R && b_pool.size(0) == a_pool.size(0));
  TORCH_CHECK(h.numel() >= perm.numel() * n_sub * R, "lora_sgmv: scratch too small");
  c10::cuda::CUDAGuard g(x.device());
  sglb::lora_sgmv(x.data_ptr(), (int)x.stride(0), a_pool.data_ptr(), b_pool.data_ptr(), R, n_sub, K, N, (int)b1, (int)b2, tile_slot.data_ptr<int>(),
                  tile_start.data_ptr<int>(), tile_cnt.data_ptr<int>(), perm.data_ptr<int>(), (int)tile_slot.numel(), h.data_ptr<float>(),
                  y.data_ptr(), (int)y.stride(0), cur_stream());
  count(2);
}

// persistent stream-K decode GEMM (M <= 256): out[M, N] = a[M, K] @ w[N, K]^T (+bias) ; epilogue 4: w = [gate; up], out[M, N/2] = silu(g) * u
void gemm_streamk(const at::Tensor& a, const at::Tensor& w, at::Tensor out, c10::optional<at::Tensor> bias, int64_t epilogue) {
  CHECK_CUDA(a); CHECK_BF16(a); CHECK_BF16(w); CHECK_BF16(out); CHECK_LAST_CONTIG(a); CHECK_LAST_CONTIG(w); CHECK_LAST_CONTIG(out);
  TORCH_CHECK(a.dim() == 2 && w.dim() == 2 && out.dim() == 2 && a.size(1) == w.size(1));
  const int M = (int)a.size(0), K = (int)a.size(1);
  const int N = epilogue == 4 ? (int)w.size(0) / 2 : (int)w.size(0);
  TORCH_CHECK(out.size(1) == N && out.size(0) == M, "gemm_streamk: bad output shape");
  TORCH_CHECK((reinterpret_cast<uintptr_t>(a.data_ptr()) & 15) == 0 && (reinterpret_cast<uintptr_t>(out.data_ptr()) & 15) == 0 &&
              (reinterpret_cast<uintptr_t>(w.data_ptr()) & 15) == 0, "gemm_streamk: operands must be 16-byte aligned (TMA)");
  if (epilogue == 1) TORCH_CHECK(bias.has_value() && bias->numel() == N);
  c10::cuda::CUDAGuard g(a.device());
  sglb::gemm_bf16_streamk(a.data_ptr(), w.data_ptr(), out.data_ptr(), bias.has_value() ? bias->data_ptr() : nullptr, M, N, K,
                          (int)a.stride(0), (int)w.stride(0), (int)out.stride(0), (int)epilogue, num_sms(), cur_stream());
  count();
}

// decode-shape GEMM (M <= 256): out is [M, N] (splits == 1) or a slab workspace [splits, M, N] that the consumer sums
int64_t gemm_skinny_splits(int64_t M, int64_t N, int64_t K, int64_t max_splits) {
  return sglb::gemm_skinny_splits((int)M, (int)N, (int)K, (int)max_splits, num_sms());
}
int64_t gemm_skinny_norm_splits(int64_t K, int64_t s) { return sglb::gemm_skinny_norm_splits((int)K, (int)s); }
void gemm_skinny(const at::Tensor& a, const at::Tensor& w, at::Tensor out, c10::optional<at::Tensor> bias, int64_t epilogue,
                 int64_t splits) {
  CHECK_CUDA(a); CHECK_BF16(a); CHECK_BF16(w); CHECK_BF16(out); CHECK_LAST_CONTIG(a); CHECK_LAST_CONTIG(w); CHECK_LAST_CONTIG(out);
  TORCH_CHECK(a.dim() == 2 && w.dim() == 2 && a.size(1) == w.size(1));
  const int M = (int)a.size(0), K = (int)a.size(1);
  const int N = epilogue == 4 ? (int)w.size(0) / 2 : (int)w.size(0);
  TORCH_CHECK(splits >= 1 && (splits == 1 ? out.dim() == 2 : (out.dim() == 3 && out.size(0) >= splits && out.is_contiguous())));
  TORCH_CHECK(out.size(-1) == N && out.size(-2) == M, "gemm_skinny: bad output shape");
  c10::cuda::CUDAGuard g(a.device());
  sglb::gemm_bf16_skinny(a.data_ptr(), w.data_ptr(), out.data_ptr(), bias.has_value() ? bias->data_ptr() : nullptr, M, N, K,
                         (int)a.stride(0), (int)w.stride(0), (int)out.stride(-2), (int)epilogue, (int)splits,
                         splits > 1 ? (long long)out.stride(0) : 0, cur_stream());
  count();
}
void gemm_skinny_push(const at::Tensor& a, const at::Tensor& w, int64_t splits, const at::Tensor& peer_slot_ptrs,
                      const at::Tensor& peer_flag_ptrs, int64_t rank, int64_t world, at::Tensor epoch, at::Tensor done) {
  CHECK_CUDA(a); CHECK_BF16(a); CHECK_BF16(w); CHECK_LAST_CONTIG(a); CHECK_LAST_CONTIG(w);
  TORCH_CHECK(a.dim() == 2 && w.dim() == 2 && a.size(1) == w.size(1) && !peer_slot_ptrs.is_cuda() && !peer_flag_ptrs.is_cuda());
  c10::cuda::CUDAGuard g(a.device());
  sglb::gemm_bf16_skinny_push(a.data_ptr(), w.data_ptr(), (int)a.size(0), (int)w.size(0), (int)a.size(1), (int)a.stride(0),
                              (int)w.stride(0), (int)splits, peer_slot_ptrs.data_ptr<int64_t>(), peer_flag_ptrs.data_ptr<int64_t>(),
                              (int)rank, (int)world, reinterpret_cast<const uint32_t*>(epoch.data_ptr<int>()),
                              reinterpret_cast<uint32_t*>(done.data_ptr<int>()), cur_stream());
  count();
}
// out = rmsnorm(residual += sum_s slabs[s]) — the consumer of a LOCAL split-K GEMM (no flags, stream order is enough)
void slab_reduce_add_rmsnorm(const at::Tensor& slabs, c10::optional<at::Tensor> residual, const at::Tensor& w, at::Tensor out,
                             double eps, bool gemma) {
  CHECK_CUDA(out); CHECK_BF16(out); CHECK_BF16(w); CHECK_BF16(slabs);
  TORCH_CHECK(slabs.dim() == 3 && slabs.is_contiguous() && out.is_contiguous() && out.dim() == 2);
  TORCH_CHECK(slabs.size(1) == out.size(0) && slabs.size(2) == out.size(1) && slabs.size(0) <= 64, "slab_reduce: bad shapes");
  c10::cuda::CUDAGuard g(out.device());
  sglb::nvl_local_reduce_add_rmsnorm(slabs.data_ptr(), nullptr, residual.has_value() ? residual->data_ptr() : nullptr, w.data_ptr(),
                                     out.data_ptr(), (int)out.size(0), (int)out.size(1), 0, (int)slabs.size(0), (float)eps, gemma, nullptr,
                                     nullptr, num_sms(), cur_stream());
  count();
}

void per_token_group_quant_fp8(const at::Tensor& x, at::Tensor q, at::Tensor scales, int64_t group, bool ue8m0) {
  CHECK_CUDA(x); CHECK_BF16(x); CHECK_LAST_CONTIG(x);
  TORCH_CHECK(group == 128, "fp8 activation quant: group size must be 128");
  TORCH_CHECK(x.dim() == 2 && q.is_contiguous() && q.element_size() == 1 && scales.scalar_type() == at::kFloat && scales.is_contiguous());
  c10::cuda::CUDAGuard g(x.device());
  sglb::per_token_group_quant_fp8(x.data_ptr(), q.data_ptr(), scales.data_ptr<float>(), (int)x.size(0), (int)x.size(1), (int)x.stride(0),
                                  ue8m0, cur_stream());
  count();
}

// out[M,N] bf16 = block-scaled (xq[M,K] e4m3, xs[M,K/128]) @ (wq[N,K] e4m3, ws[N/128,K/128])^T
void gemm_fp8_block(const at::Tensor& xq, const at::Tensor& xs, const at::Tensor& wq, const at::Tensor& ws, at::Tensor out) {
  CHECK_CUDA(xq); CHECK_BF16(out); CHECK_LAST_CONTIG(xq); CHECK_LAST_CONTIG(wq); CHECK_LAST_CONTIG(out);
  TORCH_CHECK(xq.element_size() == 1 && wq.element_size() == 1 && xq.dim() == 2 && wq.dim() == 2 && xq.size(1) == wq.size(1));
  TORCH_CHECK(xs.scalar_type() == at::kFloat && ws.scalar_type() == at::kFloat && xs.stride(-1) == 1 && ws.stride(-1) == 1);
  const int64_t kg = (xq.size(1) + 127) / 128;
  TORCH_CHECK(xs.size(0) == xq.size(0) && xs.size(1) == kg && ws.size(0) == (wq.size(0) + 127) / 128 && ws.size(1) == kg,
              "fp8 block gemm: scale shapes must be [M, K/128] and [N/128, K/128]");
  c10::cuda::CUDAGuard g(xq.device());
  sglb::gemm_fp8_block(xq.data_ptr(), xs.data_ptr<float>(), wq.data_ptr(), ws.data_ptr<float>(), out.data_ptr(), (int)xq.size(0),
                       (int)wq.size(0), (int)xq.size(1), (int)xq.stride(0), (int)wq.stride(0), (int)out.stride(0), (int)xs.stride(0),
                       (int)ws.stride(0), num_sms(), cur_stream());
  count();
}

void moe_topk_softmax(const at::Tensor& logits, at::Tensor out_w, at::Tensor out_ids, bool renorm) {
  CHECK_CUDA(logits); CHECK_LAST_CONTIG(logits); CHECK_I32(out_ids);
  TORCH_CHECK(logits.dim() == 2 && out_w.scalar_type() == at::kFloat && out_w.is_contiguous() && out_ids.is_contiguous());
  const bool bf16 = logits.scalar_type() == at::kBFloat16;
  TORCH_CHECK(bf16 || logits.scalar_type() == at::kFloat, "router logits must be bf16 or fp32");
  c10::cuda::CUDAGuard g(logits.device());
  sglb::moe_topk_softmax(logits.data_ptr(), bf16, out_w.data_ptr<float>(), out_ids.data_ptr<int>(), (int)logits.size(0),
                         (int)logits.size(1), (int)out_ids.size(1), (int)logits.stride(0), renorm, cur_stream());
  count();
}

// Whole expert MLP block on expert-sorted rows: align -> gather -> grouped GEMM (silu(gate)*up fused) -> grouped GEMM (routing
// weight fused) -> combine.  With peer pointers the combine pushes its result into every peer's NVLink arena instead of `out`.
void moe_grouped_mlp_impl(const at::Tensor& x, const at::Tensor& w13, const at::Tensor& w2, const at::Tensor& topk_w,
                          const at::Tensor& topk_ids, c10::optional<at::Tensor> out, int64_t expert_offset,
                          const int64_t* peer_slots, const int64_t* peer_flags, int rank, int world, const uint32_t* epoch,
                          uint32_t* done, int act = 0, float act_limit = 0.f, float act_alpha = 0.f) {
  CHECK_CUDA(x); CHECK_BF16(x); CHECK_BF16(w13); CHECK_BF16(w2); CHECK_I32(topk_ids); CHECK_LAST_CONTIG(x);
  TORCH_CHECK(x.dim() == 2 && w13.dim() == 3 && w2.dim() == 3 && w13.is_contiguous() && w2.is_contiguous());
  TORCH_CHECK(topk_w.scalar_type() == at::kFloat && topk_w.is_contiguous() && topk_ids.is_contiguous());
  const int T = (int)x.size(0), H = (int)x.size(1), K = (int)topk_ids.size(1), E = (int)w13.size(0), I = (int)w2.size(2);
  TORCH_CHECK(w13.size(1) == 2 * I && w13.size(2) == H && w2.size(1) == H && w2.size(0) == E);
  if (T == 0) return;
  c10::cuda::CUDAGuard g(x.device());
  auto stream = cur_stream();
  const int pairs = T * K;
  const int max_tiles = (pairs + 127) / 128 + E;
  const int cap = max_tiles * 128;
  auto i32 = x.options().dtype(at::kInt);
  auto meta = at::empty({cap + pairs + max_tiles + 1}, i32);
  int* sorted_row = meta.data_ptr<int>();
  int* inv_pos = sorted_row + cap;
  int* tile_expert = inv_pos + pairs;
  int* num_tiles = tile_expert + max_tiles;
  auto row_w = at::empty({cap}, x.options().dtype(at::kFloat));
  sglb::moe_align(topk_ids.data_ptr<int>(), topk_w.data_ptr<float>(), pairs, E, (int)expert_offset, sorted_row, inv_pos,
                  row_w.data_ptr<float>(), tile_expert, num_tiles, max_tiles, stream);
  auto xs = at::empty({cap, H}, x.options());
  sglb::moe_gather(x.data_ptr(), sorted_row, num_tiles, xs.data_ptr(), H, (int)x.stride(0), K, cap, num_sms(), stream);
  auto h = at::empty({cap, I}, x.options());
  if (act == 0) {
    sglb::gemm_bf16_tc_grouped(xs.data_ptr(), w13.data_ptr(), h.data_ptr(), nullptr, cap, I, H, H, I, E, tile_expert, num_tiles, true,
                               num_sms(), stream);
  } else {
    // clamped GLU: the gate|up block comes out of the grouped GEMM whole, the activation is its own (vectorised) pass
    auto h2 = at::empty({cap, 2 * I}, x.options());
    sglb::gemm_bf16_tc_grouped(xs.data_ptr(), w13.data_ptr(), h2.data_ptr(), nullptr, cap, 2 * I, H, H, 2 * I, E, tile_expert, num_tiles, false,
                               num_sms(), stream);
    sglb::clamped_glu(h2.data_ptr(), h.data_ptr(), true, cap, I, act_limit, act_alpha, stream);
    count();
  }
  auto& ys = xs;   // the gathered inputs are dead once the first GEMM has run (same stream): reuse as the [cap, H] output
  sglb::gemm_bf16_tc_grouped(h.data_ptr(), w2.data_ptr(), ys.data_ptr(), row_w.data_ptr<float>(), cap, H, I, I, H, E, tile_expert,
                             num_tiles, false, num_sms(), stream);
  if (peer_slots) {
    sglb::moe_combine_push(ys.data_ptr(), inv_pos, nullptr, T, H, K, peer_slots, peer_flags, rank, world, epoch, done, num_sms(), stream);
  } else {
    TORCH_CHECK(out.has_value() && out->is_contiguous());
    sglb::moe_combine(ys.data_ptr(), inv_pos, nullptr, out->data_ptr(), T, H, K, num_sms(), stream);
  }
  count(5);
}

void moe_grouped_mlp(const at::Tensor& x, const at::Tensor& w13, const at::Tensor& w2, const at::Tensor& topk_w,
                     const at::Tensor& topk_ids, at::Tensor out, int64_t expert_offset) {
  CHECK_BF16(out);
  moe_grouped_mlp_impl(x, w13, w2, topk_w, topk_ids, out, expert_offset, nullptr, nullptr, 0, 1, nullptr, nullptr);
}

void moe_grouped_mlp_glu(const at::Tensor& x, const at::Tensor& w13, const at::Tensor& w2, const at::Tensor& topk_w,
                         const at::Tensor& topk_ids, at::Tensor out, int64_t expert_offset, double limit, double alpha) {
  CHECK_BF16(out);
  moe_grouped_mlp_impl(x, w13, w2, topk_w, topk_ids, out, expert_offset, nullptr, nullptr, 0, 1, nullptr, nullptr, 1, (float)limit, (float)alpha);
}

void moe_grouped_mlp_push(const at::Tensor& x, const at::Tensor& w13, const at::Tensor& w2, const at::Tensor& topk_w,
                          const at::Tensor& topk_ids, int64_t expert_offset, const at::Tensor& peer_slot_ptrs,
                          const at::Tensor& peer_flag_ptrs, int64_t rank, int64_t world, at::Tensor epoch, at::Tensor done) {
  TORCH_CHECK(!peer_slot_ptrs.is_cuda() && !peer_flag_ptrs.is_cuda());
  moe_grouped_mlp_impl(x, w13, w2, topk_w, topk_ids, c10::nullopt, expert_offset, peer_slot_ptrs.data_ptr<int64_t>(),
                       peer_flag_ptrs.data_ptr<int64_t>(), (int)rank, (int)world, reinterpret_cast<const uint32_t*>(epoch.data_ptr<int>()),
                       reinterpret_cast<uint32_t*>(done.data_ptr<int>()));
}

}  // namespace

TORCH_LIBRARY(sglb, m) {
  m.def("gemm_streamk(Tensor a, Tensor w, Tensor(a!) out, Tensor? bias, int epilogue) -> ()", &gemm_streamk);
  m.def("kv_transfer_pages(Tensor(a!) dev_buf, Tensor(b!) host_buf, Tensor dev_pages, Tensor host_pages, int planes, int dev_plane_stride, "
        "int host_plane_stride, int host_page_stride, int chunk_bytes, bool to_host) -> ()", &kv_transfer_pages);
  m.def("lora_sgmv(Tensor x, Tensor a_pool, Tensor b_pool, Tensor tile_slot, Tensor tile_start, Tensor tile_cnt, Tensor perm, Tensor(a!) h, "
        "Tensor(b!) y, int b1, int b2) -> ()", &lora_sgmv);
  m.def("gemm_skinny_splits(int M, int N, int K, int max_splits) -> int", &gemm_skinny_splits);
  m.def("gemm_skinny_norm_splits(int K, int s) -> int", &gemm_skinny_norm_splits);
  m.def("gemm_skinny(Tensor a, Tensor w, Tensor(a!) out, Tensor? bias, int epilogue, int splits) -> ()", &gemm_skinny);
  m.def("gemm_skinny_push(Tensor a, Tensor w, int splits, Tensor peer_slot_ptrs, Tensor peer_flag_ptrs, int rank, int world, "
        "Tensor(a!) epoch, Tensor(b!) done) -> ()", &gemm_skinny_push);
  m.def("slab_reduce_add_rmsnorm(Tensor slabs, Tensor(a!)? residual, Tensor w, Tensor(b!) out, float eps, bool gemma) -> ()",
        &slab_reduce_add_rmsnorm);
  m.def("per_token_group_quant_fp8(Tensor x, Tensor(a!) q, Tensor(b!) scales, int group, bool ue8m0) -> ()", &per_token_group_quant_fp8);
  m.def("gemm_fp8_block(Tensor xq, Tensor xs, Tensor wq, Tensor ws, Tensor(a!) out) -> ()", &gemm_fp8_block);
  m.def("moe_topk_softmax(Tensor logits, Tensor(a!) out_w, Tensor(b!) out_ids, bool renorm) -> ()", &moe_topk_softmax);
  m.def("moe_grouped_mlp(Tensor x, Tensor w13, Tensor w2, Tensor topk_w, Tensor topk_ids, Tensor(a!) out, int expert_offset) -> ()",
        &moe_grouped_mlp);
  m.def("moe_grouped_mlp_glu(Tensor x, Tensor w13, Tensor w2, Tensor topk_w, Tensor topk_ids, Tensor(a!) out, int expert_offset, float limit, "
        "float alpha) -> ()", &moe_grouped_mlp_glu);
  m.def("moe_grouped_mlp_push(Tensor x, Tensor w13, Tensor w2, Tensor topk_w, Tensor topk_ids, int expert_offset, Tensor peer_slot_ptrs, "
        "Tensor peer_flag_ptrs, int rank, int world, Tensor(a!) epoch, Tensor(b!) done) -> ()", &moe_grouped_mlp_push);
  m.def("gemm_push(Tensor a, Tensor w, Tensor peer_slot_ptrs, Tensor peer_flag_ptrs, int rank, int world, Tensor(a!) epoch, "
        "Tensor(b!) done, int bn) -> ()", &gemm_push);
  m.def("nvl_local_reduce_add_rmsnorm(Tensor slot, int flags_ptr, Tensor(a!)? residual, Tensor w, Tensor(b!) out, int world, int nslabs, float eps, "
        "bool gemma, Tensor(c!) epoch, Tensor(d!) done) -> ()", &nvl_local_reduce_add_rmsnorm);
  m.def("nvl_allreduce(Tensor buf_ptrs, Tensor flag_ptrs, int mc_ptr, int slot_off, int rank, int world, Tensor(a!) out, "
        "Tensor(b!) epoch, Tensor(c!) done, int channel, int algo) -> ()", &nvl_allreduce);
  m.def("nvl_ar_add_rmsnorm(Tensor buf_ptrs, Tensor flag_ptrs, int mc_ptr, int slot_off, int rank, int world, Tensor(a!)? residual, "
        "Tensor w, Tensor(b!) out, float eps, bool gemma, Tensor(c!) epoch, Tensor(d!) done, int channel) -> ()", &nvl_ar_add_rmsnorm);
  m.def("nvl_rs_add_rmsnorm_ag(Tensor buf_ptrs, Tensor flag_ptrs, int mc_ptr, int slot_off, int out_off, int rank, int world, "
        "Tensor(a!)? residual, Tensor w, int T, int H, float eps, bool gemma, Tensor(c!) epoch, Tensor(d!) done, int channel) -> ()",
        &nvl_rs_add_rmsnorm_ag);
  m.def("launch_count() -> int", &launch_count);
  m.def("reset_launch_count() -> ()", &reset_launch_count);
  m.def("gemm_pick_bn(int M, int N, int K) -> int", &gemm_pick_bn);
  m.def("rmsnorm(Tensor(a!) x, Tensor(b!)? residual, Tensor w, Tensor(c!) out, float eps, bool gemma) -> ()", &rmsnorm);
  m.def("act_and_mul(Tensor x, Tensor(a!) out, int act) -> ()", &act_and_mul);
  m.def("rope_kv_write(Tensor(a!) q, Tensor k, Tensor v, Tensor positions, Tensor cos_sin, Tensor(b!) k_cache, "
        "Tensor(c!) v_cache, Tensor out_loc, bool neox, float k_scale, float v_scale, int nslabs=1, int slab_stride=0) -> ()", &rope_kv_write);
  m.def("apply_pt_delta(Tensor(a!) page_table, Tensor rows, Tensor cols, Tensor vals, Tensor? n, int n_max) -> ()", &apply_pt_delta);
  m.def("embedding(Tensor weight, Tensor ids, Tensor? gather_idx, Tensor(a!) out, int vocab_start) -> ()", &embedding);
  m.def("gather_rows(Tensor x, Tensor idx, Tensor(a!) out) -> ()", &gather_rows);
  m.def("attn_fwd(Tensor q, Tensor k_cache, Tensor v_cache, Tensor(a!) out, Tensor(b!)? lse, Tensor(c!)? part_o, "
        "Tensor(d!)? part_lse, Tensor page_table, Tensor req_slots, Tensor seq_lens, Tensor? cu_q, Tensor? tok2req, "
        "int max_q_len, int page_size, int num_splits, float scale, bool causal, int window, float logit_cap, "
        "float k_scale, float v_scale, int impl, Tensor? tree_anc=None, Tensor? slopes=None, Tensor? log_rates=None, int keep_first=0) -> ()", &attn_fwd);
  m.def("attn_decode_prof(Tensor buf) -> ()", &attn_decode_prof);
  m.def("green_ctx_streams(int device, int[] sm_counts) -> int[]", [](int64_t device, std::vector<int64_t> counts) {
    std::vector<long long> c(counts.begin(), counts.end());
    auto r = sglb::green_ctx_streams((int)device, c);
    return std::vector<int64_t>(r.begin(), r.end());
  });
  m.def("add_rmsnorm_f32(Tensor(a!) residual, Tensor? delta, Tensor w, Tensor(b!) out, float eps, bool zero_centred) -> ()", &add_rmsnorm_f32);
  m.def("clamped_glu(Tensor gu, Tensor(a!) out, float limit, float alpha) -> ()", &clamped_glu);
  m.def("bigram_embedding(Tensor embed, Tensor? bigram, Tensor ids, Tensor(a!)? prev_tokens, Tensor? cu_q, Tensor req_slots, Tensor seq_lens, "
        "int max_q_len, float scale, int mul_prev, int mul_cur, int buckets, Tensor(b!) out) -> ()", &bigram_embedding);
  m.def("postnorm_add_rmsnorm_f32(Tensor(a!) residual, Tensor delta, Tensor post_w, Tensor w, Tensor(b!) out, float eps, bool zero_centred=True) -> ()",
        &postnorm_add_rmsnorm_f32);
  m.def("grouped_rmsnorm(Tensor x, Tensor w, int groups, float eps, Tensor(a!) out, Tensor? gate=None, float out_scale=1.0) -> ()", &grouped_rmsnorm);
  m.def("mamba2_scan(Tensor u, Tensor? z, Tensor? dt_raw, Tensor? dt_bias, Tensor? A_log, Tensor? D, Tensor(a!) state, Tensor req_slots, Tensor seq_lens, "
        "Tensor? cu_q, int H, int P, int N, int G, Tensor(b!) out, Tensor? decay=None, Tensor? gates=None) -> ()", &mamba2_scan);
  m.def("mamba1_scan(Tensor u, Tensor dt_raw, Tensor? dt_bias, Tensor A_log, Tensor Bm, Tensor Cm, Tensor? D, Tensor? z, Tensor(a!) state, Tensor req_slots, "
        "Tensor seq_lens, Tensor? cu_q, Tensor(b!) out) -> ()", &mamba1_scan);
  m.def("attention_prepare(Tensor qkv, int H, int G, int D, int Dv, Tensor positions, Tensor(a!) k_cache, Tensor(b!) v_cache, Tensor loc, Tensor? q_norm_w, "
        "Tensor? k_norm_w, float eps, Tensor? inv_freq, Tensor? v_first, float v_lambda, Tensor(c!) q_out, int pad=0, Tensor? v_inv_freq=None, "
        "bool v_interleaved=False) -> ()", &attention_prepare);
  m.def("sigmoid_gate(Tensor o, Tensor gate, int Dv, float out_scale, Tensor(a!) out) -> ()", &sigmoid_gate);
  m.def("activation(Tensor x, int act, Tensor(a!) out, Tensor? mul=None) -> ()", &activation);
  m.def("qk_norm_cache_write(Tensor qkv, int H, int G, int D, int Dv, Tensor positions, float eps, float temp_coef, int temp_every, "
        "Tensor(a!) k_cache, Tensor(b!) v_cache, Tensor loc, bool normalise, Tensor(c!) q_out, int pad=0) -> ()", &qk_norm_cache_write);
  m.def("window_attention(Tensor q, Tensor k_cache, Tensor v_cache, int G, int Dv, Tensor page_table, Tensor req_slots, Tensor seq_lens, Tensor? cu_q, "
        "int max_q_len, int page_size, float scale, float softcap, int window, Tensor? slopes, Tensor? sinks, Tensor(a!) out, int dim, int pad=0, "
        "int keep_first=0, Tensor? log_rates=None, Tensor? gate=None, float out_scale=1.0) -> ()",
        &window_attention);
  m.def("attention_sink_gate(Tensor o, Tensor lse, Tensor sinks, int Dv, Tensor(a!) out) -> ()", &attention_sink_gate);
  m.def("moe_softmax_bias_route(Tensor logits, Tensor? corr, int n_real, Tensor(a!) w, Tensor(b!) ids, Tensor(c!) ident) -> ()", &moe_softmax_bias_route);
  m.def("moe_identity_shared_combine(Tensor(a!) y, Tensor h, Tensor? ident, Tensor? shared, Tensor? gate) -> ()", &moe_identity_shared_combine);
  m.def("gated_delta_rule(Tensor u, int Hk, int Dk, int H, int Dv, Tensor a_raw, Tensor A_log, Tensor dt_bias, Tensor b_raw, Tensor(a!) state, "
        "Tensor req_slots, Tensor seq_lens, Tensor? cu_q, Tensor? gate_raw, Tensor? norm_w, float eps, bool gate_silu, bool per_channel, Tensor(b!) out) -> ()",
        &gated_delta_rule);
  m.def("latent_attention(Tensor q, Tensor cache, int rank, Tensor page_table, Tensor req_slots, Tensor seq_lens, Tensor? cu_q, int max_q_len, "
        "int max_kv_len, int page_size, float scale, int window, Tensor? sinks, Tensor(a!) out, int v_rank=0) -> ()", &latent_attention);
  m.def("latent_prepare(Tensor x, int q_rank, Tensor? q_norm_w, int rank, int rot_dim, Tensor kv_norm_w, float eps, Tensor positions, Tensor? inv_freq, "
        "float mult, Tensor(a!) cache, Tensor loc, Tensor(b!)? cq) -> ()", &latent_prepare);
  m.def("latent_query(Tensor q, Tensor q_abs, int dim, int rot_dim, Tensor positions, Tensor? inv_freq, float mult, Tensor(a!) out) -> ()", &latent_query);
  m.def("causal_softmax(Tensor scores, int tq, int first, float scale, Tensor(a!) out) -> ()", &causal_softmax);
  m.def("rotate_heads(Tensor o, Tensor positions, Tensor inv_freq, int Dv, bool interleaved, bool inverse, Tensor? lse, Tensor? sinks, Tensor(a!) out) -> ()",
        &rotate_heads);
  m.def("parallel_add_rmsnorm_f32(Tensor(a!) residual, Tensor? d1, Tensor? d2, Tensor? d3, Tensor w1, Tensor? w2, Tensor(b!) out1, Tensor(c!)? out2, float eps, "
        "bool zero_centred) -> ()", &parallel_add_rmsnorm_f32);
  m.def("mlstm_prepare(Tensor proj, Tensor gates_raw, int H, int D, int Dv, float cap, Tensor(a!) mstate, Tensor req_slots, Tensor seq_lens, Tensor? cu_q, "
        "Tensor(b!) u, Tensor(c!) gates) -> ()", &mlstm_prepare);
  m.def("mlstm_readout(Tensor y, Tensor gates, int H, int Dv, Tensor norm_w, float eps, Tensor? gate, Tensor(a!) out) -> ()", &mlstm_readout);
  m.def("gated_delta_update(Tensor(a!) state, Tensor req_slots, Tensor u, Tensor g, Tensor beta, int Hk, Tensor(b!) out) -> ()", &gated_delta_update);
  m.def("causal_conv1d(Tensor x, Tensor w, Tensor? bias, Tensor(a!) conv_state, Tensor? cu_q, Tensor req_slots, Tensor seq_lens, int max_q_len, "
        "bool silu, Tensor(b!) u) -> ()", &causal_conv1d);
  m.def("selective_state_update(Tensor(a!) state, Tensor req_slots, Tensor x, Tensor dt, Tensor A, Tensor Bm, Tensor Cm, Tensor? D, Tensor(b!) y) -> ()",
        &selective_state_update);
  m.def("gemm(Tensor a, Tensor w, Tensor(a!) out, Tensor? bias, int epilogue, int bn) -> ()", &gemm);
  m.def("sample(Tensor logits, Tensor temperature, Tensor top_k, Tensor top_p, Tensor min_p, Tensor? seeds, "
        "Tensor? out_slots, Tensor(a!)? next_token_buf, Tensor(b!) out_tokens, Tensor(c!)? out_logprobs, int global_seed, "
        "Tensor? step_ptr, int step) -> ()", &sample);
  m.def("greedy_shard(Tensor logits, int v_valid, int v_offset, int rank, int tp, Tensor(a!) buf) -> ()", &greedy_shard);
  m.def("greedy_merge(Tensor buf, int B, Tensor? out_slots, Tensor(a!)? next_token_buf, Tensor(b!) out_tokens) -> ()", &greedy_merge);
  m.def("apply_token_bitmask(Tensor(a!) logits, Tensor bitmask, Tensor? row_idx) -> ()", &apply_token_bitmask);
  m.def("apply_penalties(Tensor(a!) logits, Tensor counts, Tensor? prompt_mask, Tensor freq, Tensor pres, Tensor rep) -> ()",
        &apply_penalties);
  m.def("bump_counts(Tensor(a!) counts, Tensor tokens) -> ()", &bump_counts);
}
