// State-space (Mamba / Mamba-2) kernels: causal depthwise conv1d over ragged batches with a per-request rolling state, and the
// single-token selective state update of decode.
//
//   causal_conv1d (prefill / extend / decode):  u[t, c] = act(bias[c] + sum_{j<k} w[c, j] * x[t - (k-1) + j, c]),   x[<0] taken from conv_state
//        conv_state[slot, c, :] <- the last k-1 inputs of the request (shifted by the new tokens)
//   selective_state_update (decode):            S[b,h,p,:] = S * exp(dt[b,h] * A[h]) + dt[b,h] * x[b,h,p] * B[b,g,:]
//                                               y[b,h,p]   = <S[b,h,p,:], C[b,g,:]> + D[h] * x[b,h,p]
//
// Both are bandwidth kernels: the conv reads x once (threads = channels: coalesced rows), the state update reads and writes the fp32 state
// exactly once (one warp per (b, h, p) row, 16-byte lanes) instead of the 4–5 passes of the PyTorch expression.
//
// Reference counterparts: kernels/aot/csrc/mamba/causal_conv1d.cu (fwd + update), layers/attention/mamba/ops/mamba_ssm.py
// (selective_state_update Triton kernel); states indexed by request slot as in mem_cache/memory_pool.py MambaPool.
#include <type_traits>

#include "common.cuh"
#include "tma_host.h"

namespace sglb {

constexpr int CONV_MAX_K = 8;
constexpr int CONV_CHUNK = 128;      // tokens per block along a request

template <typename T> __device__ __forceinline__ float ld_f(const T* p);
template <> __device__ __forceinline__ float ld_f<float>(const float* p) { return *p; }
template <> __device__ __forceinline__ float ld_f<__nv_bfloat16>(const __nv_bfloat16* p) { return __bfloat162float(*p); }
template <typename T> __device__ __forceinline__ void st_f(T* p, float v);
template <> __device__ __forceinline__ void st_f<float>(float* p, float v) { *p = v; }
template <> __device__ __forceinline__ void st_f<__nv_bfloat16>(__nv_bfloat16* p, float v) { *p = __float2bfloat16(v); }

// grid (ceil(C / 256), chunks, B); thread = channel.  cu_q == nullptr: decode (one token per request, row = request index).
template <typename T>
__global__ void __launch_bounds__(256) causal_conv1d_fwd_kernel(const T* __restrict__ x, int ldx, const T* __restrict__ w, const T* __restrict__ bias,
                                                                const T* __restrict__ conv_state, const int* __restrict__ cu_q,
                                                                const int* __restrict__ req_slots, const int* __restrict__ seq_lens, int C, int K,
                                                                int silu, float* __restrict__ u, int ldu) {
  const int c = blockIdx.x * 256 + threadIdx.x;
  const int b = blockIdx.z;
  if (c >= C) return;
  const int q0 = cu_q ? cu_q[b] : b;
  const int n = cu_q ? cu_q[b + 1] - q0 : 1;
  const int t0 = blockIdx.y * CONV_CHUNK;
  if (t0 >= n) return;
  const int t1 = min(n, t0 + CONV_CHUNK);
  const bool fresh = seq_lens[b] - n == 0;            // first tokens of the request: the state is all zeros, whatever the slot holds
  const T* st = conv_state + ((size_t)req_slots[b] * C + c) * (K - 1);
  float wk[CONV_MAX_K], win[CONV_MAX_K];
#pragma unroll
  for (int j = 0; j < CONV_MAX_K; ++j) wk[j] = j < K ? ld_f<T>(w + (size_t)c * K + j) : 0.f;
  const float bs = bias ? ld_f<T>(bias + c) : 0.f;
  float w_last = 0.f;
#pragma unroll
  for (int j = 0; j < CONV_MAX_K; ++j)
    if (j == K - 1) w_last = wk[j];
  // window = inputs t0-(K-1) .. t0-1: from x when inside this call's tokens, else from the rolling state (position relative to its end)
#pragma unroll
  for (int j = 0; j < CONV_MAX_K - 1; ++j) {
    if (j < K - 1) {
      const int t = t0 - (K - 1) + j;
      float v = 0.f;
      if (t >= 0) v = ld_f<T>(x + (size_t)(q0 + t) * ldx + c);
      else if (!fresh) v = ld_f<T>(st + (K - 1) + t);
      win[j] = v;
    }
  }
  for (int t = t0; t < t1; ++t) {
    const float xv = ld_f<T>(x + (size_t)(q0 + t) * ldx + c);
    float acc = bs + w_last * xv;
#pragma unroll
    for (int j = 0; j < CONV_MAX_K - 1; ++j)
      if (j < K - 1) acc += wk[j] * win[j];
#pragma unroll
    for (int j = 0; j < CONV_MAX_K - 1; ++j) {
      if (j < K - 2) win[j] = win[j + 1];
      else if (j == K - 2) win[j] = xv;
    }
    if (silu) acc = acc / (1.f + __expf(-acc));
    u[(size_t)(q0 + t) * ldu + c] = acc;
  }
}

// second pass (stream-ordered after the forward, which still reads the OLD state): roll the state forward by the request's new tokens
template <typename T>
__global__ void __launch_bounds__(256) causal_conv1d_state_kernel(const T* __restrict__ x, int ldx, T* __restrict__ conv_state, const int* __restrict__ cu_q,
                                                                  const int* __restrict__ req_slots, const int* __restrict__ seq_lens, int C, int K) {
  const int c = blockIdx.x * 256 + threadIdx.x;
  const int b = blockIdx.y;
  if (c >= C) return;
  const int q0 = cu_q ? cu_q[b] : b;
  const int n = cu_q ? cu_q[b + 1] - q0 : 1;
  if (n <= 0) return;
  const bool fresh = seq_lens[b] - n == 0;
  T* st = conv_state + ((size_t)req_slots[b] * C + c) * (K - 1);
  float nw[CONV_MAX_K];
#pragma unroll
  for (int j = 0; j < CONV_MAX_K - 1; ++j) {
    if (j < K - 1) {
      const int t = n - (K - 1) + j;                 // input index (relative to this call) that ends up in state column j
      float v = 0.f;
      if (t >= 0) v = ld_f<T>(x + (size_t)(q0 + t) * ldx + c);
      else if (!fresh) v = ld_f<T>(st + (K - 1) + t);
      nw[j] = v;
    }
  }
#pragma unroll
  for (int j = 0; j < CONV_MAX_K - 1; ++j)
    if (j < K - 1) st_f<T>(st + j, nw[j]);
}

void causal_conv1d(const void* x, int ldx, const void* w, const void* bias, void* conv_state, const int* cu_q, const int* req_slots,
                   const int* seq_lens, int B, int max_q_len, int C, int K, bool silu, bool bf16, float* u, int ldu, cudaStream_t stream) {
  if (B <= 0) return;
  if (K < 2 || K > CONV_MAX_K) throw std::runtime_error("sglb causal_conv1d: kernel width must be 2..8");
  dim3 g1((C + 255) / 256, (std::max(max_q_len, 1) + CONV_CHUNK - 1) / CONV_CHUNK, B), g2((C + 255) / 256, B);
  if (bf16) {
    causal_conv1d_fwd_kernel<__nv_bfloat16><<<g1, 256, 0, stream>>>((const __nv_bfloat16*)x, ldx, (const __nv_bfloat16*)w, (const __nv_bfloat16*)bias,
                                                                    (const __nv_bfloat16*)conv_state, cu_q, req_slots, seq_lens, C, K, silu ? 1 : 0, u, ldu);
    causal_conv1d_state_kernel<__nv_bfloat16><<<g2, 256, 0, stream>>>((const __nv_bfloat16*)x, ldx, (__nv_bfloat16*)conv_state, cu_q, req_slots, seq_lens, C, K);
  } else {
    causal_conv1d_fwd_kernel<float><<<g1, 256, 0, stream>>>((const float*)x, ldx, (const float*)w, (const float*)bias, (const float*)conv_state, cu_q,
                                                            req_slots, seq_lens, C, K, silu ? 1 : 0, u, ldu);
    causal_conv1d_state_kernel<float><<<g2, 256, 0, stream>>>((const float*)x, ldx, (float*)conv_state, cu_q, req_slots, seq_lens, C, K);
  }
  SGLB_CUDA_CHECK(cudaGetLastError());
}

// one warp per (b, h, p) state row of N floats; x / B / C / dt fp32 (already activated), state fp32 [slots, H, P, N]
__global__ void __launch_bounds__(256) selective_state_update_kernel(float* __restrict__ state, const int* __restrict__ req_slots,
                                                                     const float* __restrict__ x, int ldx, const float* __restrict__ dt, const float* __restrict__ A,
                                                                     const float* __restrict__ Bm, const float* __restrict__ Cm, int ldbc,
                                                                     const float* __restrict__ Dv, int B, int H, int P, int N, int G, float* __restrict__ y) {
  const int warp = (blockIdx.x * 256 + threadIdx.x) >> 5, lane = threadIdx.x & 31;
  const int rows = B * H * P;
  if (warp >= rows) return;
  const int b = warp / (H * P), hp = warp - b * H * P, h = hp / P, p = hp - h * P;
  const int g = h / (H / G);
  const float dtv = dt[(size_t)b * H + h];
  const float dA = __expf(dtv * A[h]);
  const float xv = x[(size_t)b * ldx + h * P + p];
  const float dbx = dtv * xv;
  float* s = state + (((size_t)req_slots[b] * H + h) * P + p) * N;
  const float* bb = Bm + (size_t)b * ldbc + (size_t)g * N;
  const float* cc = Cm + (size_t)b * ldbc + (size_t)g * N;
  float acc = 0.f;
  for (int i = lane * 4; i < N; i += 128) {
    float4 sv = *reinterpret_cast<const float4*>(s + i);
    const float4 bv = *reinterpret_cast<const float4*>(bb + i);
    const float4 cv = *reinterpret_cast<const float4*>(cc + i);
    sv.x = sv.x * dA + dbx * bv.x; sv.y = sv.y * dA + dbx * bv.y; sv.z = sv.z * dA + dbx * bv.z; sv.w = sv.w * dA + dbx * bv.w;
    *reinterpret_cast<float4*>(s + i) = sv;
    acc += sv.x * cv.x + sv.y * cv.y + sv.z * cv.z + sv.w * cv.w;
  }
  acc = warp_sum(acc);
  if (lane == 0) y[(size_t)b * H * P + hp] = acc + (Dv ? Dv[h] * xv : 0.f);
}

void selective_state_update(float* state, const int* req_slots, const float* x, int ldx, const float* dt, const float* A, const float* Bm,
                            const float* Cm, int ldbc, const float* Dv, int B, int H, int P, int N, int G, float* y, cudaStream_t stream) {
  if (B <= 0) return;
  if (N % 4 || H % G) throw std::runtime_error("sglb selective_state_update: d_state must be a multiple of 4, heads a multiple of groups");
  const long long warps = (long long)B * H * P;
  selective_state_update_kernel<<<(unsigned)((warps * 32 + 255) / 256), 256, 0, stream>>>(state, req_slots, x, ldx, dt, A, Bm, Cm, ldbc, Dv, B, H, P, N, G, y);
  SGLB_CUDA_CHECK(cudaGetLastError());
}

// ---------------------------------------------------------------- gated delta rule, one token per request (Qwen3-Next / GDN linear attention)
//   S <- S * exp(g);  mem = S^T k;  delta = (v - mem) * beta;  S <- S + k delta^T;  o = S^T q        (S fp32 [Dk, Dv] per (request, value head))
// q and k arrive un-normalised from the conv (+SiLU) output: l2-normalised here, q also scaled by Dk^-1/2; value head h uses key head h / r.
// One block per (value head, request), thread = value column: the Dk-long column lives in registers between the two dependent passes,
// so the 64 KB state is read once and written once (the PyTorch form makes five passes).  Reference: fla / sglang fused_recurrent_gated_delta_rule.
// Threads = (DK / 64) key slices x Dv value columns: a thread keeps 64 state values of one column in registers (128 would spill).
template <int DK>
__global__ void __launch_bounds__(256) gated_delta_update_kernel(float* __restrict__ state, const int* __restrict__ req_slots, const float* __restrict__ u,
                                                                 int ldu, int k_off, int v_off, const float* __restrict__ g, const float* __restrict__ beta,
                                                                 int Hv, int r, int Dv, int dv_pad, float* __restrict__ out) {
  constexpr int NS = DK / 64;
  __shared__ float sq[DK], sk[DK], red[32], part[NS][256];
  const int h = blockIdx.x, b = blockIdx.y, hk = h / r;
  const float* row = u + (size_t)b * ldu;
  float qs = 0.f, ks = 0.f;
  for (int i = threadIdx.x; i < DK; i += blockDim.x) {
    const float qv = row[hk * DK + i], kv = row[k_off + hk * DK + i];
    sq[i] = qv; sk[i] = kv;
    qs += qv * qv; ks += kv * kv;
  }
  qs = warp_sum(qs); ks = warp_sum(ks);
  const int w = threadIdx.x >> 5, nw = blockDim.x >> 5;
  if ((threadIdx.x & 31) == 0) { red[w] = qs; red[16 + w] = ks; }
  __syncthreads();
  float tq = 0.f, tk = 0.f;
  for (int i = 0; i < nw; ++i) { tq += red[i]; tk += red[16 + i]; }
  const float qn = rsqrtf(tq + 1e-6f) * rsqrtf((float)DK), kn = rsqrtf(tk + 1e-6f);
  const int slice = threadIdx.x / dv_pad, v = threadIdx.x - slice * dv_pad;
  const bool live = v < Dv;
  const float decay = __expf(g[(size_t)b * Hv + h]);
  float* S = state + (((size_t)req_slots[b] * Hv + h) * DK + slice * 64) * Dv + v;
  float col[64];
  float mem = 0.f;
  if (live) {
#pragma unroll
    for (int k = 0; k < 64; ++k) {
      col[k] = S[(size_t)k * Dv] * decay;
      mem += col[k] * (sk[slice * 64 + k] * kn);
    }
  }
  part[slice][v] = mem;
  __syncthreads();
  float tot = 0.f;
#pragma unroll
  for (int i = 0; i < NS; ++i) tot += part[i][v];
  __syncthreads();
  float o = 0.f;
  if (live) {
    const float delta = (row[v_off + h * Dv + v] - tot) * beta[(size_t)b * Hv + h];
#pragma unroll
    for (int k = 0; k < 64; ++k) {
      const float s2 = col[k] + (sk[slice * 64 + k] * kn) * delta;
      S[(size_t)k * Dv] = s2;
      o += s2 * (sq[slice * 64 + k] * qn);
    }
  }
  part[slice][v] = o;
  __syncthreads();
  if (slice == 0 && live) {
    float oo = 0.f;
#pragma unroll
    for (int i = 0; i < NS; ++i) oo += part[i][v];
    out[((size_t)b * Hv + h) * Dv + v] = oo;
  }
}

bool gated_delta_update(float* state, const int* req_slots, const float* u, int ldu, int k_off, int v_off, const float* g, const float* beta, int B,
                        int Hv, int r, int Dk, int Dv, float* out, cudaStream_t stream) {
  if (B <= 0) return true;
  if ((Dk != 64 && Dk != 128) || Dv > (Dk == 64 ? 256 : 128)) return false;      // <= 256 threads per block
  dim3 grid(Hv, B);
  const int dv_pad = ((Dv + 31) / 32) * 32;
  if (Dk == 64) gated_delta_update_kernel<64><<<grid, dv_pad, 0, stream>>>(state, req_slots, u, ldu, k_off, v_off, g, beta, Hv, r, Dv, dv_pad, out);
  else gated_delta_update_kernel<128><<<grid, 2 * dv_pad, 0, stream>>>(state, req_slots, u, ldu, k_off, v_off, g, beta, Hv, r, Dv, dv_pad, out);
  SGLB_CUDA_CHECK(cudaGetLastError());
  return true;
}

// ---------------------------------------------------------------- Mamba-2 recurrence over a ragged batch (prompt portions and decode tokens alike)
//   dt = softplus(dt_raw + dt_bias);  S <- exp(-exp(A_log) dt) S + dt B x^T;  y = S^T C + D x;  y <- y * silu(z)       (S fp32 [N, P] per head)
// The columns of S (one per channel p of the head) never mix, so a CTA owns (request, head, a block of PC = 128 / KS columns) and walks the
// request's tokens in order; a column lives in the registers of KS neighbouring lanes (ROWS consecutive rows each, row = ks * ROWS + r) and
// S^T C closes with log2(KS) shuffles.  B and C sit in shared memory in pieces of ROWS + 4 floats per lane slice, so that every lane reads its
// rows with 16-byte loads and the KS slices of a warp do not collide.  Tokens are staged TC at a time through two shared-memory buffers: while the recurrence runs TC steps out of one
// buffer (broadcast reads, nothing global inside the serial chain), cp.async fills the other with the next tokens' B, C and x, and their z
// and dt wait in registers; outputs are collected in shared memory and written out coalesced per chunk.  The state is read once and written
// once per call; a request whose cached length is zero starts from S = 0 whatever its slot holds.  Token order is fixed, so a position's
// output is bit-identical however the prompt was cut or batched.
// Reference counterpart: layers/attention/mamba/ops (chunked SSD scan for prompts, selective_state_update for decode).
namespace {

struct Mamba2Params {
  const float* u; int ldu;                       // conv outputs [T, ldu] = [x (H*P) | B (G*N) | C (G*N)]
  const void* z; int ldz;                        // gate rows (model dtype) or null
  const void* dt_raw; int lddt;                  // [T, >= H] (model dtype)
  const float* dt_bias; const float* A_log; const float* D;
  const float* decay;                            // non-null: step size 1 and the head's constant decay (dt_raw, dt_bias, A_log unused)
  const float* gates; int gstride;               // non-null: [T, H, gstride] with every token's decay at [0] and step at [1] (likewise)
  float* state;                                  // [slots, H, N, P]
  const int* req_slots; const int* seq_lens; const int* cu_q;
  float* out;                                    // [T, H*P]
  int H, P, N, G, pchunks;
};

__device__ __forceinline__ float m2_softplus(float x) { return x > 20.f ? x : log1pf(expf(x)); }
__device__ __forceinline__ void m2_cp4(float* dst, const float* src) {
  asm volatile("cp.async.ca.shared.global [%0], [%1], 4;" ::"r"(smem_u32(dst)), "l"(src) : "memory");
}
__device__ __forceinline__ void m2_cp_wait() { asm volatile("cp.async.wait_all;" ::: "memory"); }

template <typename TZ, int ROWS, int KS, int TC, int CPT>
__global__ void __launch_bounds__(128) mamba2_scan_kernel(const Mamba2Params p) {
  extern __shared__ float sm[];
  constexpr int PCH = 128 / KS;                     // columns one pass of the CTA's threads covers
  constexpr int PC = CPT * PCH;                     // columns of the CTA: a thread owns CPT of them, PCH apart, and reuses every B / C read for all
  constexpr int ZR = (TC * PC + 127) / 128;         // z values a thread holds for the next chunk
  const int b = blockIdx.y;
  const int q0 = p.cu_q ? p.cu_q[b] : b;
  const int n = p.cu_q ? p.cu_q[b + 1] - q0 : 1;
  if (n <= 0) return;
  const int h = blockIdx.x / p.pchunks, pc = blockIdx.x - h * p.pchunks;
  const int H = p.H, P = p.P, N = p.N;
  const int g = h / (H / p.G);
  const int tid = threadIdx.x, col = tid / KS, ks = tid % KS;
  int pp[CPT];
  bool live[CPT];
#pragma unroll
  for (int c = 0; c < CPT; ++c) {
    pp[c] = pc * PC + c * PCH + col;
    live[c] = pp[c] < P;
  }
  constexpr int RP = ROWS + 4;                              // padded length of a lane slice of B / C
  constexpr int NS = KS * RP;                               // floats per token of B (and of C) in shared memory
  constexpr int stage = 2 * TC * NS + 2 * TC * PC + 2 * TC; // floats per buffer: B | C | x | z | dt | decay
  float* sY = sm + 2 * stage;                               // [TC][PC]
  float S[CPT][ROWS];
  float* st = p.state + ((size_t)p.req_slots[b] * H + h) * N * P;
  const bool fresh = p.seq_lens[b] - n == 0;
#pragma unroll
  for (int c = 0; c < CPT; ++c)
#pragma unroll
    for (int r = 0; r < ROWS; ++r) {
      const int i = ks * ROWS + r;
      S[c][r] = (live[c] && !fresh && i < N) ? st[(size_t)i * P + pp[c]] : 0.f;
    }
  if (N < KS * ROWS) {                 // rows beyond N stay zero in both buffers (the copies never touch them)
    for (int idx = tid; idx < 2 * stage; idx += 128) sm[idx] = 0.f;
    __syncthreads();
  }
  const bool fixed = p.decay || p.gates;
  const float a_exp = fixed ? 0.f : expf(p.A_log[h]);
  const float dskip = p.D ? p.D[h] : 0.f;
  const float dtb = fixed ? 0.f : p.dt_bias[h];
  const float fixed_decay = p.decay ? p.decay[h] : 0.f;
  const TZ* zg = reinterpret_cast<const TZ*>(p.z);
  const TZ* dg = reinterpret_cast<const TZ*>(p.dt_raw);
  const int inner = H * P;
  const int pw = min(PC, P - pc * PC);                      // live columns of this CTA
  float zr[ZR];
  float dtr = 0.f, dar = 0.f;

  auto issue = [&](int t0, float* buf) {      // start the copies of chunk [t0, t0 + TC) into buf; z and dt go to registers
    const int tc = min(TC, n - t0);
    float* sB = buf; float* sC = sB + TC * NS; float* sX = sC + TC * NS;
    for (int idx = tid; idx < tc * N; idx += 128) {
      const int tt = idx / N, i = idx - tt * N;
      const float* row = p.u + (size_t)(q0 + t0 + tt) * p.ldu + inner + g * N + i;
      const int at = tt * NS + (i / ROWS) * RP + (i % ROWS);
      m2_cp4(sB + at, row);
      m2_cp4(sC + at, row + p.G * N);
    }
    for (int idx = tid; idx < tc * PC; idx += 128) {
      const int tt = idx / PC, c = idx - tt * PC;
      if (c < pw) m2_cp4(sX + idx, p.u + (size_t)(q0 + t0 + tt) * p.ldu + h * P + pc * PC + c);
    }
#pragma unroll
    for (int k = 0; k < ZR; ++k) {
      const int idx = tid + k * 128, tt = idx / PC, c = idx - tt * PC;
      zr[k] = (zg && tt < tc && c < pw) ? ld_f<TZ>(zg + (size_t)(q0 + t0 + tt) * p.ldz + h * P + pc * PC + c) : 0.f;
    }
    if (p.gates) {
      if (tid < tc) {
        const float* gt = p.gates + ((size_t)(q0 + t0 + tid) * H + h) * p.gstride;
        dar = gt[0];
        dtr = gt[1];
      }
    } else if (dg && tid < tc) dtr = ld_f<TZ>(dg + (size_t)(q0 + t0 + tid) * p.lddt + h);
  };
  auto land = [&](int t0, float* buf) {       // finish what issue() started
    const int tc = min(TC, n - t0);
    float* sZ = buf + 2 * TC * NS + TC * PC; float* sDt = sZ + TC * PC; float* sDa = sDt + TC;
#pragma unroll
    for (int k = 0; k < ZR; ++k) {
      const int idx = tid + k * 128;
      if (idx < TC * PC) sZ[idx] = zr[k];
    }
    if (tid < tc) {
      const float dt = p.gates ? dtr : p.decay ? 1.f : m2_softplus(dtr + dtb);
      sDt[tid] = dt;
      sDa[tid] = p.gates ? dar : p.decay ? fixed_decay : expf(-a_exp * dt);
    }
    m2_cp_wait();
  };

  issue(0, sm);
  land(0, sm);
  __syncthreads();
  int cur = 0;
  for (int t0 = 0; t0 < n; t0 += TC, cur ^= 1) {
    const int tc = min(TC, n - t0);
    float* buf = sm + cur * stage;
    float* nxt = sm + (cur ^ 1) * stage;
    const bool more = t0 + TC < n;
    if (more) issue(t0 + TC, nxt);
    const float* sB = buf; const float* sC = sB + TC * NS; const float* sX = sC + TC * NS; const float* sZ = sX + TC * PC;
    const float* sDt = sZ + TC * PC; const float* sDa = sDt + TC;
    for (int tt = 0; tt < tc; ++tt) {
      const float dt = sDt[tt], da = sDa[tt];
      float xv[CPT], dbx[CPT], a0[CPT], a1[CPT];
#pragma unroll
      for (int c = 0; c < CPT; ++c) {
        xv[c] = live[c] ? sX[tt * PC + c * PCH + col] : 0.f;
        dbx[c] = dt * xv[c];
        a0[c] = a1[c] = 0.f;
      }
      const float4* bb = reinterpret_cast<const float4*>(sB + tt * NS + ks * RP);
      const float4* cc = reinterpret_cast<const float4*>(sC + tt * NS + ks * RP);
#pragma unroll
      for (int r = 0; r < ROWS; r += 4) {
        const float4 bv = bb[r >> 2], cv = cc[r >> 2];
#pragma unroll
        for (int c = 0; c < CPT; ++c) {
          S[c][r] = S[c][r] * da + dbx[c] * bv.x;
          S[c][r + 1] = S[c][r + 1] * da + dbx[c] * bv.y;
          S[c][r + 2] = S[c][r + 2] * da + dbx[c] * bv.z;
          S[c][r + 3] = S[c][r + 3] * da + dbx[c] * bv.w;
          a0[c] += S[c][r] * cv.x;
          a1[c] += S[c][r + 1] * cv.y;
          a0[c] += S[c][r + 2] * cv.z;
          a1[c] += S[c][r + 3] * cv.w;
        }
      }
#pragma unroll
      for (int c = 0; c < CPT; ++c) {
        float acc = a0[c] + a1[c];
#pragma unroll
        for (int o = 1; o < KS; o <<= 1) acc += __shfl_xor_sync(0xffffffffu, acc, o);
        if (ks == 0) sY[tt * PC + c * PCH + col] = acc + dskip * xv[c];
      }
    }
    __syncthreads();                                         // sY complete, everyone is done with buf
    for (int idx = tid; idx < tc * PC; idx += 128) {
      const int tt = idx / PC, c = idx - tt * PC;
      if (c < pw) {
        float y = sY[idx];
        if (zg) {
          const float zz = sZ[idx];
          y *= zz / (1.f + expf(-zz));
        }
        p.out[(size_t)(q0 + t0 + tt) * inner + h * P + pc * PC + c] = y;
      }
    }
    if (more) land(t0 + TC, nxt);
    __syncthreads();                                         // nxt visible, sY free
  }
#pragma unroll
  for (int c = 0; c < CPT; ++c) {
    if (!live[c]) continue;
#pragma unroll
    for (int r = 0; r < ROWS; ++r) {
      const int i = ks * ROWS + r;
      if (i < N) st[(size_t)i * P + pp[c]] = S[c][r];
    }
  }
}

template <typename TZ, int ROWS, int KS, int TC, int CPT>
void launch_m2c(Mamba2Params p, int B, cudaStream_t stream) {
  constexpr int PC = CPT * (128 / KS);
  p.pchunks = (p.P + PC - 1) / PC;
  const size_t smem = sizeof(float) * (2 * ((size_t)2 * TC * KS * (ROWS + 4) + 2 * TC * PC + 2 * TC) + (size_t)TC * PC);
  auto kern = mamba2_scan_kernel<TZ, ROWS, KS, TC, CPT>;
  if (smem > 48 * 1024) SGLB_CUDA_CHECK(cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));
  kern<<<dim3(p.H * p.pchunks, B), 128, smem, stream>>>(p);
  SGLB_CUDA_CHECK(cudaGetLastError());
}

// two columns per thread halve the staging and the shared-memory reads per column; taken when the head is wide enough and the grid still
// fills the GPU about twice over
template <typename TZ, int ROWS, int KS, int TC>
void launch_m2(const Mamba2Params& p, int B, cudaStream_t stream) {
  constexpr int PC2 = 2 * (128 / KS);
  const long long ctas2 = (long long)p.H * ((p.P + PC2 - 1) / PC2) * B;
  if (ROWS <= 16 && p.P >= PC2 && ctas2 >= 256) launch_m2c<TZ, ROWS, KS, TC, 2>(p, B, stream);
  else launch_m2c<TZ, ROWS, KS, TC, 1>(p, B, stream);
}

template <typename TZ>
void dispatch_m2(const Mamba2Params& p, int B, cudaStream_t stream) {
  const int N = p.N;
  if (N <= 16) launch_m2<TZ, 16, 1, 16>(p, B, stream);
  else if (N <= 32) launch_m2<TZ, 16, 2, 16>(p, B, stream);
  else if (N <= 64) launch_m2<TZ, 16, 4, 16>(p, B, stream);
  else if (N <= 128) launch_m2<TZ, 16, 8, 16>(p, B, stream);
  else if (N <= 256) launch_m2<TZ, 16, 16, 16>(p, B, stream);
  else if (N <= 512) launch_m2<TZ, 16, 32, 8>(p, B, stream);
  else launch_m2<TZ, 32, 32, 8>(p, B, stream);
}

}  // namespace

void mamba2_scan(const float* u, int ldu, const void* z, int ldz, const void* dt_raw, int lddt, bool bf16, const float* dt_bias, const float* A_log,
                 const float* D, float* state, const int* req_slots, const int* seq_lens, const int* cu_q, int B, int H, int P, int N, int G, float* out,
                 const float* decay, const float* gates, int gstride, cudaStream_t stream) {
  if (B <= 0) return;
  if (N > 1024 || B > 65535 || H % G) throw std::runtime_error("sglb mamba2_scan: state size up to 1024, heads a multiple of groups");
  if (!decay && !gates && (!dt_raw || !dt_bias || !A_log)) throw std::runtime_error("sglb mamba2_scan: step-size inputs, a constant decay or per-token gates");
  Mamba2Params p;
  p.decay = decay; p.gates = gates; p.gstride = gstride;
  p.u = u; p.ldu = ldu; p.z = z; p.ldz = ldz; p.dt_raw = dt_raw; p.lddt = lddt; p.dt_bias = dt_bias; p.A_log = A_log; p.D = D; p.state = state;
  p.req_slots = req_slots; p.seq_lens = seq_lens; p.cu_q = cu_q; p.out = out; p.H = H; p.P = P; p.N = N; p.G = G; p.pchunks = 1;
  if (bf16) dispatch_m2<__nv_bfloat16>(p, B, stream);
  else dispatch_m2<float>(p, B, stream);
}

// ---------------------------------------------------------------- matrix memory with exponential gates and a running maximum (mLSTM): what surrounds the scan
//   i = cap tanh(raw_i / cap);  f = logsigmoid(cap tanh(raw_f / cap));  m_t = max(f + m_(t-1), i), m = 0 at the start of a sequence;
//   decay_t = exp(f + m_(t-1) - m_t), step_t = exp(i - m_t), floor_t = exp(-m_t).
// With those the memory S_t = decay_t S_(t-1) + step_t k v^T and its normaliser n_t (the same recurrence on a value that is always 1) run on
// mamba2_scan(gates): x = [v | 1] per head, B = k, C = q / sqrt(D).
// mlstm_prepare, one launch with two kinds of CTA: the first hold four warps, a warp per (request, head), which walks m through the
// request's tokens 32 at a time (gate activations lane-parallel, the max-chain by shuffles, the three exponentials lane-parallel again) and
// leaves m in mstate [slots, H]; the T CTAs behind them write a token's [x | B | C] row in fp32 each.  Everything fp32.
// mlstm_readout: o = y[:Dv] / (max(|y[Dv]|, floor) + 1e-6) per head, divided by its root mean square, times weight, times sigmoid(gate); a warp
// per (token, head).
namespace {

template <typename T> __device__ __forceinline__ float ml_ld(const T* p);
template <> __device__ __forceinline__ float ml_ld<float>(const float* p) { return *p; }
template <> __device__ __forceinline__ float ml_ld<__nv_bfloat16>(const __nv_bfloat16* p) { return __bfloat162float(*p); }
template <typename T> __device__ __forceinline__ void ml_st(T* p, float v);
template <> __device__ __forceinline__ void ml_st<float>(float* p, float v) { *p = v; }
template <> __device__ __forceinline__ void ml_st<__nv_bfloat16>(__nv_bfloat16* p, float v) { *p = __float2bfloat16(v); }

template <typename T>
__global__ void __launch_bounds__(128) mlstm_prepare_kernel(const T* __restrict__ proj, int ld, const float* __restrict__ raw, int H, int D, int Dv, float cap,
                                                            float* __restrict__ mstate, const int* __restrict__ req_slots, const int* __restrict__ seq_lens,
                                                            const int* __restrict__ cu_q, int Tn, int B, float* __restrict__ u, float* __restrict__ gates) {
  const int tid = threadIdx.x;
  const int gate_ctas = (B * H + 3) / 4;             // they come first: their serial walk overlaps the row conversion of the CTAs behind them
  if ((int)blockIdx.x >= gate_ctas) {
    const int t = blockIdx.x - gate_ctas;
    const T* row = proj + (size_t)t * ld;
    const int nk = H * D, P = Dv + 1, nx = H * P;
    float* dst = u + (size_t)t * (nx + 2 * nk);
    for (int h = 0; h < H; ++h) {
      const T* src = row + 2 * nk + h * Dv;
      float* d = dst + h * P;
      for (int c = tid; c < Dv; c += 128) d[c] = ml_ld<T>(src + c);
      if (tid == 0) d[Dv] = 1.f;
    }
    const float qs = 1.0f / sqrtf((float)D);
    for (int idx = tid; idx < nk; idx += 128) {
      dst[nx + idx] = ml_ld<T>(row + nk + idx);
      dst[nx + nk + idx] = ml_ld<T>(row + idx) * qs;
    }
    return;
  }
  const int w = (int)blockIdx.x * 4 + (tid >> 5), lane = tid & 31;
  if (w >= B * H) return;
  const int b = w / H, h = w - b * H;
  const int q0 = cu_q ? cu_q[b] : b;
  const int n = cu_q ? cu_q[b + 1] - q0 : 1;
  if (n <= 0) return;
  float* ms = mstate + (size_t)req_slots[b] * H + h;
  float m = seq_lens[b] - n == 0 ? 0.f : *ms;
  for (int t0 = 0; t0 < n; t0 += 32) {
    const int tt = t0 + lane;
    float ig = 0.f, fg = 0.f;
    if (tt < n) {
      const float* r = raw + (size_t)(q0 + tt) * 2 * H;
      float ri = r[h], rf = r[H + h];
      if (cap > 0.f) { ri = cap * tanhf(ri / cap); rf = cap * tanhf(rf / cap); }
      ig = ri;
      fg = fminf(rf, 0.f) - log1pf(expf(-fabsf(rf)));
    }
    float m_prev = 0.f, m_new = 0.f;
    const int cnt = min(32, n - t0);
    for (int j = 0; j < cnt; ++j) {
      const float fj = __shfl_sync(0xffffffffu, fg, j), ij = __shfl_sync(0xffffffffu, ig, j);
      const float mn = fmaxf(fj + m, ij);
      if (lane == j) { m_prev = m; m_new = mn; }
      m = mn;
    }
    if (tt < n) {
      float* g = gates + ((size_t)(q0 + tt) * H + h) * 3;
      g[0] = expf(fg + m_prev - m_new);
      g[1] = expf(ig - m_new);
      g[2] = expf(-m_new);
    }
  }
  if (lane == 0) *ms = m;
}

template <typename TO>
__global__ void __launch_bounds__(128) mlstm_readout_kernel(const float* __restrict__ y, const float* __restrict__ gates, int rows, int H, int Dv,
                                                            const TO* __restrict__ w, float eps, const TO* __restrict__ gate, int ldg, TO* __restrict__ out) {
  const int row = blockIdx.x * 4 + (threadIdx.x >> 5), lane = threadIdx.x & 31;          // row = t * H + h
  if (row >= rows) return;
  const int t = row / H, h = row - t * H;
  const float* yy = y + (size_t)row * (Dv + 1);
  const float inv = 1.0f / (fmaxf(fabsf(yy[Dv]), gates[(size_t)row * 3 + 2]) + 1e-6f);
  float ss = 0.f;
  for (int c = lane; c < Dv; c += 32) {
    const float o = yy[c] * inv;
    ss += o * o;
  }
  const float rs = inv / sqrtf(warp_sum(ss) / (float)Dv + eps);
  const TO* wr = w + (size_t)h * Dv;
  const TO* gr = gate ? gate + (size_t)t * ldg + (size_t)h * Dv : nullptr;
  TO* dst = out + (size_t)row * Dv;
  for (int c = lane; c < Dv; c += 32) {
    float v = yy[c] * rs * ml_ld<TO>(wr + c);
    if (gr) v *= 1.f / (1.f + expf(-ml_ld<TO>(gr + c)));
    ml_st<TO>(dst + c, v);
  }
}

}  // namespace

void mlstm_prepare(const void* proj, int ld, bool bf16, const float* raw, int T, int B, int H, int D, int Dv, float cap, float* mstate, const int* req_slots,
                   const int* seq_lens, const int* cu_q, float* u, float* gates, cudaStream_t stream) {
  if (T <= 0 || B <= 0) return;
  const int grid = T + (B * H + 3) / 4;
  if (bf16)
    mlstm_prepare_kernel<__nv_bfloat16><<<grid, 128, 0, stream>>>((const __nv_bfloat16*)proj, ld, raw, H, D, Dv, cap, mstate, req_slots, seq_lens, cu_q, T, B,
                                                                  u, gates);
  else
    mlstm_prepare_kernel<float><<<grid, 128, 0, stream>>>((const float*)proj, ld, raw, H, D, Dv, cap, mstate, req_slots, seq_lens, cu_q, T, B, u, gates);
  SGLB_CUDA_CHECK(cudaGetLastError());
}

void mlstm_readout(const float* y, const float* gates, int T, int H, int Dv, const void* w, float eps, const void* gate, int ldg, void* out, bool out_bf16,
                   cudaStream_t stream) {
  if (T <= 0 || H <= 0) return;
  const int rows = T * H;
  if (out_bf16)
    mlstm_readout_kernel<__nv_bfloat16><<<(rows + 3) / 4, 128, 0, stream>>>(y, gates, rows, H, Dv, (const __nv_bfloat16*)w, eps, (const __nv_bfloat16*)gate,
                                                                            ldg, (__nv_bfloat16*)out);
  else
    mlstm_readout_kernel<float><<<(rows + 3) / 4, 128, 0, stream>>>(y, gates, rows, H, Dv, (const float*)w, eps, (const float*)gate, ldg, (float*)out);
  SGLB_CUDA_CHECK(cudaGetLastError());
}

// ---------------------------------------------------------------- Mamba-1 selective scan over a ragged batch
//   dt = softplus(dt_raw + dt_bias) per channel;  S[c, n] <- exp(-dt_c exp(A_log[c, n])) S[c, n] + dt_c u_c B_n;  y_c = sum_n S[c, n] C_n + D_c u_c;
//   y <- y * silu(z).  State fp32 [slots, C, N]; a request whose cached length is zero starts from S = 0 whatever its slot holds.
// Mapping: CTA = (block of CH channels, request), 128 threads; a channel's N states lie in the registers of LPC neighbouring lanes, NPT per
// lane (A likewise: exp(A_log) is computed once per call); tokens are staged TC at a time through shared memory (B, C per state; dt, u, z
// per channel), so the serial chain reads no global memory, and the next chunk's inputs are fetched into registers while the current one is
// computed; the read-out is reduced over the channel's lanes with shuffles and leaves through shared memory in rows.  Token order is fixed;
// how many states a lane holds (and so the order of the read-out's sum) follows the grid size, and single decode tokens take a kernel
// without staging: a position's output depends on how the prompt was cut or batched by fp32 rounding only.
namespace {

struct Mamba1Params {
  const float* u; const float* dt_raw; int lddt;
  const float* dt_bias; const float* A_log;
  const void* Bm; const void* Cm; int ldbc;
  const float* D; const void* z; int ldz;
  float* state;
  const int* req_slots; const int* seq_lens; const int* cu_q;
  void* out;
  int C, N;
};

template <typename T> __device__ __forceinline__ float m1_ld(const T* p);
template <> __device__ __forceinline__ float m1_ld<float>(const float* p) { return *p; }
template <> __device__ __forceinline__ float m1_ld<__nv_bfloat16>(const __nv_bfloat16* p) { return __bfloat162float(*p); }
template <typename T> __device__ __forceinline__ void m1_st(T* p, float v);
template <> __device__ __forceinline__ void m1_st<float>(float* p, float v) { *p = v; }
template <> __device__ __forceinline__ void m1_st<__nv_bfloat16>(__nv_bfloat16* p, float v) { *p = __float2bfloat16(v); }

template <typename TBC, typename TZ, typename TO, int NPT, int LPC, int TC>
__global__ void __launch_bounds__(128) mamba1_scan_kernel(const Mamba1Params p) {
  constexpr int CH = 128 / LPC;                     // channels per CTA
  constexpr int NP = NPT * LPC;                     // padded state size
  __shared__ float sB[TC][NP], sC[TC][NP], sDt[TC][CH], sU[TC][CH], sZ[TC][CH], sY[TC][CH];
  const int b = blockIdx.y;
  const int q0 = p.cu_q ? p.cu_q[b] : b;
  const int n = p.cu_q ? p.cu_q[b + 1] - q0 : 1;
  if (n <= 0) return;
  const int C = p.C, N = p.N;
  const int tid = threadIdx.x, cl = tid / LPC, ks = tid % LPC;
  const int c0 = blockIdx.x * CH, c = c0 + cl;
  const bool live = c < C;
  const bool fresh = p.seq_lens[b] - n == 0;
  float* st = p.state + ((size_t)p.req_slots[b] * C + (live ? c : 0)) * N;
  float S[NPT], A[NPT];
  const bool vec4 = NPT % 4 == 0 && (N % 4) == 0;   // a lane's states are whole 16-byte groups
  if (vec4) {
#pragma unroll
    for (int r = 0; r + 3 < NPT; r += 4) {
      const int i = ks * NPT + r;
      const bool ok = live && i < N;
      const float4 sv = (ok && !fresh) ? *reinterpret_cast<const float4*>(st + i) : make_float4(0.f, 0.f, 0.f, 0.f);
      const float4 av = ok ? *reinterpret_cast<const float4*>(p.A_log + (size_t)c * N + i) : make_float4(0.f, 0.f, 0.f, 0.f);
      S[r] = sv.x; S[r + 1] = sv.y; S[r + 2] = sv.z; S[r + 3] = sv.w;
      A[r] = ok ? -expf(av.x) : 0.f; A[r + 1] = ok ? -expf(av.y) : 0.f; A[r + 2] = ok ? -expf(av.z) : 0.f; A[r + 3] = ok ? -expf(av.w) : 0.f;
    }
  } else {
#pragma unroll
    for (int r = 0; r < NPT; ++r) {
      const int i = ks * NPT + r;
      const bool ok = live && i < N;
      S[r] = (ok && !fresh) ? st[i] : 0.f;
      A[r] = ok ? -expf(p.A_log[(size_t)c * N + i]) : 0.f;
    }
  }
  const float dskip = (p.D && live) ? p.D[c] : 0.f;
  const TBC* Bg = reinterpret_cast<const TBC*>(p.Bm);
  const TBC* Cg = reinterpret_cast<const TBC*>(p.Cm);
  const TZ* zg = reinterpret_cast<const TZ*>(p.z);
  TO* og = reinterpret_cast<TO*>(p.out);
  const int cw = min(CH, C - c0);                   // live channels of this CTA
  constexpr int NBC = (TC * NP + 127) / 128;        // B (and C) values a thread fetches per chunk
  constexpr int NCH = (TC * CH + 127) / 128;        // dt (and u, z) values a thread fetches per chunk
  float rB[NBC], rC[NBC], rDt[NCH], rU[NCH], rZ[NCH];
  auto fetch = [&](int t0) {                        // the chunk's inputs into registers: the loads fly while the previous chunk is computed
    const int tc = min(TC, n - t0);
#pragma unroll
    for (int k = 0; k < NBC; ++k) {
      const int idx = tid + k * 128, tt = idx / NP, i = idx - tt * NP;
      const bool ok = tt < tc && i < N;
      const size_t row = (size_t)(q0 + t0 + (ok ? tt : 0)) * p.ldbc;
      rB[k] = ok ? m1_ld<TBC>(Bg + row + i) : 0.f;
      rC[k] = ok ? m1_ld<TBC>(Cg + row + i) : 0.f;
    }
#pragma unroll
    for (int k = 0; k < NCH; ++k) {
      const int idx = tid + k * 128, tt = idx / CH, kk = idx - tt * CH;
      const bool ok = tt < tc && kk < cw;
      const size_t tok = (size_t)(q0 + t0 + (ok ? tt : 0));
      rDt[k] = ok ? p.dt_raw[tok * p.lddt + c0 + kk] + (p.dt_bias ? p.dt_bias[c0 + kk] : 0.f) : 0.f;
      rU[k] = ok ? p.u[tok * C + c0 + kk] : 0.f;
      rZ[k] = (ok && zg) ? m1_ld<TZ>(zg + tok * p.ldz + c0 + kk) : 0.f;
    }
  };
  fetch(0);
  for (int t0 = 0; t0 < n; t0 += TC) {
    const int tc = min(TC, n - t0);
    __syncthreads();                                // the previous chunk's rows are out
#pragma unroll
    for (int k = 0; k < NBC; ++k) {
      const int idx = tid + k * 128;
      if (idx < TC * NP) { (&sB[0][0])[idx] = rB[k]; (&sC[0][0])[idx] = rC[k]; }
    }
#pragma unroll
    for (int k = 0; k < NCH; ++k) {
      const int idx = tid + k * 128;
      if (idx < TC * CH) {
        const float raw = rDt[k];
        (&sDt[0][0])[idx] = raw > 20.f ? raw : log1pf(expf(raw));
        (&sU[0][0])[idx] = rU[k];
        (&sZ[0][0])[idx] = rZ[k];
      }
    }
    __syncthreads();
    if (t0 + TC < n) fetch(t0 + TC);
    for (int tt = 0; tt < tc; ++tt) {
      const float dt = sDt[tt][cl], uv = sU[tt][cl];
      const float dbu = dt * uv;
      float acc = 0.f;
#pragma unroll
      for (int r = 0; r < NPT; ++r) {
        const int i = ks * NPT + r;
        const float da = sizeof(TO) == 4 ? expf(dt * A[r]) : __expf(dt * A[r]);
        S[r] = da * S[r] + dbu * sB[tt][i];
        acc += S[r] * sC[tt][i];
      }
#pragma unroll
      for (int o = 1; o < LPC; o <<= 1) acc += __shfl_xor_sync(0xffffffffu, acc, o);
      if (ks == 0) sY[tt][cl] = acc + dskip * uv;
    }
    __syncthreads();
    for (int idx = tid; idx < tc * CH; idx += 128) {
      const int tt = idx / CH, k = idx - tt * CH;
      if (k < cw) {
        float y = sY[tt][k];
        if (zg) {
          const float zz = sZ[tt][k];
          y *= zz / (1.f + expf(-zz));
        }
        m1_st<TO>(og + (size_t)(q0 + t0 + tt) * C + c0 + k, y);
      }
    }
  }
  if (live && vec4) {
#pragma unroll
    for (int r = 0; r + 3 < NPT; r += 4) {
      const int i = ks * NPT + r;
      if (i < N) *reinterpret_cast<float4*>(st + i) = make_float4(S[r], S[r + 1], S[r + 2], S[r + 3]);
    }
  } else if (live) {
#pragma unroll
    for (int r = 0; r < NPT; ++r) {
      const int i = ks * NPT + r;
      if (i < N) st[i] = S[r];
    }
  }
}

template <typename TBC, typename TZ, typename TO, int NPT, int LPC>
void launch_m1(const Mamba1Params& p, int B, cudaStream_t stream) {
  constexpr int CH = 128 / LPC;
  constexpr int TC = NPT * LPC <= 64 ? 16 : (NPT * LPC <= 128 ? 8 : 4);          // tokens per staged chunk: the prefetch registers stay few
  mamba1_scan_kernel<TBC, TZ, TO, NPT, LPC, TC><<<dim3((p.C + CH - 1) / CH, B), 128, 0, stream>>>(p);
  SGLB_CUDA_CHECK(cudaGetLastError());
}

// fewer states per lane = more lanes and CTAs per channel block: taken (for the usual equal input / output types and small states) when the
// grid would otherwise leave SMs idle — one long prompt is a serial chain per channel, so parallelism has to come from the state dimension
template <typename TBC, typename TZ, typename TO, int LPC4>
void launch_m1_small(const Mamba1Params& p, int B, cudaStream_t stream) {
  if constexpr (std::is_same<TBC, TZ>::value && std::is_same<TBC, TO>::value) {
    const long long ctas4 = (long long)((p.C + 128 / LPC4 - 1) / (128 / LPC4)) * B;          // CTAs with 4 states per lane
    if (ctas4 < 600 && p.N > 2 * LPC4) {
      if (ctas4 < 300 && LPC4 * 4 <= 32) launch_m1<TBC, TZ, TO, 1, LPC4 * 4>(p, B, stream);
      else launch_m1<TBC, TZ, TO, 2, LPC4 * 2>(p, B, stream);
      return;
    }
  }
  launch_m1<TBC, TZ, TO, 4, LPC4>(p, B, stream);
}

// one token per request (decode): no staging.  A lane holds 4 states of its channel; a channel's LPC lanes sit in one warp; the state is read
// and written with 16-byte accesses, everything else is a handful of scalars per lane.
template <typename TBC, typename TZ, typename TO, int LPC>
__global__ void __launch_bounds__(256) mamba1_decode_kernel(const Mamba1Params p) {
  const int b = blockIdx.y;
  const int gid = blockIdx.x * 256 + threadIdx.x;
  const int c = gid / LPC, ks = gid - c * LPC;
  const int C = p.C, N = p.N;
  const bool live = c < C;
  const int i = ks * 4;
  const bool ok = live && i < N;
  const bool fresh = p.seq_lens[b] - 1 == 0;
  float* st = p.state + ((size_t)p.req_slots[b] * C + (live ? c : 0)) * N + (ok ? i : 0);
  float4 S = make_float4(0.f, 0.f, 0.f, 0.f), A = S, Bv = S, Cv = S;
  if (ok) {
    if (!fresh) S = *reinterpret_cast<const float4*>(st);
    A = *reinterpret_cast<const float4*>(p.A_log + (size_t)c * N + i);
    const TBC* br = reinterpret_cast<const TBC*>(p.Bm) + (size_t)b * p.ldbc + i;
    const TBC* cr = reinterpret_cast<const TBC*>(p.Cm) + (size_t)b * p.ldbc + i;
    Bv = make_float4(m1_ld<TBC>(br), m1_ld<TBC>(br + 1), m1_ld<TBC>(br + 2), m1_ld<TBC>(br + 3));
    Cv = make_float4(m1_ld<TBC>(cr), m1_ld<TBC>(cr + 1), m1_ld<TBC>(cr + 2), m1_ld<TBC>(cr + 3));
  }
  float dt = 0.f, u = 0.f;
  if (live) {
    const float raw = p.dt_raw[(size_t)b * p.lddt + c] + (p.dt_bias ? p.dt_bias[c] : 0.f);
    dt = raw > 20.f ? raw : log1pf(expf(raw));
    u = p.u[(size_t)b * C + c];
  }
  const float dbu = dt * u;
  auto ex = [](float x) { return sizeof(TO) == 4 ? expf(x) : __expf(x); };
  S.x = ex(-dt * expf(A.x)) * S.x + dbu * Bv.x;
  S.y = ex(-dt * expf(A.y)) * S.y + dbu * Bv.y;
  S.z = ex(-dt * expf(A.z)) * S.z + dbu * Bv.z;
  S.w = ex(-dt * expf(A.w)) * S.w + dbu * Bv.w;
  float acc = S.x * Cv.x + S.y * Cv.y + S.z * Cv.z + S.w * Cv.w;
#pragma unroll
  for (int o = 1; o < LPC; o <<= 1) acc += __shfl_xor_sync(0xffffffffu, acc, o);
  if (ok) *reinterpret_cast<float4*>(st) = S;
  if (live && ks == 0) {
    float y = acc + (p.D ? p.D[c] : 0.f) * u;
    if (p.z) {
      const float zz = m1_ld<TZ>(reinterpret_cast<const TZ*>(p.z) + (size_t)b * p.ldz + c);
      y *= zz / (1.f + expf(-zz));
    }
    m1_st<TO>(reinterpret_cast<TO*>(p.out) + (size_t)b * C + c, y);
  }
}

template <typename TBC, typename TZ, typename TO, int LPC>
void launch_m1_decode(const Mamba1Params& p, int B, cudaStream_t stream) {
  const long long lanes = (long long)p.C * LPC;
  mamba1_decode_kernel<TBC, TZ, TO, LPC><<<dim3((unsigned)((lanes + 255) / 256), B), 256, 0, stream>>>(p);
  SGLB_CUDA_CHECK(cudaGetLastError());
}

template <typename TBC, typename TZ, typename TO>
void dispatch_m1(const Mamba1Params& p, int B, cudaStream_t stream) {
  const int N = p.N;
  if (p.cu_q == nullptr && N % 4 == 0 && N <= 128) {          // decode batches
    if (N <= 4) launch_m1_decode<TBC, TZ, TO, 1>(p, B, stream);
    else if (N <= 8) launch_m1_decode<TBC, TZ, TO, 2>(p, B, stream);
    else if (N <= 16) launch_m1_decode<TBC, TZ, TO, 4>(p, B, stream);
    else if (N <= 32) launch_m1_decode<TBC, TZ, TO, 8>(p, B, stream);
    else if (N <= 64) launch_m1_decode<TBC, TZ, TO, 16>(p, B, stream);
    else launch_m1_decode<TBC, TZ, TO, 32>(p, B, stream);
    return;
  }
  if (N <= 4) launch_m1<TBC, TZ, TO, 4, 1>(p, B, stream);
  else if (N <= 8) launch_m1_small<TBC, TZ, TO, 2>(p, B, stream);
  else if (N <= 16) launch_m1_small<TBC, TZ, TO, 4>(p, B, stream);
  else if (N <= 32) launch_m1_small<TBC, TZ, TO, 8>(p, B, stream);
  else if (N <= 64) launch_m1<TBC, TZ, TO, 8, 8>(p, B, stream);
  else if (N <= 128) launch_m1<TBC, TZ, TO, 8, 16>(p, B, stream);
  else launch_m1<TBC, TZ, TO, 8, 32>(p, B, stream);
}

template <typename TBC, typename TZ>
void dispatch_m1_out(const Mamba1Params& p, int B, bool out_bf16, cudaStream_t stream) {
  if (out_bf16) dispatch_m1<TBC, TZ, __nv_bfloat16>(p, B, stream);
  else dispatch_m1<TBC, TZ, float>(p, B, stream);
}

}  // namespace

void mamba1_scan(const float* u, const float* dt_raw, int lddt, const float* dt_bias, const float* A_log, const void* Bm, const void* Cm, int ldbc, bool bc_bf16,
                 const float* D, const void* z, int ldz, bool z_bf16, float* state, const int* req_slots, const int* seq_lens, const int* cu_q, int B, int C,
                 int N, void* out, bool out_bf16, cudaStream_t stream) {
  if (B <= 0 || C <= 0) return;
  if (N > 256 || B > 65535) throw std::runtime_error("sglb mamba1_scan: state size up to 256");
  Mamba1Params p;
  p.u = u; p.dt_raw = dt_raw; p.lddt = lddt; p.dt_bias = dt_bias; p.A_log = A_log; p.Bm = Bm; p.Cm = Cm; p.ldbc = ldbc; p.D = D; p.z = z; p.ldz = ldz;
  p.state = state; p.req_slots = req_slots; p.seq_lens = seq_lens; p.cu_q = cu_q; p.out = out; p.C = C; p.N = N;
  if (bc_bf16) {
    if (z_bf16) dispatch_m1_out<__nv_bfloat16, __nv_bfloat16>(p, B, out_bf16, stream);
    else dispatch_m1_out<__nv_bfloat16, float>(p, B, out_bf16, stream);
  } else {
    if (z_bf16) dispatch_m1_out<float, __nv_bfloat16>(p, B, out_bf16, stream);
    else dispatch_m1_out<float, float>(p, B, out_bf16, stream);
  }
}

}  // namespace sglb
