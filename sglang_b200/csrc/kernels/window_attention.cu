// Grouped-query attention over a paged cache whose scores carry the position: unit-RMS q / k, a query temperature that grows with the
// position, a tanh score cap, a per-head distance bias, a sliding window and a soft-max sink per head.
//
//   qk_norm_cache_write : per token, every q and k head <- head / sqrt(mean(head^2) + eps); q also times 1 + coef * ln(floor((p + 1) / every) + 1);
//                         k heads go to the first G*D columns of the key plane's row, v to the first G*Dv columns of the value plane's row.
//   window_attention    : s_ij = cap * tanh(q_i . k_j * scale / cap) - slope_h * (i - j), visible for 0 <= i - j < window;
//                         p_ij = exp(s_ij) / (exp(sink_h) + sum_j' exp(s_ij')); o_i = sum_j p_ij v_j.
//                         Options: the sequence's first ``keep_first`` positions stay visible behind the window (their tiles are walked before
//                         the window's); the bias is slope_h * ln(1 + rate_h * (i - j)) instead of linear; the output is multiplied by
//                         sigmoid(gate) per head or per element and by a constant in the epilogue, and may be a column block of a wider buffer.
//   attention_prepare   : per token, q and k RMS-normed over their whole projection times a weight, the first coordinates of every head
//                         rotated by position (pairs half a rotary width apart), v blended with another layer's values, k / v rows to the cache.
//   sigmoid_gate        : o[:, :, :Dv] * sigmoid(gate) * constant, for attention kernels without a gate epilogue.
//
// window_attention mapping: one CTA per (tile of queries, chunk of the heads that share a key head, request): 32 rows = QT queries x HC heads.
// Key tiles of 64 positions are gathered through the page table into shared memory as fp32 with 16-byte global loads where the sizes allow
// (keys padded to a multiple of 4 columns, rows offset by 4 floats so that 16-byte reads of neighbouring keys do not collide).  A warp owns
// 4 rows: for the scores a lane owns 2 keys and reuses each 16-byte key read for its 4 rows; probabilities go through a warp-private shared
// tile; for the output a lane owns CV value columns and reuses each value read for its 4 rows.  The online soft-max starts from (max = sink, sum = 1), which is the sink's term.
// The same kernel serves prompt portions (ragged over cu_q) and decode tokens (cu_q == nullptr: one query per request).  All math is fp32;
// the cache and q are bf16 or fp32.
#include <stdexcept>

#include "common.cuh"
#include "tma_host.h"

namespace sglb {
namespace {

template <typename T> __device__ __forceinline__ float wa_ld(const T* p);
template <> __device__ __forceinline__ float wa_ld<float>(const float* p) { return *p; }
template <> __device__ __forceinline__ float wa_ld<__nv_bfloat16>(const __nv_bfloat16* p) { return __bfloat162float(*p); }
template <typename T> __device__ __forceinline__ void wa_st(T* p, float v);
template <> __device__ __forceinline__ void wa_st<float>(float* p, float v) { *p = v; }
template <> __device__ __forceinline__ void wa_st<__nv_bfloat16>(__nv_bfloat16* p, float v) { *p = __float2bfloat16(v); }

// fp32 serving takes the accurate exponential; bf16 caches the fast one (its error is far below a bf16 rounding)
template <typename T> __device__ __forceinline__ float wa_exp(float x) { return sizeof(T) == 4 ? expf(x) : __expf(x); }

template <typename T>
__global__ void __launch_bounds__(128) qk_norm_cache_write_kernel(const T* __restrict__ qkv, int ld, int H, int G, int D, int Dv,
                                                                  const int* __restrict__ positions, float eps, float coef, int every,
                                                                  T* __restrict__ kc, T* __restrict__ vc, size_t ldc, const int* __restrict__ loc,
                                                                  int normalise, T* __restrict__ q_out, int Dq, int hsk, int hsv) {
  const int t = blockIdx.x;
  const T* row = qkv + (size_t)t * ld;
  const size_t slot = (size_t)loc[t];
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  float temp = 1.f;
  if (coef != 0.f) temp = 1.f + coef * logf((float)((positions[t] + 1) / every) + 1.f);
  for (int hd = warp; hd < H + G; hd += 4) {
    const T* src = row + (size_t)hd * D;
    float ss = 0.f;
    for (int i = lane; i < D; i += 32) {
      const float v = wa_ld<T>(src + i);
      ss += v * v;
    }
    ss = warp_sum(ss);
    float mult = normalise ? 1.0f / sqrtf(ss / (float)D + eps) : 1.f;
    T* dst;
    int width;                      // head stride of the destination: columns beyond D are zero padding
    if (hd < H) {
      dst = q_out + ((size_t)t * H + hd) * Dq;
      width = Dq;
      mult *= temp;
    } else {
      dst = kc + slot * ldc + (size_t)(hd - H) * hsk;
      width = hsk;
    }
    for (int i = lane; i < width; i += 32) wa_st<T>(dst + i, i < D ? wa_ld<T>(src + i) * mult : 0.f);
  }
  const T* vs = row + (size_t)(H + G) * D;
  T* vd = vc + slot * ldc;
  for (int i = threadIdx.x; i < G * hsv; i += 128) {
    const int gh = i / hsv, c = i - gh * hsv;
    wa_st<T>(vd + i, c < Dv ? wa_ld<T>(vs + gh * Dv + c) : 0.f);
  }
}

constexpr int WA_KT = 64;        // keys per tile
constexpr int WA_ROWS = 32;      // (query, head) rows per CTA: 8 warps x 4 rows
constexpr int WA_NT = 256;       // threads per CTA

struct WinAttnParams {
  const void* q; const void* kc; const void* vc; void* out;
  size_t ldc;                                  // elements between cache rows
  const int* page_table; int pt_stride; int page_size;
  const int* req_slots; const int* seq_lens; const int* cu_q;
  const float* slopes; const float* sinks;
  const float* log_rates;                      // non-null: the bias is slopes_h * ln(1 + log_rates_h * distance)
  const void* gate; int ldg; int gate_per_head; // non-null: output times sigmoid(gate[t, h]) or sigmoid(gate[t, h * Dv + c])
  int ldo; float out_scale;                    // output rows of ldo elements; everything times out_scale
  int keep_first;                              // with a window: positions < keep_first stay visible
  int H, G, HG, HC, nchunks, QT, D, Dp, Dv;
  int Dq, hsk, hsv;                            // head strides of q and of the key / value rows (>= D, D, Dv: padded layouts)
  float scale, softcap; int window;
  int vec;                                     // 16-byte gathers: head sizes, row stride and base addresses allow them
};

// 16 bytes of a cache row -> fp32 in shared memory
__device__ __forceinline__ void wa_load16(const float* src, float* dst) { *reinterpret_cast<float4*>(dst) = *reinterpret_cast<const float4*>(src); }
__device__ __forceinline__ void wa_load16(const __nv_bfloat16* src, float* dst) {
  const U4 v = ldg128(src);
  *reinterpret_cast<float4*>(dst) = make_float4(bf16_lo(v.x), bf16_hi(v.x), bf16_lo(v.y), bf16_hi(v.y));
  *reinterpret_cast<float4*>(dst + 4) = make_float4(bf16_lo(v.z), bf16_hi(v.z), bf16_lo(v.w), bf16_hi(v.w));
}

template <typename T, int CV>
__global__ void __launch_bounds__(WA_NT) window_attention_kernel(const WinAttnParams p) {
  extern __shared__ __align__(16) float smem[];
  const int b = blockIdx.z;
  const int q0 = p.cu_q ? p.cu_q[b] : b;
  const int n = p.cu_q ? p.cu_q[b + 1] - q0 : 1;
  const int qt0 = blockIdx.x * p.QT;
  if (qt0 >= n) return;
  const int nq = min(p.QT, n - qt0);
  const int L = p.seq_lens[b];
  const int pos0 = L - n + qt0;                         // position of the tile's first query
  const int g = blockIdx.y / p.nchunks, chunk = blockIdx.y - g * p.nchunks;
  const int hbase = g * p.HG + chunk * p.HC;            // first head of this CTA
  const int nh = min(p.HC, p.HG - chunk * p.HC);        // heads of this CTA
  const int D = p.D, Dp = p.Dp, Dv = p.Dv, HC = p.HC;
  const int ldk = Dp + 4, ldv = 32 * CV;
  float* sQ = smem;                                     // [32][Dp]
  float* sK = sQ + WA_ROWS * Dp;                        // [64][Dp + 4]
  float* sV = sK + WA_KT * ldk;                         // [64][32 * CV]
  float* sP = sV + WA_KT * ldv;                         // [32][64]
  int* sSlot = reinterpret_cast<int*>(sP + WA_ROWS * WA_KT);   // [64]
  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  const T* qg = reinterpret_cast<const T*>(p.q);
  const T* kg = reinterpret_cast<const T*>(p.kc);
  const T* vg = reinterpret_cast<const T*>(p.vc);
  // ---- queries (times the score scale), zero rows where the tile has no query or head
  for (int idx = tid; idx < WA_ROWS * Dp; idx += WA_NT) {
    const int r = idx / Dp, d = idx - r * Dp;
    const int qi = r / HC, hc = r - qi * HC;
    float v = 0.f;
    if (qi < nq && hc < nh && d < D) v = wa_ld<T>(qg + ((size_t)(q0 + qt0 + qi) * p.H + hbase + hc) * p.Dq + d) * p.scale;
    sQ[idx] = v;
  }
  // ---- per-row constants and online soft-max state (the sink is the first term: max = sink, sum = 1)
  const int r0 = warp * 4;
  float m[4], l[4], slope[4], rate[4], O[4][CV];
  int qpos[4];
  bool rowok[4];
#pragma unroll
  for (int r = 0; r < 4; ++r) {
    const int qi = (r0 + r) / HC, hc = (r0 + r) - qi * HC;
    rowok[r] = qi < nq && hc < nh;
    const int h = hbase + (rowok[r] ? hc : 0);
    qpos[r] = pos0 + qi;
    slope[r] = p.slopes ? p.slopes[h] : 0.f;
    rate[r] = p.log_rates ? p.log_rates[h] : 0.f;
    m[r] = p.sinks ? p.sinks[h] : -INFINITY;
    l[r] = p.sinks ? 1.f : 0.f;
#pragma unroll
    for (int c = 0; c < CV; ++c) O[r][c] = 0.f;
  }
  const int klo = p.window > 0 ? max(0, pos0 - p.window + 1) : 0;
  const int kend = pos0 + nq;                           // one past the last key any query of the tile sees
  const int nkeep = min(p.keep_first, klo);             // kept first positions that lie before the window: a segment of their own
  const int* pt = p.page_table + (size_t)p.req_slots[b] * p.pt_stride;
  const float inv_cap = p.softcap > 0.f ? 1.f / p.softcap : 0.f;
  for (int seg = nkeep > 0 ? 0 : 1; seg < 2; ++seg) {
  const int kbeg = seg == 0 ? 0 : klo, khi = seg == 0 ? nkeep : kend;
  for (int kt = kbeg; kt < khi; kt += WA_KT) {
    __syncthreads();                                    // everyone is done with the previous tile (and sQ is written)
    if (tid < WA_KT) {
      const int j = kt + tid;
      sSlot[tid] = j < khi ? pt[j / p.page_size] * p.page_size + j % p.page_size : -1;
    }
    __syncthreads();
    if (p.vec) {
      constexpr int EPV = 16 / (int)sizeof(T);          // elements per 16-byte load
      const int ck = D / EPV, cv = Dv / EPV;
      for (int idx = tid; idx < WA_KT * ck; idx += WA_NT) {
        const int jj = idx / ck, ch = idx - jj * ck;
        const int s = sSlot[jj];
        float* dst = sK + jj * ldk + ch * EPV;
        if (s >= 0) {
          wa_load16(kg + (size_t)s * p.ldc + (size_t)g * p.hsk + ch * EPV, dst);
        } else {
#pragma unroll
          for (int e = 0; e < EPV; ++e) dst[e] = 0.f;
        }
      }
      for (int idx = tid; idx < WA_KT * cv; idx += WA_NT) {
        const int jj = idx / cv, ch = idx - jj * cv;
        const int s = sSlot[jj];
        float* dst = sV + jj * ldv + ch * EPV;
        if (s >= 0) {
          wa_load16(vg + (size_t)s * p.ldc + (size_t)g * p.hsv + ch * EPV, dst);
        } else {
#pragma unroll
          for (int e = 0; e < EPV; ++e) dst[e] = 0.f;
        }
      }
    } else {
      for (int idx = tid; idx < WA_KT * Dp; idx += WA_NT) {
        const int jj = idx / Dp, d = idx - jj * Dp;
        const int s = sSlot[jj];
        sK[jj * ldk + d] = (s >= 0 && d < D) ? wa_ld<T>(kg + (size_t)s * p.ldc + (size_t)g * p.hsk + d) : 0.f;
      }
      for (int idx = tid; idx < WA_KT * ldv; idx += WA_NT) {
        const int jj = idx / ldv, c = idx - jj * ldv;
        const int s = sSlot[jj];
        sV[idx] = (s >= 0 && c < Dv) ? wa_ld<T>(vg + (size_t)s * p.ldc + (size_t)g * p.hsv + c) : 0.f;
      }
    }
    __syncthreads();
    // ---- scores: lane owns keys lane and lane + 32, for the warp's 4 rows
    float acc[2][4];
#pragma unroll
    for (int kk = 0; kk < 2; ++kk)
#pragma unroll
      for (int r = 0; r < 4; ++r) acc[kk][r] = 0.f;
    const float* k0p = sK + lane * ldk;
    const float* k1p = sK + (lane + 32) * ldk;
    for (int d = 0; d < Dp; d += 4) {
      const float4 ka = *reinterpret_cast<const float4*>(k0p + d);
      const float4 kb = *reinterpret_cast<const float4*>(k1p + d);
#pragma unroll
      for (int r = 0; r < 4; ++r) {
        const float4 qv = *reinterpret_cast<const float4*>(sQ + (r0 + r) * Dp + d);
        acc[0][r] += qv.x * ka.x + qv.y * ka.y + qv.z * ka.z + qv.w * ka.w;
        acc[1][r] += qv.x * kb.x + qv.y * kb.y + qv.z * kb.z + qv.w * kb.w;
      }
    }
    // ---- cap, distance bias, mask, online soft-max
#pragma unroll
    for (int r = 0; r < 4; ++r) {
      float s[2];
#pragma unroll
      for (int kk = 0; kk < 2; ++kk) {
        const int j = kt + lane + 32 * kk;
        const int dist = qpos[r] - j;
        float v = acc[kk][r];
        if (p.softcap > 0.f) v = p.softcap * tanhf(v * inv_cap);
        if (p.log_rates) v -= slope[r] * log1pf(rate[r] * (float)max(dist, 0));
        else v -= slope[r] * (float)dist;
        const bool vis = rowok[r] && j < khi && dist >= 0 && (p.window <= 0 || dist < p.window || j < p.keep_first);
        s[kk] = vis ? v : -INFINITY;
      }
      const float mt = warp_max(fmaxf(s[0], s[1]));
      const float mn = fmaxf(m[r], mt);
      const float corr = (m[r] == -INFINITY) ? 0.f : wa_exp<T>(m[r] - mn);
      const float p0 = (s[0] == -INFINITY) ? 0.f : wa_exp<T>(s[0] - mn);
      const float p1 = (s[1] == -INFINITY) ? 0.f : wa_exp<T>(s[1] - mn);
      l[r] = l[r] * corr + warp_sum(p0 + p1);
      m[r] = mn;
#pragma unroll
      for (int c = 0; c < CV; ++c) O[r][c] *= corr;
      sP[(r0 + r) * WA_KT + lane] = p0;
      sP[(r0 + r) * WA_KT + lane + 32] = p1;
    }
    __syncwarp();
    // ---- output: lane owns value columns lane + 32 c
    const int jn = min(WA_KT, khi - kt);
    for (int jj = 0; jj < jn; jj += 4) {
      float4 pr[4];
#pragma unroll
      for (int r = 0; r < 4; ++r) pr[r] = *reinterpret_cast<const float4*>(sP + (r0 + r) * WA_KT + jj);
#pragma unroll
      for (int c = 0; c < CV; ++c) {
        const float v0 = sV[(jj + 0) * ldv + lane + 32 * c], v1 = sV[(jj + 1) * ldv + lane + 32 * c];
        const float v2 = sV[(jj + 2) * ldv + lane + 32 * c], v3 = sV[(jj + 3) * ldv + lane + 32 * c];
#pragma unroll
        for (int r = 0; r < 4; ++r) O[r][c] += pr[r].x * v0 + pr[r].y * v1 + pr[r].z * v2 + pr[r].w * v3;
      }
    }
    __syncwarp();
  }
  }
  T* og = reinterpret_cast<T*>(p.out);
  const T* gg = reinterpret_cast<const T*>(p.gate);
#pragma unroll
  for (int r = 0; r < 4; ++r) {
    if (!rowok[r]) continue;
    const int qi = (r0 + r) / HC, hc = (r0 + r) - qi * HC;
    const size_t tok = (size_t)(q0 + qt0 + qi);
    const int h = hbase + hc;
    float inv = (l[r] > 0.f ? 1.f / l[r] : 0.f) * p.out_scale;
    const T* grow = gg ? gg + tok * p.ldg : nullptr;
    if (grow && p.gate_per_head) inv *= 1.f / (1.f + expf(-wa_ld<T>(grow + h)));
    T* dst = og + tok * p.ldo + (size_t)h * Dv;
#pragma unroll
    for (int c = 0; c < CV; ++c) {
      const int col = lane + 32 * c;
      if (col < Dv) {
        float v = O[r][c] * inv;
        if (grow && !p.gate_per_head) v *= 1.f / (1.f + expf(-wa_ld<T>(grow + (size_t)h * Dv + col)));
        wa_st<T>(dst + col, v);
      }
    }
  }
}

template <typename T, int CV>
void launch_wa(const WinAttnParams& p, int B, int max_q_len, cudaStream_t stream) {
  const size_t smem = sizeof(float) * ((size_t)WA_ROWS * p.Dp + (size_t)WA_KT * (p.Dp + 4) + (size_t)WA_KT * 32 * CV + (size_t)WA_ROWS * WA_KT) +
                      sizeof(int) * WA_KT;
  auto kern = window_attention_kernel<T, CV>;
  if (smem > 48 * 1024) SGLB_CUDA_CHECK(cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));
  dim3 grid((max_q_len + p.QT - 1) / p.QT, p.G * p.nchunks, B);
  kern<<<grid, WA_NT, smem, stream>>>(p);
  SGLB_CUDA_CHECK(cudaGetLastError());
}

template <typename T>
void dispatch_wa(const WinAttnParams& p, int B, int max_q_len, cudaStream_t stream) {
  const int cv = (p.Dv + 31) / 32;
  if (cv <= 1) launch_wa<T, 1>(p, B, max_q_len, stream);
  else if (cv <= 2) launch_wa<T, 2>(p, B, max_q_len, stream);
  else if (cv <= 4) launch_wa<T, 4>(p, B, max_q_len, stream);
  else launch_wa<T, 8>(p, B, max_q_len, stream);
}

// out[t, h, :Dv] = o[t, h, :Dv] * sigmoid(lse[t, h] - sink[h]): a sink joins the soft-max denominator of an attention whose kernel returned the
// log-sum-exp of its scores (exp(lse) / (exp(lse) + exp(sink))); also drops the zero padding behind Dv
__global__ void __launch_bounds__(128) sink_gate_kernel(const __nv_bfloat16* __restrict__ o, int ldo, const float* __restrict__ lse,
                                                        const float* __restrict__ sinks, int H, int Dv, __nv_bfloat16* __restrict__ out) {
  const int row = blockIdx.x;                     // t * H + h
  const float gte = 1.f / (1.f + expf(sinks[row % H] - lse[row]));
  const __nv_bfloat16* src = o + (size_t)row * ldo;
  __nv_bfloat16* dst = out + (size_t)row * Dv;
  for (int i = threadIdx.x; i < Dv; i += 128) dst[i] = __float2bfloat16(__bfloat162float(src[i]) * gte);
}

// out[t, h * Dv + c] = o[t, h, c] * sigmoid(gate) * scale, c < Dv: gate [t, h] (per head) or [t, h * Dv + c]; o rows of ldo_in elements per head
template <typename T>
__global__ void __launch_bounds__(128) sigmoid_gate_kernel(const T* __restrict__ o, int hs, const T* __restrict__ gate, int ldg, int per_head, int H, int Dv,
                                                           float scale, T* __restrict__ out, int ldo) {
  const int t = blockIdx.x / H, h = blockIdx.x - t * H;
  const T* src = o + (size_t)blockIdx.x * hs;
  const T* g = gate + (size_t)t * ldg;
  T* dst = out + (size_t)t * ldo + (size_t)h * Dv;
  const float gh = per_head ? scale / (1.f + expf(-wa_ld<T>(g + h))) : 0.f;
  for (int i = threadIdx.x; i < Dv; i += 128) {
    const float m = per_head ? gh : scale / (1.f + expf(-wa_ld<T>(g + (size_t)h * Dv + i)));
    wa_st<T>(dst + i, wa_ld<T>(src + i) * m);
  }
}

// out[t, h * Dv + c] = the head o[t, h, :Dv] (rows of hs elements) times sigmoid(lse[t, h] - sink[h]) (lse null: times 1), turned over its whole
// width by -+ position * inv_freq[m]: pair m = columns (m, m + Dv/2) or, inter, (2m, 2m + 1).  Angle, sine and cosine fp32.  One CTA per token:
// a thread owns a pair index and walks the heads, so that the sine and cosine of an angle are computed once for all heads.
template <typename T>
__global__ void __launch_bounds__(128) rotate_heads_kernel(const T* __restrict__ o, int hs, const int* __restrict__ positions, const float* __restrict__ inv_freq,
                                                           int H, int Dv, int inter, float sign, const float* __restrict__ lse,
                                                           const float* __restrict__ sinks, T* __restrict__ out) {
  const int t = blockIdx.x;
  const int hv = Dv >> 1;
  const int pw = hv >= 128 ? 128 : hv;               // threads across the pairs of a head; the others of the CTA take further heads
  const int hstep = 128 / pw, h0 = threadIdx.x / pw;
  if (h0 >= hstep) return;
  const float pos = (float)positions[t];
  for (int m = threadIdx.x - h0 * pw; m < hv; m += pw) {
    float sn, cs;
    sincosf(pos * inv_freq[m], &sn, &cs);
    sn *= sign;
    const int ia = inter ? 2 * m : m, ib = inter ? 2 * m + 1 : m + hv;
    for (int h = h0; h < H; h += hstep) {
      const size_t row = (size_t)t * H + h;
      const float gte = lse ? 1.f / (1.f + expf(sinks[h] - lse[row])) : 1.f;
      const T* src = o + row * hs;
      T* dst = out + row * Dv;
      const float a = wa_ld<T>(src + ia) * gte, b = wa_ld<T>(src + ib) * gte;
      wa_st<T>(dst + ia, a * cs - b * sn);
      wa_st<T>(dst + ib, b * cs + a * sn);
    }
  }
}

// rows of raw scores -> soft-max weights under a causal limit, for attention that runs as two matrix products around this kernel:
// s fp32 [R, n], row r = h * tq + i belongs to query i of its request portion and sees keys j <= first + i;
// out[r, j] = exp(scale * s[r, j] - m) / sum over the visible keys (0 beyond them), m the row's largest visible scaled score.  One CTA per row.
template <typename TO, int KEEP>
__global__ void __launch_bounds__(256) causal_softmax_kernel(const float* __restrict__ s, TO* __restrict__ out, int tq, int n, int first, float scale) {
  __shared__ float red[8];
  const size_t row = blockIdx.x;
  const int lim = min(n, first + (int)(row % tq) + 1);
  const float* sr = s + row * n;
  TO* orow = out + row * n;
  float v[KEEP > 0 ? KEEP : 1];                  // KEEP > 0: the row's visible scores stay in registers (n <= 256 * KEEP), read and exponentiated once
  float m = -INFINITY;
  if (KEEP > 0) {
#pragma unroll
    for (int k = 0; k < KEEP; ++k) {
      const int j = threadIdx.x + k * 256;
      v[k] = j < lim ? sr[j] * scale : -INFINITY;
      m = fmaxf(m, v[k]);
    }
  } else {
    for (int j = threadIdx.x; j < lim; j += 256) m = fmaxf(m, sr[j] * scale);
  }
  m = warp_max(m);
  if ((threadIdx.x & 31) == 0) red[threadIdx.x >> 5] = m;
  __syncthreads();
  m = red[0];
#pragma unroll
  for (int i = 1; i < 8; ++i) m = fmaxf(m, red[i]);
  __syncthreads();
  float l = 0.f;
  if (KEEP > 0) {
#pragma unroll
    for (int k = 0; k < KEEP; ++k) {
      v[k] = wa_exp<TO>(v[k] - m);               // exp(-inf) = 0 beyond the limit
      l += v[k];
    }
  } else {
    for (int j = threadIdx.x; j < lim; j += 256) l += wa_exp<TO>(sr[j] * scale - m);
  }
  l = warp_sum(l);
  if ((threadIdx.x & 31) == 0) red[threadIdx.x >> 5] = l;
  __syncthreads();
  l = 0.f;
#pragma unroll
  for (int i = 0; i < 8; ++i) l += red[i];
  const float inv = 1.f / l;
  if (KEEP > 0) {
#pragma unroll
    for (int k = 0; k < KEEP; ++k) {
      const int j = threadIdx.x + k * 256;
      if (j < n) wa_st<TO>(orow + j, v[k] * inv);
    }
  } else {
    for (int j = threadIdx.x; j < n; j += 256) wa_st<TO>(orow + j, j < lim ? wa_exp<TO>(sr[j] * scale - m) * inv : 0.f);
  }
}

struct PrepParams {
  const void* qkv; int ld;                     // rows [q (H*D) | k (G*D) | v (G*Dv) | ...]
  int H, G, D, Dv;
  const int* positions;
  const void* qw; const void* kw; float eps;   // projection-wide RMS norm weights (null: no norm)
  const float* inv_freq; int half;             // rotary frequencies (null: no rotation); pairs (i, i + half), i < half
  const void* v_first; int ldvf; float lam;    // values to blend with (null: none)
  const float* v_inv_freq; int v_inter;        // values rotated over their whole head (null: no): pairs (m, m + Dv/2) or, v_inter, (2m, 2m + 1)
  void* kc; void* vc; size_t ldc; const int* loc;
  void* q_out; int Dq, hsk, hsv;               // head strides of q, key rows, value rows (>= D, D, Dv: zero padding behind the values)
};

template <typename T>
__global__ void __launch_bounds__(128) attention_prepare_kernel(const PrepParams p) {
  __shared__ float red[8];
  const int t = blockIdx.x;
  const int tid = threadIdx.x;
  const T* row = reinterpret_cast<const T*>(p.qkv) + (size_t)t * p.ld;
  const size_t slot = (size_t)p.loc[t];
  const int nq = p.H * p.D, nk = p.G * p.D;
  float rq = 1.f, rk = 1.f;
  if (p.qw) {                                   // mean of squares over the whole q projection, then the whole k projection
    float sq = 0.f, sk = 0.f;
    for (int i = tid; i < nq; i += 128) { const float v = wa_ld<T>(row + i); sq += v * v; }
    for (int i = tid; i < nk; i += 128) { const float v = wa_ld<T>(row + nq + i); sk += v * v; }
    sq = warp_sum(sq); sk = warp_sum(sk);
    if ((tid & 31) == 0) { red[tid >> 5] = sq; red[4 + (tid >> 5)] = sk; }
    __syncthreads();
    rq = 1.0f / sqrtf((red[0] + red[1] + red[2] + red[3]) / (float)nq + p.eps);
    rk = 1.0f / sqrtf((red[4] + red[5] + red[6] + red[7]) / (float)nk + p.eps);
  }
  const float pos = (float)p.positions[t];
  const T* qw = reinterpret_cast<const T*>(p.qw);
  const T* kw = reinterpret_cast<const T*>(p.kw);
  T* qo = reinterpret_cast<T*>(p.q_out) + (size_t)t * p.H * p.Dq;
  T* ko = reinterpret_cast<T*>(p.kc) + slot * p.ldc;
  T* vo = reinterpret_cast<T*>(p.vc) + slot * p.ldc;
  const int half = p.inv_freq ? p.half : 0;
  // q heads then k heads: element (head, i) of the padded destination
  const int total = p.H * p.Dq + p.G * p.hsk;
  for (int idx = tid; idx < total; idx += 128) {
    const bool isq = idx < p.H * p.Dq;
    const int rel = isq ? idx : idx - p.H * p.Dq;
    const int hs = isq ? p.Dq : p.hsk;
    const int hd = rel / hs, i = rel - hd * hs;
    T* dst = (isq ? qo : ko) + rel;
    if (i >= p.D) { wa_st<T>(dst, 0.f); continue; }
    const T* src = row + (isq ? 0 : nq) + hd * p.D;
    const T* w = isq ? qw : kw;
    const float r = isq ? rq : rk;
    auto val = [&](int c) { const float v = wa_ld<T>(src + c) * r; return w ? v * wa_ld<T>(w + hd * p.D + c) : v; };
    float v = val(i);
    if (i < 2 * half) {
      const int fi = i < half ? i : i - half;
      float sn, cs;
      sincosf(pos * p.inv_freq[fi], &sn, &cs);
      const float other = val(i < half ? i + half : i - half);
      v = i < half ? v * cs - other * sn : v * cs + other * sn;
    }
    wa_st<T>(dst, v);
  }
  const T* vs = row + nq + nk;
  const T* vf = p.v_first ? reinterpret_cast<const T*>(p.v_first) + (size_t)t * p.ldvf : nullptr;
  const int hv = p.Dv / 2;
  for (int idx = tid; idx < p.G * p.hsv; idx += 128) {
    const int gh = idx / p.hsv, c = idx - gh * p.hsv;
    float v = 0.f;
    if (c < p.Dv) {
      auto val = [&](int cc) {
        const float x = wa_ld<T>(vs + gh * p.Dv + cc);
        return vf ? (1.f - p.lam) * x + p.lam * wa_ld<T>(vf + gh * p.Dv + cc) : x;
      };
      v = val(c);
      if (p.v_inv_freq) {
        const bool first = p.v_inter ? (c & 1) == 0 : c < hv;
        const int m = p.v_inter ? c >> 1 : (first ? c : c - hv);
        const float other = val(p.v_inter ? (c ^ 1) : (first ? c + hv : c - hv));
        float sn, cs;
        sincosf(pos * p.v_inv_freq[m], &sn, &cs);
        v = first ? v * cs - other * sn : v * cs + other * sn;
      }
    }
    wa_st<T>(vo + idx, v);
  }
}

// two neighbouring elements at once (4-byte or 8-byte accesses)
__device__ __forceinline__ float2 wa_ld2(const float* p) { return *reinterpret_cast<const float2*>(p); }
__device__ __forceinline__ float2 wa_ld2(const __nv_bfloat16* p) {
  const uint32_t v = *reinterpret_cast<const uint32_t*>(p);
  return make_float2(bf16_lo(v), bf16_hi(v));
}
__device__ __forceinline__ void wa_st2(float* p, float a, float b) { *reinterpret_cast<float2*>(p) = make_float2(a, b); }
__device__ __forceinline__ void wa_st2(__nv_bfloat16* p, float a, float b) { *reinterpret_cast<uint32_t*>(p) = pack_bf16(a, b); }

// the same work two columns at a time: even head sizes, rotary half-width and strides.  A rotated item is the four numbers
// (i, i + 1, i + half, i + half + 1) of a head: two angles, each pair rotated once; a tail item is two unrotated columns (or zero padding).
template <typename T>
__global__ void __launch_bounds__(128) attention_prepare_vec_kernel(const PrepParams p) {
  __shared__ float red[8];
  const int t = blockIdx.x;
  const int tid = threadIdx.x;
  const T* row = reinterpret_cast<const T*>(p.qkv) + (size_t)t * p.ld;
  const size_t slot = (size_t)p.loc[t];
  const int nq = p.H * p.D, nk = p.G * p.D;
  float rq = 1.f, rk = 1.f;
  if (p.qw) {
    float sq = 0.f, sk = 0.f;
    for (int i = 2 * tid; i < nq; i += 256) { const float2 v = wa_ld2(row + i); sq += v.x * v.x + v.y * v.y; }
    for (int i = 2 * tid; i < nk; i += 256) { const float2 v = wa_ld2(row + nq + i); sk += v.x * v.x + v.y * v.y; }
    sq = warp_sum(sq); sk = warp_sum(sk);
    if ((tid & 31) == 0) { red[tid >> 5] = sq; red[4 + (tid >> 5)] = sk; }
    __syncthreads();
    rq = 1.0f / sqrtf((red[0] + red[1] + red[2] + red[3]) / (float)nq + p.eps);
    rk = 1.0f / sqrtf((red[4] + red[5] + red[6] + red[7]) / (float)nk + p.eps);
  }
  const float pos = (float)p.positions[t];
  const T* qw = reinterpret_cast<const T*>(p.qw);
  const T* kw = reinterpret_cast<const T*>(p.kw);
  T* qo = reinterpret_cast<T*>(p.q_out) + (size_t)t * p.H * p.Dq;
  T* ko = reinterpret_cast<T*>(p.kc) + slot * p.ldc;
  T* vo = reinterpret_cast<T*>(p.vc) + slot * p.ldc;
  const int half = p.inv_freq ? p.half : 0;
  const int nrot = half / 2;                              // rotated items per head
  const int per_q = nrot + (p.Dq - 2 * half) / 2, per_k = nrot + (p.hsk - 2 * half) / 2;
  const int total = p.H * per_q + p.G * per_k;
  for (int idx = tid; idx < total; idx += 128) {
    const bool isq = idx < p.H * per_q;
    const int rel = isq ? idx : idx - p.H * per_q;
    const int per = isq ? per_q : per_k, hs = isq ? p.Dq : p.hsk;
    const int hd = rel / per, it = rel - hd * per;
    const T* src = row + (isq ? 0 : nq) + hd * p.D;
    const T* w = isq ? qw : kw;
    const float r = isq ? rq : rk;
    T* dst = (isq ? qo : ko) + (size_t)hd * hs;
    auto val2 = [&](int c) {
      float2 v = wa_ld2(src + c);
      v.x *= r; v.y *= r;
      if (w) { const float2 ww = wa_ld2(w + hd * p.D + c); v.x *= ww.x; v.y *= ww.y; }
      return v;
    };
    if (it < nrot) {
      const int i = 2 * it;
      const float2 a = val2(i), b = val2(i + half);
      float s0, c0, s1, c1;
      sincosf(pos * p.inv_freq[i], &s0, &c0);
      sincosf(pos * p.inv_freq[i + 1], &s1, &c1);
      wa_st2(dst + i, a.x * c0 - b.x * s0, a.y * c1 - b.y * s1);
      wa_st2(dst + i + half, b.x * c0 + a.x * s0, b.y * c1 + a.y * s1);
    } else {
      const int c = 2 * half + 2 * (it - nrot);
      if (c < p.D) { const float2 v = val2(c); wa_st2(dst + c, v.x, v.y); }
      else wa_st2(dst + c, 0.f, 0.f);
    }
  }
  const T* vs = row + nq + nk;
  const T* vf = p.v_first ? reinterpret_cast<const T*>(p.v_first) + (size_t)t * p.ldvf : nullptr;
  const int hv2 = p.hsv / 2;
  for (int idx = tid; idx < p.G * hv2; idx += 128) {
    const int gh = idx / hv2, c = 2 * (idx - gh * hv2);
    float2 v = make_float2(0.f, 0.f);
    if (c < p.Dv) {
      auto val2 = [&](int cc) {
        float2 x = wa_ld2(vs + gh * p.Dv + cc);
        if (vf) {
          const float2 f = wa_ld2(vf + gh * p.Dv + cc);
          x.x = (1.f - p.lam) * x.x + p.lam * f.x;
          x.y = (1.f - p.lam) * x.y + p.lam * f.y;
        }
        return x;
      };
      v = val2(c);
      if (p.v_inv_freq && p.v_inter) {            // (c, c + 1) is pair c / 2
        float sn, cs;
        sincosf(pos * p.v_inv_freq[c >> 1], &sn, &cs);
        v = make_float2(v.x * cs - v.y * sn, v.y * cs + v.x * sn);
      } else if (p.v_inv_freq) {                  // columns c, c + 1 belong to two pairs whose partners lie half a head away (Dv / 2 even)
        const int hv = p.Dv / 2;
        const bool first = c < hv;
        const int m = first ? c : c - hv;
        const float2 o = val2(first ? c + hv : c - hv);
        float s0, c0, s1, c1;
        sincosf(pos * p.v_inv_freq[m], &s0, &c0);
        sincosf(pos * p.v_inv_freq[m + 1], &s1, &c1);
        v = first ? make_float2(v.x * c0 - o.x * s0, v.y * c1 - o.y * s1) : make_float2(v.x * c0 + o.x * s0, v.y * c1 + o.y * s1);
      }
    }
    wa_st2(vo + (size_t)gh * p.hsv + c, v.x, v.y);
  }
}

}  // namespace

void sigmoid_gate(const void* o, int head_stride, const void* gate, int ldg, bool per_head, bool bf16, int T, int H, int Dv, float scale, void* out, int ldo,
                  cudaStream_t stream) {
  if (T <= 0 || H <= 0) return;
  if (bf16)
    sigmoid_gate_kernel<__nv_bfloat16><<<T * H, 128, 0, stream>>>((const __nv_bfloat16*)o, head_stride, (const __nv_bfloat16*)gate, ldg, per_head ? 1 : 0, H, Dv,
                                                                  scale, (__nv_bfloat16*)out, ldo);
  else
    sigmoid_gate_kernel<float><<<T * H, 128, 0, stream>>>((const float*)o, head_stride, (const float*)gate, ldg, per_head ? 1 : 0, H, Dv, scale, (float*)out, ldo);
  SGLB_CUDA_CHECK(cudaGetLastError());
}

void attention_prepare(const void* qkv, int ld, bool bf16, int T, int H, int G, int D, int Dv, const int* positions, const void* q_norm_w, const void* k_norm_w,
                       float eps, const float* inv_freq, int half, const void* v_first, int ldvf, float lam, void* kc, void* vc, size_t ldc, const int* loc,
                       void* q_out, int pad, const float* v_inv_freq, bool v_interleaved, cudaStream_t stream) {
  if (T <= 0) return;
  PrepParams p;
  p.v_inv_freq = v_inv_freq; p.v_inter = v_interleaved ? 1 : 0;
  p.qkv = qkv; p.ld = ld; p.H = H; p.G = G; p.D = D; p.Dv = Dv; p.positions = positions; p.qw = q_norm_w; p.kw = k_norm_w; p.eps = eps;
  p.inv_freq = inv_freq; p.half = half; p.v_first = v_first; p.ldvf = ldvf; p.lam = lam; p.kc = kc; p.vc = vc; p.ldc = ldc; p.loc = loc; p.q_out = q_out;
  p.Dq = pad > 0 ? pad : D; p.hsk = pad > 0 ? pad : D; p.hsv = pad > 0 ? pad : Dv;
  const size_t a2 = bf16 ? 4 : 8;          // bytes of a two-element access
  auto al = [&](const void* q) { return q == nullptr || ((uintptr_t)q % a2) == 0; };
  const bool vec = D % 2 == 0 && Dv % 2 == 0 && half % 2 == 0 && ld % 2 == 0 && ldc % 2 == 0 && p.Dq % 2 == 0 && p.hsk % 2 == 0 && p.hsv % 2 == 0 &&
                   (v_inv_freq == nullptr || v_interleaved || Dv % 4 == 0) && (v_first == nullptr || ldvf % 2 == 0) && al(qkv) && al(kc) && al(vc) && al(q_out) && al(v_first) && al(q_norm_w) && al(k_norm_w);
  if (vec) {
    if (bf16) attention_prepare_vec_kernel<__nv_bfloat16><<<T, 128, 0, stream>>>(p);
    else attention_prepare_vec_kernel<float><<<T, 128, 0, stream>>>(p);
  } else {
    if (bf16) attention_prepare_kernel<__nv_bfloat16><<<T, 128, 0, stream>>>(p);
    else attention_prepare_kernel<float><<<T, 128, 0, stream>>>(p);
  }
  SGLB_CUDA_CHECK(cudaGetLastError());
}

void rotate_heads(const void* o, int head_stride, bool bf16, const int* positions, const float* inv_freq, int T, int H, int Dv, bool interleaved, bool inverse,
                  const float* lse, const float* sinks, void* out, cudaStream_t stream) {
  if (T <= 0 || H <= 0) return;
  const float sign = inverse ? -1.f : 1.f;
  const unsigned grid = (unsigned)T;
  if (bf16)
    rotate_heads_kernel<__nv_bfloat16><<<grid, 128, 0, stream>>>((const __nv_bfloat16*)o, head_stride, positions, inv_freq, H, Dv, interleaved ? 1 : 0, sign,
                                                                  lse, sinks, (__nv_bfloat16*)out);
  else
    rotate_heads_kernel<float><<<grid, 128, 0, stream>>>((const float*)o, head_stride, positions, inv_freq, H, Dv, interleaved ? 1 : 0, sign, lse, sinks,
                                                          (float*)out);
  SGLB_CUDA_CHECK(cudaGetLastError());
}

void causal_softmax(const float* scores, void* out, bool out_bf16, int rows, int tq, int n, int first, float scale, cudaStream_t stream) {
  if (rows <= 0 || n <= 0) return;
#define SGLB_CSM(TO, KEEP) causal_softmax_kernel<TO, KEEP><<<rows, 256, 0, stream>>>(scores, (TO*)out, tq, n, first, scale)
  if (out_bf16) {
    if (n <= 1024) SGLB_CSM(__nv_bfloat16, 4); else if (n <= 2048) SGLB_CSM(__nv_bfloat16, 8); else if (n <= 4096) SGLB_CSM(__nv_bfloat16, 16); else SGLB_CSM(__nv_bfloat16, 0);
  } else {
    if (n <= 1024) SGLB_CSM(float, 4); else if (n <= 2048) SGLB_CSM(float, 8); else if (n <= 4096) SGLB_CSM(float, 16); else SGLB_CSM(float, 0);
  }
#undef SGLB_CSM
  SGLB_CUDA_CHECK(cudaGetLastError());
}

void attention_sink_gate(const void* o, int ldo, const float* lse, const float* sinks, int rows, int H, int Dv, void* out, cudaStream_t stream) {
  if (rows <= 0) return;
  sink_gate_kernel<<<rows, 128, 0, stream>>>((const __nv_bfloat16*)o, ldo, lse, sinks, H, Dv, (__nv_bfloat16*)out);
  SGLB_CUDA_CHECK(cudaGetLastError());
}

void qk_norm_cache_write(const void* qkv, int ld, bool bf16, int T, int H, int G, int D, int Dv, const int* positions, float eps, float coef, int every,
                         void* kc, void* vc, size_t ldc, const int* loc, bool normalise, void* q_out, int pad, cudaStream_t stream) {
  if (T <= 0) return;
  const int Dq = pad > 0 ? pad : D, hsk = pad > 0 ? pad : D, hsv = pad > 0 ? pad : Dv;      // pad: every head occupies ``pad`` columns, zeros behind its values
  if (bf16)
    qk_norm_cache_write_kernel<__nv_bfloat16><<<T, 128, 0, stream>>>((const __nv_bfloat16*)qkv, ld, H, G, D, Dv, positions, eps, coef, every,
                                                                     (__nv_bfloat16*)kc, (__nv_bfloat16*)vc, ldc, loc, normalise ? 1 : 0, (__nv_bfloat16*)q_out, Dq, hsk, hsv);
  else
    qk_norm_cache_write_kernel<float><<<T, 128, 0, stream>>>((const float*)qkv, ld, H, G, D, Dv, positions, eps, coef, every, (float*)kc, (float*)vc, ldc,
                                                             loc, normalise ? 1 : 0, (float*)q_out, Dq, hsk, hsv);
  SGLB_CUDA_CHECK(cudaGetLastError());
}

void window_attention(const void* q, const void* kc, const void* vc, bool bf16, size_t ldc, int H, int G, int D, int Dv, const int* page_table,
                      int pt_stride, int page_size, const int* req_slots, const int* seq_lens, const int* cu_q, int B, int max_q_len, float scale,
                      float softcap, int window, const float* slopes, const float* sinks, void* out, int pad, int keep_first, const float* log_rates,
                      const void* gate, int ldg, bool gate_per_head, int ldo, float out_scale, cudaStream_t stream) {
  if (B <= 0 || max_q_len <= 0) return;
  if (D > 256 || Dv > 256 || B > 65535 || H % G) throw std::runtime_error("sglb window_attention: head sizes up to 256, heads a multiple of key heads");
  WinAttnParams p;
  p.q = q; p.kc = kc; p.vc = vc; p.out = out; p.ldc = ldc;
  p.page_table = page_table; p.pt_stride = pt_stride; p.page_size = page_size;
  p.req_slots = req_slots; p.seq_lens = seq_lens; p.cu_q = cu_q; p.slopes = slopes; p.sinks = sinks;
  p.log_rates = slopes ? log_rates : nullptr; p.gate = gate; p.ldg = ldg; p.gate_per_head = gate_per_head ? 1 : 0; p.ldo = ldo; p.out_scale = out_scale;
  p.keep_first = window > 0 ? std::max(0, keep_first) : 0;
  p.H = H; p.G = G; p.HG = H / G;
  p.HC = std::min(p.HG, WA_ROWS);
  p.nchunks = (p.HG + p.HC - 1) / p.HC;
  p.QT = std::max(1, WA_ROWS / p.HC);
  p.D = D; p.Dp = (D + 3) / 4 * 4; p.Dv = Dv;
  p.Dq = pad > 0 ? pad : D; p.hsk = pad > 0 ? pad : D; p.hsv = pad > 0 ? pad : Dv;
  p.scale = scale; p.softcap = softcap; p.window = window;
  const size_t esz = bf16 ? 2 : 4;
  const int epv = (int)(16 / esz);
  p.vec = (D % epv == 0 && Dv % epv == 0 && p.hsk % epv == 0 && p.hsv % epv == 0 && (ldc * esz) % 16 == 0 && ((uintptr_t)kc % 16) == 0 && ((uintptr_t)vc % 16) == 0) ? 1 : 0;
  if (p.G * p.nchunks > 65535) throw std::runtime_error("sglb window_attention: too many heads for one launch");
  if (bf16) dispatch_wa<__nv_bfloat16>(p, B, max_q_len, stream);
  else dispatch_wa<float>(p, B, max_q_len, stream);
}

}  // namespace sglb
