// Absorbed latent attention over a paged cache, with a sliding window and per-head soft-max sinks.
//
// The cache holds ONE latent row c_j of R numbers per token; keys and values of all heads are linear maps of it, and those maps are applied
// outside this kernel (query side: q~ = W_uk^T q; output side: W_uv o~).  What runs here is multi-query attention over the latent rows:
//     p_j  = exp(scale * q~ . c_j - m) / (sum_j' exp(scale * q~ . c_j' - m) + exp(sink - m))    for keys 0 <= i - j < window
//     o~   = sum_j p_j c_j
// One kernel serves prompt portions (QT = 8 queries of a request per CTA) and decode (QT = 1).  A CTA owns QT consecutive queries x HG heads
// (HG chosen on the host so that the tile fits shared memory).  It walks the keys its queries can see — the window plus QT - 1 — in tiles of
// 32: the tile's latent rows go to shared memory once (fp32, row stride R + 1) and are used by every (query, head) pair as key AND as value.
// A warp owns whole pairs: lane = key for the scores (R multiply-adds against a broadcast query), lane = latent column for the output
// (probabilities broadcast by shuffle), running max / sum in registers, output accumulator in shared memory.  The sink is the initial
// state of the running soft-max (m = sink, l = 1, o = 0), so it is counted once and needs no branch at the end.  All arithmetic is fp32.
#include "common.cuh"
#include "tma_host.h"

namespace sglb {
namespace {

constexpr int KT = 32;           // keys per tile (= lanes)
constexpr int NW = 8;            // warps per CTA

template <typename T> __device__ __forceinline__ float ldc(const T* p);
template <> __device__ __forceinline__ float ldc<float>(const float* p) { return *p; }
template <> __device__ __forceinline__ float ldc<__nv_bfloat16>(const __nv_bfloat16* p) { return __bfloat162float(*p); }
template <typename T> __device__ __forceinline__ void stc(T* p, float v);
template <> __device__ __forceinline__ void stc<float>(float* p, float v) { *p = v; }
template <> __device__ __forceinline__ void stc<__nv_bfloat16>(__nv_bfloat16* p, float v) { *p = __float2bfloat16(v); }

struct LatentParams {
  const float* q; float* out;                 // [T, H, R]
  const void* cache; int ldc;                 // rows of ldc elements, the first R are the latent
  const int* page_table; int pt_stride; int page_size;
  const int* req_slots; const int* seq_lens; const int* cu_q;
  const float* sinks;
  int H, R, RP, HG, window;                    // RP: row stride of the key tile in shared memory (R + 4 when R % 4 == 0, else R + 1)
  int Rv;                                      // leading columns of a row that are its value (<= R; the rest only scores); out rows are Rv wide
  float scale;
  int vec8;
  int nsplit;                                  // decode only: the visible keys of a request are cut into nsplit ranges, one CTA each
  float* part_o; float* part_ml;               // [T, nsplit, H, R] unnormalised outputs and [T, nsplit, H, 2] (running max, sum)
};

template <typename TCache, int QT, int PP>
__global__ void __launch_bounds__(NW * 32) latent_attention_kernel(const LatentParams p) {
  extern __shared__ __align__(16) float sm[];
  const int b = blockIdx.y;
  const int qbase = p.cu_q ? p.cu_q[b] : b;
  const int n = p.cu_q ? p.cu_q[b + 1] - qbase : 1;
  const int split = QT == 1 ? blockIdx.x : 0;          // decode: blockIdx.x is the key range, prompts: the query tile
  const int t0 = QT == 1 ? 0 : blockIdx.x * QT;
  if (t0 >= n) return;
  const int nq = min(QT, n - t0);
  const int L = p.seq_lens[b];
  const int pos0 = L - n + t0;                 // position of the CTA's first query
  const int h0 = blockIdx.z * p.HG;
  const int nh = min(p.HG, p.H - h0);
  const int R = p.R, RP = p.RP, Rv = p.Rv;
  const bool vec = (R & 3) == 0;               // 16-byte shared-memory loads of queries and latent rows
  const bool vec8 = p.vec8 != 0;               // 16-byte global loads of cache rows (rank, row stride and base allow it)
  const int P = nq * nh;                       // (query, head) pairs of this CTA: pair = qi * nh + hi
  float* s_p = sm;                             // [NW][4][KT] probabilities of the pairs a warp is working on (first: keeps 16-byte alignment)
  float* s_q = s_p + NW * 4 * KT;              // [QT * HG][R]
  float* s_o = s_q + QT * p.HG * R;            // [QT * HG][R]
  float* s_c = s_o + QT * p.HG * R;            // [KT][R + 1]
  int* s_slot = (int*)(s_c + KT * RP);         // [KT]
  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  for (int idx = tid; idx < P * R; idx += NW * 32) {
    const int pr = idx / R, r = idx - pr * R;
    const int qi = pr / nh, hi = pr - qi * nh;
    s_q[idx] = p.q[((size_t)(qbase + t0 + qi) * p.H + h0 + hi) * R + r];
    s_o[idx] = 0.f;
  }
  // running soft-max state of the pairs this warp owns (pair = warp + k * NW)
  constexpr int PPW_MAX = 16;
  float m_run[PPW_MAX], l_run[PPW_MAX];
#pragma unroll
  for (int k = 0; k < PPW_MAX; ++k) {
    const int pr = warp + k * NW;
    const bool sink_here = p.sinks && pr < P && split == 0;          // the sink is counted once: by the first key range
    m_run[k] = sink_here ? p.sinks[h0 + pr % nh] : -INFINITY;
    l_run[k] = sink_here ? 1.f : 0.f;
  }
  int last = pos0 + nq - 1;
  int first = p.window > 0 ? max(0, pos0 - p.window + 1) : 0;
  if (QT == 1 && p.nsplit > 1) {
    const int per = (last - first + p.nsplit) / p.nsplit;             // ceil((last - first + 1) / nsplit)
    first += split * per;
    last = min(last, first + per - 1);
  }
  const int* pt = p.page_table + (size_t)p.req_slots[b] * p.pt_stride;
  const TCache* cache = (const TCache*)p.cache;
  for (int k0 = first; k0 <= last; k0 += KT) {
    __syncthreads();                           // the previous tile is consumed (and s_q / s_o are initialised)
    if (tid < KT) {
      const int kp = k0 + tid;
      s_slot[tid] = kp <= last ? pt[kp / p.page_size] * p.page_size + kp % p.page_size : -1;
    }
    __syncthreads();
    if (vec8) {                                // 16-byte global loads: 8 bf16 or 2 x 4 fp32 latent values per thread and step
      const int R8 = R >> 3;
      for (int idx = tid; idx < KT * R8; idx += NW * 32) {
        const int k = idx / R8, r = (idx - k * R8) << 3;
        const int slot = s_slot[k];
        float v[8];
        if (slot < 0) {
#pragma unroll
          for (int i = 0; i < 8; ++i) v[i] = 0.f;
        } else if (sizeof(TCache) == 2) {
          const U4 w = ldg128(cache + (size_t)slot * p.ldc + r);
          v[0] = bf16_lo(w.x); v[1] = bf16_hi(w.x); v[2] = bf16_lo(w.y); v[3] = bf16_hi(w.y);
          v[4] = bf16_lo(w.z); v[5] = bf16_hi(w.z); v[6] = bf16_lo(w.w); v[7] = bf16_hi(w.w);
        } else {
          const float4 w0 = *reinterpret_cast<const float4*>(cache + (size_t)slot * p.ldc + r);
          const float4 w1 = *reinterpret_cast<const float4*>(cache + (size_t)slot * p.ldc + r + 4);
          v[0] = w0.x; v[1] = w0.y; v[2] = w0.z; v[3] = w0.w; v[4] = w1.x; v[5] = w1.y; v[6] = w1.z; v[7] = w1.w;
        }
        float4* dst = reinterpret_cast<float4*>(s_c + k * RP + r);
        dst[0] = make_float4(v[0], v[1], v[2], v[3]);
        dst[1] = make_float4(v[4], v[5], v[6], v[7]);
      }
    } else {
      for (int idx = tid; idx < KT * R; idx += NW * 32) {
        const int k = idx / R, r = idx - k * R;
        const int slot = s_slot[k];
        s_c[k * RP + r] = slot >= 0 ? ldc<TCache>(cache + (size_t)slot * p.ldc + r) : 0.f;
      }
    }
    __syncthreads();
    const int kp = k0 + lane;
    // the warp's pairs go four at a time: one latent value from shared memory feeds four score sums, one probability shuffle four columns
#pragma unroll
    for (int g0 = 0; g0 < PPW_MAX; g0 += PP) {
      if (warp + g0 * NW >= P) break;
      bool act[PP], vis[PP];
      const float* qv[PP];
      bool any = false;
#pragma unroll
      for (int u = 0; u < PP; ++u) {
        const int pr = warp + (g0 + u) * NW;
        const int qpos = pos0 + (pr < P ? pr / nh : 0);
        const int lo = p.window > 0 ? qpos - p.window + 1 : 0;
        act[u] = pr < P && !(k0 > qpos || k0 + KT - 1 < lo);          // some key of this tile is visible to the pair (warp-uniform)
        vis[u] = act[u] && kp <= qpos && kp >= lo && kp <= last;          // (a decode key range may end inside the tile)
        qv[u] = s_q + (pr < P ? pr : 0) * R;
        any = any || act[u];
      }
      if (!any) continue;
      const float* cv = s_c + lane * RP;
      float a[PP], a2[PP];
#pragma unroll
      for (int u = 0; u < PP; ++u) a[u] = a2[u] = 0.f;
      if (vec) {
        const float4* c4 = reinterpret_cast<const float4*>(cv);
        for (int r4 = 0; r4 < (R >> 2); ++r4) {
          const float4 c = c4[r4];
#pragma unroll
          for (int u = 0; u < PP; ++u) {
            const float4 q4 = reinterpret_cast<const float4*>(qv[u])[r4];
            a[u] += q4.x * c.x + q4.y * c.y;
            a2[u] += q4.z * c.z + q4.w * c.w;
          }
        }
      } else {
        for (int r = 0; r < R; ++r) {
          const float c0 = cv[r];
#pragma unroll
          for (int u = 0; u < PP; ++u) a[u] += qv[u][r] * c0;
        }
      }
      float pj[PP], alpha[PP];
#pragma unroll
      for (int u = 0; u < PP; ++u) {
        pj[u] = 0.f;
        alpha[u] = 1.f;
        if (!act[u]) continue;
        const int k = g0 + u;
        const float sc = vis[u] ? (a[u] + a2[u]) * p.scale : -INFINITY;
        const float m_new = fmaxf(m_run[k], warp_max(sc));
        if (m_new == -INFINITY) { act[u] = false; continue; }
        alpha[u] = m_run[k] == -INFINITY ? 0.f : expf(m_run[k] - m_new);
        pj[u] = vis[u] ? expf(sc - m_new) : 0.f;
        l_run[k] = l_run[k] * alpha[u] + warp_sum(pj[u]);
        m_run[k] = m_new;
      }
      // probabilities go through shared memory: one 16-byte broadcast load brings four keys' weights of a pair
      float* sp = s_p + warp * 4 * KT;
#pragma unroll
      for (int u = 0; u < PP; ++u) sp[u * KT + lane] = pj[u];
      __syncwarp();
      for (int c0 = 0; c0 < Rv; c0 += 64) {                 // two column groups per pass
        float acc[PP][2];
#pragma unroll
        for (int u = 0; u < PP; ++u) acc[u][0] = acc[u][1] = 0.f;
        const int cc0 = min(c0 + lane, Rv - 1), cc1 = min(c0 + 32 + lane, Rv - 1);
#pragma unroll 2
        for (int j = 0; j < KT; j += 4) {
          float w[PP][4];
#pragma unroll
          for (int u = 0; u < PP; ++u) {
            const float4 t = *reinterpret_cast<const float4*>(sp + u * KT + j);
            w[u][0] = t.x; w[u][1] = t.y; w[u][2] = t.z; w[u][3] = t.w;
          }
#pragma unroll
          for (int jj = 0; jj < 4; ++jj) {
            const float v0 = s_c[(j + jj) * RP + cc0], v1 = s_c[(j + jj) * RP + cc1];
#pragma unroll
            for (int u = 0; u < PP; ++u) {
              acc[u][0] += w[u][jj] * v0;
              acc[u][1] += w[u][jj] * v1;
            }
          }
        }
#pragma unroll
        for (int u = 0; u < PP; ++u) {
          if (!act[u]) continue;
          float* ov = s_o + (warp + (g0 + u) * NW) * R;
          const int ca = c0 + lane, cb = c0 + 32 + lane;
          if (ca < Rv) ov[ca] = ov[ca] * alpha[u] + acc[u][0];
          if (cb < Rv) ov[cb] = ov[cb] * alpha[u] + acc[u][1];
        }
      }
      __syncwarp();                                          // sp is rewritten by the warp's next group of pairs
    }
  }
  __syncwarp();
#pragma unroll
  for (int k = 0; k < PPW_MAX; ++k) {
    const int pr = warp + k * NW;
    if (pr >= P) break;
    const int qi = pr / nh, hi = pr - qi * nh;
    if (QT == 1 && p.nsplit > 1) {
      const size_t row = ((size_t)(qbase + qi) * p.nsplit + split) * p.H + h0 + hi;
      for (int c = lane; c < Rv; c += 32) p.part_o[row * Rv + c] = s_o[pr * R + c];
      if (lane == 0) { p.part_ml[row * 2] = m_run[k]; p.part_ml[row * 2 + 1] = l_run[k]; }
      continue;
    }
    const float inv = 1.f / l_run[k];
    float* dst = p.out + ((size_t)(qbase + t0 + qi) * p.H + h0 + hi) * Rv;
    for (int c = lane; c < Rv; c += 32) dst[c] = s_o[pr * R + c] * inv;
  }
}

// decode, nsplit > 1: out[t, h, :] = sum_s o_s exp(m_s - m) / sum_s l_s exp(m_s - m); one warp per (token, head)
__global__ void __launch_bounds__(128) latent_merge_kernel(const float* __restrict__ part_o, const float* __restrict__ part_ml, float* __restrict__ out,
                                                           int rows, int H, int R, int nsplit) {
  const int row = blockIdx.x * 4 + (threadIdx.x >> 5), lane = threadIdx.x & 31;
  if (row >= rows) return;
  const int t = row / H, h = row - t * H;
  float m = -INFINITY;
  for (int s = 0; s < nsplit; ++s) m = fmaxf(m, part_ml[(((size_t)t * nsplit + s) * H + h) * 2]);
  float l = 0.f;
  for (int s = 0; s < nsplit; ++s) {
    const float* ml = part_ml + (((size_t)t * nsplit + s) * H + h) * 2;
    if (ml[0] != -INFINITY) l += ml[1] * expf(ml[0] - m);
  }
  const float inv = 1.f / l;
  for (int c = lane; c < R; c += 32) {
    float acc = 0.f;
    for (int s = 0; s < nsplit; ++s) {
      const size_t pr = ((size_t)t * nsplit + s) * H + h;
      const float ms = part_ml[pr * 2];
      if (ms != -INFINITY) acc += part_o[pr * R + c] * expf(ms - m);
    }
    out[(size_t)row * R + c] = acc * inv;
  }
}

template <typename TCache, int QT, int PP>
void launch_pp(const LatentParams& p, dim3 grid, size_t smem, cudaStream_t stream) {
  auto kern = latent_attention_kernel<TCache, QT, PP>;
  if (smem > 48 * 1024) SGLB_CUDA_CHECK(cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));
  kern<<<grid, NW * 32, smem, stream>>>(p);
  SGLB_CUDA_CHECK(cudaGetLastError());
}

template <typename TCache, int QT>
void launch(LatentParams p, int B, int max_q_len, int max_kv_len, float* workspace, size_t workspace_floats, cudaStream_t stream) {
  // heads per CTA: as many as fit 200 KB next to the key tile, at most 16 pairs per warp
  p.RP = (p.R % 4 == 0) ? p.R + 4 : p.R + 1;
  const size_t tile = (size_t)KT * p.RP * 4 + KT * 4 + (size_t)NW * 4 * KT * 4;
  const size_t per_head = (size_t)QT * p.R * 4 * 2;
  int hg = (int)std::min<size_t>((size_t)p.H, (200 * 1024 - tile) / per_head);
  hg = std::min(hg, 16 * NW / QT);
  if (hg < 1) throw std::runtime_error("sglb latent_attention: latent rank too large for one CTA");
  const int hgroups = (p.H + hg - 1) / hg;
  p.HG = hg;
  p.nsplit = 1;
  if (QT == 1) {
    // decode has few queries: cut every request's visible keys into ranges (>= 64 keys each) until ~2 CTAs per SM are in flight
    const int span = p.window > 0 ? std::min(p.window, max_kv_len) : max_kv_len;
    int ns = std::min(std::min(296 / std::max(1, B * hgroups), span / 64), 32);
    ns = std::max(ns, 1);
    if ((size_t)B * ns * p.H * (p.R + 2) > workspace_floats) ns = 1;
    p.nsplit = ns;
    p.part_o = workspace;
    p.part_ml = workspace + (size_t)B * ns * p.H * p.Rv;
  }
  const size_t smem = tile + per_head * hg;
  dim3 grid(QT == 1 ? p.nsplit : (max_q_len + QT - 1) / QT, B, hgroups);
  const int ppw = (QT * hg + NW - 1) / NW;               // pairs per warp: group them 4, 2 or 1 at a time
  if (ppw >= 3) launch_pp<TCache, QT, 4>(p, grid, smem, stream);
  else if (ppw == 2) launch_pp<TCache, QT, 2>(p, grid, smem, stream);
  else launch_pp<TCache, QT, 1>(p, grid, smem, stream);
  if (QT == 1 && p.nsplit > 1) {
    const int rows = B * p.H;
    latent_merge_kernel<<<(rows + 3) / 4, 128, 0, stream>>>(p.part_o, p.part_ml, p.out, rows, p.H, p.Rv, p.nsplit);
    SGLB_CUDA_CHECK(cudaGetLastError());
  }
}


// ---------------------------------------------------------------- what lies around the absorbed kernel when queries pass a latent and a rotary part is shared
// latent_prepare: per token, rows of x = [query latent (Rq) | key/value latent (R) | rotary key (Dr)]:
//   cq = query latent / rms * wq (x's type);  cache[loc, :R] = key/value latent / rms * wk;  cache[loc, R:R+Dr] = rotary key turned by
//   position * inv_freq[m] on neighbouring pairs (2m, 2m + 1), sine and cosine times mult.  Norms, angle, sine and cosine fp32.
template <typename T>
__global__ void __launch_bounds__(128) latent_prepare_kernel(const T* __restrict__ x, int ld, int Rq, const T* __restrict__ wq, int R, int Dr,
                                                             const T* __restrict__ wk, float eps, const int* __restrict__ positions,
                                                             const float* __restrict__ inv_freq, float mult, T* __restrict__ cache, size_t cstride,
                                                             const int* __restrict__ loc, T* __restrict__ cq) {
  __shared__ float red[8];
  const int t = blockIdx.x, tid = threadIdx.x;
  const T* row = x + (size_t)t * ld;
  float sq = 0.f, sk = 0.f;
  for (int i = tid; i < Rq; i += 128) { const float v = ldc<T>(row + i); sq += v * v; }
  for (int i = tid; i < R; i += 128) { const float v = ldc<T>(row + Rq + i); sk += v * v; }
  sq = warp_sum(sq); sk = warp_sum(sk);
  if ((tid & 31) == 0) { red[tid >> 5] = sq; red[4 + (tid >> 5)] = sk; }
  __syncthreads();
  const float rq = Rq > 0 ? 1.0f / sqrtf((red[0] + red[1] + red[2] + red[3]) / (float)Rq + eps) : 0.f;
  const float rk = 1.0f / sqrtf((red[4] + red[5] + red[6] + red[7]) / (float)R + eps);
  T* crow = cache + (size_t)loc[t] * cstride;
  for (int i = tid; i < Rq; i += 128) stc<T>(cq + (size_t)t * Rq + i, ldc<T>(row + i) * rq * ldc<T>(wq + i));
  for (int i = tid; i < R; i += 128) stc<T>(crow + i, ldc<T>(row + Rq + i) * rk * ldc<T>(wk + i));
  const float pos = (float)positions[t];
  for (int m = tid; m < Dr / 2; m += 128) {
    const float a = ldc<T>(row + Rq + R + 2 * m), b = ldc<T>(row + Rq + R + 2 * m + 1);
    float sn = 0.f, cs = 1.f;
    if (inv_freq) {
      sincosf(pos * inv_freq[m], &sn, &cs);
      sn *= mult; cs *= mult;
    }
    stc<T>(crow + R + 2 * m, a * cs - b * sn);
    stc<T>(crow + R + 2 * m + 1, b * cs + a * sn);
  }
}

// latent_query: out[t, h, :R] = q_abs[h, t, :] (the unrotated query already multiplied into the key up-projection), out[t, h, R:] = the rotary
// columns q[t, h, D:D+Dr] turned like the key's; grid (T, H)
template <typename T>
__global__ void __launch_bounds__(128) latent_query_kernel(const T* __restrict__ q, const float* __restrict__ q_abs, int Tn, int H, int D, int Dr, int R,
                                                           const int* __restrict__ positions, const float* __restrict__ inv_freq, float mult,
                                                           float* __restrict__ out) {
  const int t = blockIdx.x, h = blockIdx.y, tid = threadIdx.x;
  float* dst = out + ((size_t)t * H + h) * (R + Dr);
  const float* src = q_abs + ((size_t)h * Tn + t) * R;
  for (int i = tid; i < R; i += 128) dst[i] = src[i];
  const T* qr = q + ((size_t)t * H + h) * (D + Dr) + D;
  const float pos = (float)positions[t];
  for (int m = tid; m < Dr / 2; m += 128) {
    const float a = ldc<T>(qr + 2 * m), b = ldc<T>(qr + 2 * m + 1);
    float sn = 0.f, cs = 1.f;
    if (inv_freq) {
      sincosf(pos * inv_freq[m], &sn, &cs);
      sn *= mult; cs *= mult;
    }
    dst[R + 2 * m] = a * cs - b * sn;
    dst[R + 2 * m + 1] = b * cs + a * sn;
  }
}

}  // namespace

void latent_prepare(const void* x, int ld, bool bf16, int T, int Rq, const void* wq, int R, int Dr, const void* wk, float eps, const int* positions,
                    const float* inv_freq, float mult, void* cache, size_t ldc, const int* loc, void* cq, cudaStream_t stream) {
  if (T <= 0) return;
  using bf = __nv_bfloat16;
  if (bf16)
    latent_prepare_kernel<bf><<<T, 128, 0, stream>>>((const bf*)x, ld, Rq, (const bf*)wq, R, Dr, (const bf*)wk, eps, positions, inv_freq, mult, (bf*)cache,
                                                     ldc, loc, (bf*)cq);
  else
    latent_prepare_kernel<float><<<T, 128, 0, stream>>>((const float*)x, ld, Rq, (const float*)wq, R, Dr, (const float*)wk, eps, positions, inv_freq, mult,
                                                        (float*)cache, ldc, loc, (float*)cq);
  SGLB_CUDA_CHECK(cudaGetLastError());
}

void latent_query(const void* q, bool bf16, const float* q_abs, int T, int H, int D, int Dr, int R, const int* positions, const float* inv_freq, float mult,
                  float* out, cudaStream_t stream) {
  if (T <= 0 || H <= 0) return;
  if (H > 65535) throw std::runtime_error("sglb latent_query: more than 65535 heads");
  dim3 grid(T, H);
  if (bf16)
    latent_query_kernel<__nv_bfloat16><<<grid, 128, 0, stream>>>((const __nv_bfloat16*)q, q_abs, T, H, D, Dr, R, positions, inv_freq, mult, out);
  else
    latent_query_kernel<float><<<grid, 128, 0, stream>>>((const float*)q, q_abs, T, H, D, Dr, R, positions, inv_freq, mult, out);
  SGLB_CUDA_CHECK(cudaGetLastError());
}

void latent_attention(const float* q, const void* cache, bool cache_bf16, int ldc, int R, const int* page_table, int pt_stride, int page_size,
                      const int* req_slots, const int* seq_lens, const int* cu_q, int B, int max_q_len, int max_kv_len, int H, float scale,
                      int window, const float* sinks, float* out, float* workspace, size_t workspace_floats, int v_rank, cudaStream_t stream) {
  if (B <= 0 || max_q_len <= 0) return;
  if (v_rank <= 0 || v_rank > R) throw std::runtime_error("sglb latent_attention: the value is a leading part of the row");
  if (B > 65535) throw std::runtime_error("sglb latent_attention: more than 65535 requests in one call");
  LatentParams p;
  p.q = q; p.out = out; p.cache = cache; p.ldc = ldc; p.page_table = page_table; p.pt_stride = pt_stride; p.page_size = page_size;
  p.req_slots = req_slots; p.seq_lens = seq_lens; p.cu_q = cu_q; p.sinks = sinks; p.H = H; p.R = R; p.RP = R + 1; p.HG = 1; p.Rv = v_rank;
  const int esz = cache_bf16 ? 2 : 4;
  p.vec8 = (R % 8 == 0 && ((size_t)ldc * esz) % 16 == 0 && ((uintptr_t)cache % 16) == 0) ? 1 : 0; p.window = window; p.scale = scale; p.nsplit = 1; p.part_o = nullptr; p.part_ml = nullptr;
  const bool decode = cu_q == nullptr || max_q_len == 1;
  if (cache_bf16) {
    if (decode) launch<__nv_bfloat16, 1>(p, B, 1, max_kv_len, workspace, workspace_floats, stream);
    else launch<__nv_bfloat16, 8>(p, B, max_q_len, max_kv_len, workspace, workspace_floats, stream);
  } else {
    if (decode) launch<float, 1>(p, B, 1, max_kv_len, workspace, workspace_floats, stream);
    else launch<float, 8>(p, B, max_q_len, max_kv_len, workspace, workspace_floats, stream);
  }
}

}  // namespace sglb
