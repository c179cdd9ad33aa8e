// fp32 residual stream helpers.
//
//   add_rmsnorm_f32 : residual (fp32, in place) += delta (bf16 | fp32 | none); out = residual / rms(residual) * (w | 1 + w) in bf16 | fp32.
//                     One block per row; the sum, the mean of squares and the scaling are fp32, eps sits inside the root.  The weight is a
//                     vector or one number for all coordinates.
//   clamped_glu     : [gate | up] halves -> min(g, limit) * sigmoid(alpha * g) * (clamp(u, -limit, limit) + 1), fp32 math.
#include <stdexcept>

#include "common.cuh"
#include "tma_host.h"

namespace sglb {
namespace {

template <typename T> __device__ __forceinline__ float ldf(const T* p);
template <> __device__ __forceinline__ float ldf<float>(const float* p) { return *p; }
template <> __device__ __forceinline__ float ldf<__nv_bfloat16>(const __nv_bfloat16* p) { return __bfloat162float(*p); }
template <typename T> __device__ __forceinline__ void stf(T* p, float v);
template <> __device__ __forceinline__ void stf<float>(float* p, float v) { *p = v; }
template <> __device__ __forceinline__ void stf<__nv_bfloat16>(__nv_bfloat16* p, float v) { *p = __float2bfloat16(v); }

template <typename TD, typename TO>
__global__ void __launch_bounds__(256) add_rmsnorm_f32_kernel(float* __restrict__ res, const TD* __restrict__ delta, const TO* __restrict__ w,
                                                              TO* __restrict__ out, int H, float eps, int zero_centred, int ws) {
  __shared__ float red[8];
  __shared__ float s_rs;
  float* r = res + (size_t)blockIdx.x * H;
  const TD* d = delta ? delta + (size_t)blockIdx.x * H : nullptr;
  float ss = 0.f;
  for (int i = threadIdx.x; i < H; i += 256) {
    float v = r[i];
    if (d) {
      v += ldf<TD>(d + i);
      r[i] = v;
    }
    ss += v * v;
  }
  ss = warp_sum(ss);
  if ((threadIdx.x & 31) == 0) red[threadIdx.x >> 5] = ss;
  __syncthreads();
  if (threadIdx.x < 32) {
    float t = threadIdx.x < 8 ? red[threadIdx.x] : 0.f;
    t = warp_sum(t);
    if (threadIdx.x == 0) s_rs = 1.0f / sqrtf(t / (float)H + eps);
  }
  __syncthreads();
  const float rs = s_rs;
  TO* o = out + (size_t)blockIdx.x * H;
  for (int i = threadIdx.x; i < H; i += 256) {          // each thread re-reads exactly the elements it wrote
    float wv = ldf<TO>(w + i * ws);                   // ws = 0: one gain for all coordinates
    if (zero_centred) wv += 1.f;
    stf<TO>(o + i, r[i] * rs * wv);
  }
}

template <typename T>
__global__ void __launch_bounds__(256) clamped_glu_kernel(const T* __restrict__ gu, T* __restrict__ out, int I, float limit, float alpha) {
  const T* row = gu + (size_t)blockIdx.x * 2 * I;
  const int i = blockIdx.y * 256 + threadIdx.x;
  if (i >= I) return;
  const float g = fminf(ldf<T>(row + i), limit);
  const float u = fminf(fmaxf(ldf<T>(row + I + i), -limit), limit);
  stf<T>(out + (size_t)blockIdx.x * I + i, g / (1.f + expf(-alpha * g)) * (u + 1.f));
}

// 16-byte lanes: 8 bf16 gate values and the 8 matching up values per thread
__global__ void __launch_bounds__(256) clamped_glu_bf16x8_kernel(const __nv_bfloat16* __restrict__ gu, __nv_bfloat16* __restrict__ out, int I,
                                                                 float limit, float alpha) {
  const int i = (blockIdx.y * 256 + threadIdx.x) * 8;
  if (i >= I) return;
  const __nv_bfloat16* row = gu + (size_t)blockIdx.x * 2 * I;
  const U4 g = ldg128(row + i), u = ldg128(row + I + i);
  const uint32_t gw[4] = {g.x, g.y, g.z, g.w}, uw[4] = {u.x, u.y, u.z, u.w};
  uint32_t o[4];
#pragma unroll
  for (int k = 0; k < 4; ++k) {
    const float g0 = fminf(bf16_lo(gw[k]), limit), g1 = fminf(bf16_hi(gw[k]), limit);
    const float u0 = fminf(fmaxf(bf16_lo(uw[k]), -limit), limit), u1 = fminf(fmaxf(bf16_hi(uw[k]), -limit), limit);
    o[k] = pack_bf16(g0 / (1.f + __expf(-alpha * g0)) * (u0 + 1.f), g1 / (1.f + __expf(-alpha * g1)) * (u1 + 1.f));
  }
  st128(out + (size_t)blockIdx.x * I + i, U4{o[0], o[1], o[2], o[3]});
}

// block-wide sum for 256 threads (every thread gets the total)
__device__ __forceinline__ float block_sum_256(float v, float* red) {
  v = warp_sum(v);
  __syncthreads();                       // red may still be read from an earlier call
  if ((threadIdx.x & 31) == 0) red[threadIdx.x >> 5] = v;
  __syncthreads();
  float t = 0.f;
#pragma unroll
  for (int i = 0; i < 8; ++i) t += red[i];
  return t;
}

// residual += rmsnorm(delta) * (1 + post_w);  out = rmsnorm(residual) * (1 + w): the post-norm of a branch, the residual add and the next
// pre-norm of a sandwich-normed block in one pass over the row.  ``one`` = 1 for weights stored around zero, 0 for plain weights; a weight
// stride of 0 means one gain for all coordinates.
template <typename TD, typename TO>
__global__ void __launch_bounds__(256) postnorm_add_rmsnorm_f32_kernel(float* __restrict__ res, const TD* __restrict__ delta, const TO* __restrict__ post_w,
                                                                       const TO* __restrict__ w, TO* __restrict__ out, int H, float eps, float one,
                                                                       int wsp, int ws) {
  __shared__ float red[8];
  float* r = res + (size_t)blockIdx.x * H;
  const TD* d = delta + (size_t)blockIdx.x * H;
  float sd = 0.f;
  for (int i = threadIdx.x; i < H; i += 256) {
    const float v = ldf<TD>(d + i);
    sd += v * v;
  }
  const float rd = 1.0f / sqrtf(block_sum_256(sd, red) / (float)H + eps);
  float ss = 0.f;
  for (int i = threadIdx.x; i < H; i += 256) {
    const float v = r[i] + ldf<TD>(d + i) * rd * (one + ldf<TO>(post_w + i * wsp));
    r[i] = v;
    ss += v * v;
  }
  const float rs = 1.0f / sqrtf(block_sum_256(ss, red) / (float)H + eps);
  TO* o = out + (size_t)blockIdx.x * H;
  for (int i = threadIdx.x; i < H; i += 256) stf<TO>(o + i, r[i] * rs * (one + ldf<TO>(w + i * ws)));      // each thread re-reads what it wrote
}


// residual += d1 + d2 + d3 (each optional; d1 / d2 in the model dtype, d3 fp32; the deltas are summed first);  out1 = rmsnorm(residual) * (one + w1),
// out2 likewise under w2 (optional): the residual update of a block whose two branches read the same input, with both pre-norms of the next
// block, in one pass over the row.  Four columns per access; a thread keeps up to four accesses of the row in registers.
template <typename T> __device__ __forceinline__ float4 ld4f(const T* p);
template <> __device__ __forceinline__ float4 ld4f<float>(const float* p) { return *reinterpret_cast<const float4*>(p); }
template <> __device__ __forceinline__ float4 ld4f<__nv_bfloat16>(const __nv_bfloat16* p) {
  const uint2 v = *reinterpret_cast<const uint2*>(p);
  return make_float4(bf16_lo(v.x), bf16_hi(v.x), bf16_lo(v.y), bf16_hi(v.y));
}
template <typename T> __device__ __forceinline__ void st4f(T* p, float4 v);
template <> __device__ __forceinline__ void st4f<float>(float* p, float4 v) { *reinterpret_cast<float4*>(p) = v; }
template <> __device__ __forceinline__ void st4f<__nv_bfloat16>(__nv_bfloat16* p, float4 v) {
  *reinterpret_cast<uint2*>(p) = make_uint2(pack_bf16(v.x, v.y), pack_bf16(v.z, v.w));
}

template <typename TD, typename TO, int VEC>
__global__ void __launch_bounds__(256) parallel_add_rmsnorm_f32_kernel(float* __restrict__ res, const TD* __restrict__ d1, const TD* __restrict__ d2,
                                                                       const float* __restrict__ d3, const TO* __restrict__ w1, const TO* __restrict__ w2,
                                                                       TO* __restrict__ out1, TO* __restrict__ out2, int H, float eps, float one) {
  __shared__ float red[8];
  const size_t off = (size_t)blockIdx.x * H;
  float* r = res + off;
  const bool any = d1 || d2 || d3;
  float ss = 0.f;
  if constexpr (VEC == 4) {
    constexpr int KEEP = 4;
    float4 keep[KEEP];
    const int n4 = H >> 2;
#pragma unroll
    for (int k = 0; k < KEEP; ++k) {
      const int i = (threadIdx.x + k * 256) * 4;
      keep[k] = make_float4(0.f, 0.f, 0.f, 0.f);
      if (i < H) {
        float4 v = *reinterpret_cast<const float4*>(r + i);
        if (any) {
          float4 d = make_float4(0.f, 0.f, 0.f, 0.f);
          if (d1) { const float4 t = ld4f<TD>(d1 + off + i); d.x += t.x; d.y += t.y; d.z += t.z; d.w += t.w; }
          if (d2) { const float4 t = ld4f<TD>(d2 + off + i); d.x += t.x; d.y += t.y; d.z += t.z; d.w += t.w; }
          if (d3) { const float4 t = *reinterpret_cast<const float4*>(d3 + off + i); d.x += t.x; d.y += t.y; d.z += t.z; d.w += t.w; }
          v.x += d.x; v.y += d.y; v.z += d.z; v.w += d.w;
          *reinterpret_cast<float4*>(r + i) = v;
        }
        keep[k] = v;
        ss += v.x * v.x + v.y * v.y + v.z * v.z + v.w * v.w;
      }
    }
    for (int c = threadIdx.x + KEEP * 256; c < n4; c += 256) {          // rows wider than 4096: the rest is read again below
      const int i = c * 4;
      float4 v = *reinterpret_cast<const float4*>(r + i);
      if (any) {
        float4 d = make_float4(0.f, 0.f, 0.f, 0.f);
        if (d1) { const float4 t = ld4f<TD>(d1 + off + i); d.x += t.x; d.y += t.y; d.z += t.z; d.w += t.w; }
        if (d2) { const float4 t = ld4f<TD>(d2 + off + i); d.x += t.x; d.y += t.y; d.z += t.z; d.w += t.w; }
        if (d3) { const float4 t = *reinterpret_cast<const float4*>(d3 + off + i); d.x += t.x; d.y += t.y; d.z += t.z; d.w += t.w; }
        v.x += d.x; v.y += d.y; v.z += d.z; v.w += d.w;
        *reinterpret_cast<float4*>(r + i) = v;
      }
      ss += v.x * v.x + v.y * v.y + v.z * v.z + v.w * v.w;
    }
    const float rs = 1.0f / sqrtf(block_sum_256(ss, red) / (float)H + eps);
    auto emit = [&](int i, float4 v) {
      const float4 a = ld4f<TO>(w1 + i);
      st4f<TO>(out1 + off + i, make_float4(v.x * rs * (one + a.x), v.y * rs * (one + a.y), v.z * rs * (one + a.z), v.w * rs * (one + a.w)));
      if (out2) {
        const float4 b = ld4f<TO>(w2 + i);
        st4f<TO>(out2 + off + i, make_float4(v.x * rs * (one + b.x), v.y * rs * (one + b.y), v.z * rs * (one + b.z), v.w * rs * (one + b.w)));
      }
    };
#pragma unroll
    for (int k = 0; k < KEEP; ++k) {
      const int i = (threadIdx.x + k * 256) * 4;
      if (i < H) emit(i, keep[k]);
    }
    for (int c = threadIdx.x + KEEP * 256; c < n4; c += 256) emit(c * 4, *reinterpret_cast<const float4*>(r + c * 4));      // each thread re-reads what it wrote
  } else {
    for (int i = threadIdx.x; i < H; i += 256) {
      float v = r[i];
      if (any) {
        float d = 0.f;
        if (d1) d += ldf<TD>(d1 + off + i);
        if (d2) d += ldf<TD>(d2 + off + i);
        if (d3) d += d3[off + i];
        v += d;
        r[i] = v;
      }
      ss += v * v;
    }
    const float rs = 1.0f / sqrtf(block_sum_256(ss, red) / (float)H + eps);
    for (int i = threadIdx.x; i < H; i += 256) {          // each thread re-reads exactly the elements it wrote
      const float y = r[i] * rs;
      stf<TO>(out1 + off + i, y * (one + ldf<TO>(w1 + i)));
      if (out2) stf<TO>(out2 + off + i, y * (one + ldf<TO>(w2 + i)));
    }
  }
}

// x fp32 [T, C] in ``groups`` equal parts: part / sqrt(mean(part^2) + eps) * w [* sigmoid(gate)] * out_scale; grid (T, groups); gate and out are
// rows of ldg / ldo elements
template <typename TO>
__global__ void __launch_bounds__(256) grouped_rmsnorm_kernel(const float* __restrict__ x, const TO* __restrict__ w, TO* __restrict__ out, int C, int per,
                                                              float eps, const TO* __restrict__ gate, int ldg, int ldo, float out_scale) {
  __shared__ float red[8];
  const size_t base = (size_t)blockIdx.x * C + (size_t)blockIdx.y * per;
  float ss = 0.f;
  for (int i = threadIdx.x; i < per; i += 256) {
    const float v = x[base + i];
    ss += v * v;
  }
  const float rs = 1.0f / sqrtf(block_sum_256(ss, red) / (float)per + eps) * out_scale;
  const int c0 = blockIdx.y * per;
  TO* o = out + (size_t)blockIdx.x * ldo + c0;
  const TO* gr = gate ? gate + (size_t)blockIdx.x * ldg + c0 : nullptr;
  for (int i = threadIdx.x; i < per; i += 256) {
    float v = x[base + i] * rs * ldf<TO>(w + c0 + i);
    if (gr) v *= 1.f / (1.f + expf(-ldf<TO>(gr + i)));
    stf<TO>(o + i, v);
  }
}

// the same with one warp per (row, part): a CTA of 8 warps walks the parts of its row (many small parts: no CTA-wide barrier, 16-byte loads)
template <typename TO>
__global__ void __launch_bounds__(256) grouped_rmsnorm_warp_kernel(const float* __restrict__ x, const TO* __restrict__ w, TO* __restrict__ out, int C,
                                                                   int per, int groups, float eps) {
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  for (int g = warp; g < groups; g += 8) {
    const size_t base = (size_t)blockIdx.x * C + (size_t)g * per;
    const float4* xv = reinterpret_cast<const float4*>(x + base);
    float ss = 0.f;
    for (int i = lane; i < per / 4; i += 32) {
      const float4 v = xv[i];
      ss += v.x * v.x + v.y * v.y + v.z * v.z + v.w * v.w;
    }
    const float rs = 1.0f / sqrtf(warp_sum(ss) / (float)per + eps);
    const TO* wr = w + (size_t)g * per;
    for (int i = lane; i < per / 4; i += 32) {
      const float4 v = xv[i];
      TO* o = out + base + 4 * i;
      stf<TO>(o, v.x * rs * ldf<TO>(wr + 4 * i));
      stf<TO>(o + 1, v.y * rs * ldf<TO>(wr + 4 * i + 1));
      stf<TO>(o + 2, v.z * rs * ldf<TO>(wr + 4 * i + 2));
      stf<TO>(o + 3, v.w * rs * ldf<TO>(wr + 4 * i + 3));
    }
  }
}

}  // namespace

void postnorm_add_rmsnorm_f32(float* residual, const void* delta, bool delta_bf16, const void* post_w, const void* w, void* out, bool out_bf16, int T,
                              int H, float eps, bool zero_centred, int wsp, int ws, cudaStream_t stream) {
  if (T <= 0) return;
  using bf = __nv_bfloat16;
  const float one = zero_centred ? 1.f : 0.f;
  if (out_bf16) {
    if (delta_bf16)
      postnorm_add_rmsnorm_f32_kernel<bf, bf><<<T, 256, 0, stream>>>(residual, (const bf*)delta, (const bf*)post_w, (const bf*)w, (bf*)out, H, eps, one, wsp, ws);
    else
      postnorm_add_rmsnorm_f32_kernel<float, bf><<<T, 256, 0, stream>>>(residual, (const float*)delta, (const bf*)post_w, (const bf*)w, (bf*)out, H, eps, one, wsp, ws);
  } else {
    if (delta_bf16)
      postnorm_add_rmsnorm_f32_kernel<bf, float><<<T, 256, 0, stream>>>(residual, (const bf*)delta, (const float*)post_w, (const float*)w, (float*)out, H, eps, one, wsp, ws);
    else
      postnorm_add_rmsnorm_f32_kernel<float, float><<<T, 256, 0, stream>>>(residual, (const float*)delta, (const float*)post_w, (const float*)w,
                                                                           (float*)out, H, eps, one, wsp, ws);
  }
  SGLB_CUDA_CHECK(cudaGetLastError());
}

void parallel_add_rmsnorm_f32(float* residual, const void* d1, const void* d2, bool delta_bf16, const float* d3, const void* w1, const void* w2, void* out1,
                              void* out2, bool out_bf16, int T, int H, float eps, bool zero_centred, cudaStream_t stream) {
  if (T <= 0) return;
  using bf = __nv_bfloat16;
  const float one = zero_centred ? 1.f : 0.f;
  auto al = [](const void* p) { return p == nullptr || ((uintptr_t)p % 16) == 0; };
  const bool vec = H % 4 == 0 && al(residual) && al(d1) && al(d2) && al(d3) && al(w1) && al(w2) && al(out1) && al(out2);
#define SGLB_PAR(TD, TO)                                                                                                                         \
  do {                                                                                                                                           \
    if (vec)                                                                                                                                     \
      parallel_add_rmsnorm_f32_kernel<TD, TO, 4><<<T, 256, 0, stream>>>(residual, (const TD*)d1, (const TD*)d2, d3, (const TO*)w1, (const TO*)w2, \
                                                                        (TO*)out1, (TO*)out2, H, eps, one);                                     \
    else                                                                                                                                         \
      parallel_add_rmsnorm_f32_kernel<TD, TO, 1><<<T, 256, 0, stream>>>(residual, (const TD*)d1, (const TD*)d2, d3, (const TO*)w1, (const TO*)w2, \
                                                                        (TO*)out1, (TO*)out2, H, eps, one);                                     \
  } while (0)
  if (out_bf16) { if (delta_bf16) SGLB_PAR(bf, bf); else SGLB_PAR(float, bf); }
  else { if (delta_bf16) SGLB_PAR(bf, float); else SGLB_PAR(float, float); }
#undef SGLB_PAR
  SGLB_CUDA_CHECK(cudaGetLastError());
}

void grouped_rmsnorm(const float* x, const void* w, void* out, bool out_bf16, int T, int C, int groups, float eps, const void* gate, int ldg, int ldo,
                     float out_scale, cudaStream_t stream) {
  if (T <= 0) return;
  if (groups <= 0 || C % groups || groups > 65535) throw std::runtime_error("sglb grouped_rmsnorm: the width must split into equal parts");
  const int per = C / groups;
  if (!gate && ldo == C && out_scale == 1.f && groups >= 4 && per % 4 == 0 && per <= 4096 && ((uintptr_t)x % 16) == 0) {
    if (out_bf16) grouped_rmsnorm_warp_kernel<__nv_bfloat16><<<T, 256, 0, stream>>>(x, (const __nv_bfloat16*)w, (__nv_bfloat16*)out, C, per, groups, eps);
    else grouped_rmsnorm_warp_kernel<float><<<T, 256, 0, stream>>>(x, (const float*)w, (float*)out, C, per, groups, eps);
    SGLB_CUDA_CHECK(cudaGetLastError());
    return;
  }
  dim3 g(T, groups);
  if (out_bf16)
    grouped_rmsnorm_kernel<__nv_bfloat16><<<g, 256, 0, stream>>>(x, (const __nv_bfloat16*)w, (__nv_bfloat16*)out, C, per, eps, (const __nv_bfloat16*)gate, ldg,
                                                                 ldo, out_scale);
  else grouped_rmsnorm_kernel<float><<<g, 256, 0, stream>>>(x, (const float*)w, (float*)out, C, per, eps, (const float*)gate, ldg, ldo, out_scale);
  SGLB_CUDA_CHECK(cudaGetLastError());
}

void add_rmsnorm_f32(float* residual, const void* delta, bool delta_bf16, const void* w, void* out, bool out_bf16, int T, int H, float eps,
                     bool zero_centred, int ws, cudaStream_t stream) {
  if (T <= 0) return;
  const int z = zero_centred ? 1 : 0;
  if (out_bf16) {
    if (delta_bf16)
      add_rmsnorm_f32_kernel<__nv_bfloat16, __nv_bfloat16><<<T, 256, 0, stream>>>(residual, (const __nv_bfloat16*)delta, (const __nv_bfloat16*)w,
                                                                                  (__nv_bfloat16*)out, H, eps, z, ws);
    else
      add_rmsnorm_f32_kernel<float, __nv_bfloat16><<<T, 256, 0, stream>>>(residual, (const float*)delta, (const __nv_bfloat16*)w, (__nv_bfloat16*)out, H,
                                                                          eps, z, ws);
  } else {
    if (delta_bf16)
      add_rmsnorm_f32_kernel<__nv_bfloat16, float><<<T, 256, 0, stream>>>(residual, (const __nv_bfloat16*)delta, (const float*)w, (float*)out, H, eps, z, ws);
    else
      add_rmsnorm_f32_kernel<float, float><<<T, 256, 0, stream>>>(residual, (const float*)delta, (const float*)w, (float*)out, H, eps, z, ws);
  }
  SGLB_CUDA_CHECK(cudaGetLastError());
}

void clamped_glu(const void* gu, void* out, bool bf16, int T, int I, float limit, float alpha, cudaStream_t stream) {
  if (T <= 0 || I <= 0) return;
  if ((I + 255) / 256 > 65535) throw std::runtime_error("sglb clamped_glu: feed-forward width too large for one launch");
  dim3 g(T, (I + 255) / 256);
  if (bf16 && I % 8 == 0 && ((uintptr_t)gu % 16) == 0 && ((uintptr_t)out % 16) == 0) {
    clamped_glu_bf16x8_kernel<<<dim3(T, (I / 8 + 255) / 256), 256, 0, stream>>>((const __nv_bfloat16*)gu, (__nv_bfloat16*)out, I, limit, alpha);
    SGLB_CUDA_CHECK(cudaGetLastError());
    return;
  }
  if (bf16)
    clamped_glu_kernel<__nv_bfloat16><<<g, 256, 0, stream>>>((const __nv_bfloat16*)gu, (__nv_bfloat16*)out, I, limit, alpha);
  else
    clamped_glu_kernel<float><<<g, 256, 0, stream>>>((const float*)gu, (float*)out, I, limit, alpha);
  SGLB_CUDA_CHECK(cudaGetLastError());
}

}  // namespace sglb
