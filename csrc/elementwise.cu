// Elementwise kernels that have no producer to fuse into.
//
// pnm_silu_derivative: out = silu^(k)(x) [* g], k = 0..4, one pass, 16-byte vectors.  The k-th derivative is evaluated
// in closed form from s = sigmoid(x):  s' = s(1-s), s'' = s'(1-2s), s''' = s''(1-2s) - 2 s'^2,
// s'''' = s'''(1-2s) - 6 s' s'', and silu^(k) = k s^(k-1) + x s^(k).  Used for higher-order derivatives of
// physics-informed networks, where autograd would otherwise build a chain of ~10 elementwise launches per order.
#include <cuda_bf16.h>
#include <cuda_runtime.h>
#include <stdint.h>

#include "common.cuh"
#include "pnm_api.h"

namespace pnm {

template <int K>
__device__ __forceinline__ float silu_d(float x) {
  const float s = 1.f / (1.f + __expf(-x));
  if (K == 0) return x * s;
  const float d1 = s * (1.f - s);
  if (K == 1) return s + x * d1;
  const float t = 1.f - 2.f * s;
  const float d2 = d1 * t;
  if (K == 2) return 2.f * d1 + x * d2;
  const float d3 = d2 * t - 2.f * d1 * d1;
  if (K == 3) return 3.f * d2 + x * d3;
  const float d4 = d3 * t - 6.f * d1 * d2;
  return 4.f * d3 + x * d4;
}

template <typename T> struct EVec;
template <> struct EVec<float> {
  static constexpr int N = 4;
  static __device__ __forceinline__ void load(const float* p, float* f) {
    const float4 u = *reinterpret_cast<const float4*>(p); f[0] = u.x; f[1] = u.y; f[2] = u.z; f[3] = u.w;
  }
  static __device__ __forceinline__ void store(float* p, const float* f) { *reinterpret_cast<float4*>(p) = make_float4(f[0], f[1], f[2], f[3]); }
  static __device__ __forceinline__ float get(const float* p) { return *p; }
  static __device__ __forceinline__ void put(float* p, float v) { *p = v; }
};
template <> struct EVec<__nv_bfloat16> {
  static constexpr int N = 8;
  static __device__ __forceinline__ void load(const __nv_bfloat16* p, float* f) {
    const uint4 u = *reinterpret_cast<const uint4*>(p);
    const __nv_bfloat162* h = reinterpret_cast<const __nv_bfloat162*>(&u);
#pragma unroll
    for (int i = 0; i < 4; ++i) { const float2 v = __bfloat1622float2(h[i]); f[2 * i] = v.x; f[2 * i + 1] = v.y; }
  }
  static __device__ __forceinline__ void store(__nv_bfloat16* p, const float* f) {
    uint4 u;
    __nv_bfloat162* h = reinterpret_cast<__nv_bfloat162*>(&u);
#pragma unroll
    for (int i = 0; i < 4; ++i) h[i] = __floats2bfloat162_rn(f[2 * i], f[2 * i + 1]);
    *reinterpret_cast<uint4*>(p) = u;
  }
  static __device__ __forceinline__ float get(const __nv_bfloat16* p) { return __bfloat162float(*p); }
  static __device__ __forceinline__ void put(__nv_bfloat16* p, float v) { *p = __float2bfloat16(v); }
};

template <typename T, int K>
__global__ void __launch_bounds__(256) silu_derivative_kernel(const T* __restrict__ x, const T* __restrict__ g, T* __restrict__ out,
                                                               long long n) {
  constexpr int V = EVec<T>::N;
  const long long nvec = n / V, stride = (long long)gridDim.x * blockDim.x;
  float f[V], m[V];
  for (long long v = blockIdx.x * (long long)blockDim.x + threadIdx.x; v < nvec; v += stride) {
    EVec<T>::load(x + v * V, f);
    if (g) EVec<T>::load(g + v * V, m);
#pragma unroll
    for (int i = 0; i < V; ++i) f[i] = silu_d<K>(f[i]) * (g ? m[i] : 1.f);
    EVec<T>::store(out + v * V, f);
  }
  // ragged tail (n not a multiple of the vector width)
  for (long long i = nvec * V + blockIdx.x * (long long)blockDim.x + threadIdx.x; i < n; i += stride)
    EVec<T>::put(out + i, silu_d<K>(EVec<T>::get(x + i)) * (g ? EVec<T>::get(g + i) : 1.f));
}

template <typename T>
int launch_silu(const void* x, const void* g, void* out, long long n, int order, cudaStream_t st) {
  const T* xi = static_cast<const T*>(x);
  const T* gi = static_cast<const T*>(g);
  T* o = static_cast<T*>(out);
  const long long nvec = n / EVec<T>::N + 1;
  const unsigned grid = (unsigned)min((long long)148 * 16, (nvec + 255) / 256);
  switch (order) {
    case 0: silu_derivative_kernel<T, 0><<<grid, 256, 0, st>>>(xi, gi, o, n); break;
    case 1: silu_derivative_kernel<T, 1><<<grid, 256, 0, st>>>(xi, gi, o, n); break;
    case 2: silu_derivative_kernel<T, 2><<<grid, 256, 0, st>>>(xi, gi, o, n); break;
    case 3: silu_derivative_kernel<T, 3><<<grid, 256, 0, st>>>(xi, gi, o, n); break;
    case 4: silu_derivative_kernel<T, 4><<<grid, 256, 0, st>>>(xi, gi, o, n); break;
    default: return -1;
  }
  return (int)cudaGetLastError();
}

}  // namespace pnm

extern "C" int pnm_silu_derivative(const void* x, const void* g, void* out, long long n, int order, int dtype, void* stream) {
  if (n <= 0) return 0;
  if ((reinterpret_cast<uintptr_t>(x) | reinterpret_cast<uintptr_t>(out) | reinterpret_cast<uintptr_t>(g)) & 15) return -2;
  cudaStream_t st = (cudaStream_t)stream;
  return dtype == 0 ? pnm::launch_silu<__nv_bfloat16>(x, g, out, n, order, st) : pnm::launch_silu<float>(x, g, out, n, order, st);
}

// ---------------------------------------------------------------------------------------------------------------------
// EDM noise conditioning in one launch: sinusoidal embedding of the noise level (sin half first, then cos half: the
// "swapped" order the U-Net uses), optional additive term (class / augmentation embedding), then two Linear + SiLU
// layers.  out[b, :] = silu(W1 silu(W0 (emb(noise[b]) + extra[b]) + b0) + b1).
//
// One CTA per batch row.  A warp owns one output channel at a time: its lanes stride over the input channels (coalesced
// reads of one weight row) and reduce by shuffles; the hidden vector lives in shared memory between the two layers.  The
// weights (fp32 or bf16) are a megabyte or two and stay in L2 across the CTAs.
namespace pnm {

template <typename T> __device__ __forceinline__ float cond_ld(const T* p);
template <> __device__ __forceinline__ float cond_ld<float>(const float* p) { return *p; }
template <> __device__ __forceinline__ float cond_ld<__nv_bfloat16>(const __nv_bfloat16* p) { return __bfloat162float(*p); }

template <typename T>
__global__ void __launch_bounds__(512) edm_conditioning_kernel(const float* __restrict__ noise, const float* __restrict__ freqs,
                                                               const float* __restrict__ extra, const T* __restrict__ w0,
                                                               const T* __restrict__ b0, const T* __restrict__ w1,
                                                               const T* __restrict__ b1, float* __restrict__ out, int C, int E) {
  extern __shared__ float cond_smem[];
  float* emb = cond_smem;      // [C]
  float* hid = cond_smem + C;  // [E]
  const int b = blockIdx.x, half = C / 2;
  const float sigma = noise[b];
  for (int c = threadIdx.x; c < C; c += blockDim.x) {
    const float a = sigma * freqs[c < half ? c : c - half];
    float v = c < half ? sinf(a) : cosf(a);
    if (extra) v += extra[(size_t)b * C + c];
    emb[c] = v;
  }
  __syncthreads();
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31, nwarps = blockDim.x >> 5;
  for (int e = warp; e < E; e += nwarps) {
    const T* row = w0 + (size_t)e * C;
    float acc = 0.f;
    for (int c = lane; c < C; c += 32) acc = fmaf(cond_ld(row + c), emb[c], acc);
    for (int o = 16; o > 0; o >>= 1) acc += __shfl_xor_sync(0xffffffffu, acc, o);
    if (lane == 0) {
      const float z = acc + (b0 ? cond_ld(b0 + e) : 0.f);
      hid[e] = z / (1.f + __expf(-z));
    }
  }
  __syncthreads();
  for (int e = warp; e < E; e += nwarps) {
    const T* row = w1 + (size_t)e * E;
    float acc = 0.f;
    for (int c = lane; c < E; c += 32) acc = fmaf(cond_ld(row + c), hid[c], acc);
    for (int o = 16; o > 0; o >>= 1) acc += __shfl_xor_sync(0xffffffffu, acc, o);
    if (lane == 0) {
      const float z = acc + (b1 ? cond_ld(b1 + e) : 0.f);
      out[(size_t)b * E + e] = z / (1.f + __expf(-z));
    }
  }
}

}  // namespace pnm

extern "C" int pnm_edm_conditioning(const float* noise, const float* freqs, const float* extra, const void* w0, const void* b0,
                                    const void* w1, const void* b1, float* out, int B, int C, int E, int weight_dtype,
                                    void* stream) {
  if (!noise || !freqs || !w0 || !w1 || !out || B <= 0 || C <= 0 || (C & 1) || E <= 0) return -1;
  const size_t smem = size_t(C + E) * sizeof(float);
  if (smem > 48 * 1024) return -1;
  cudaStream_t st = reinterpret_cast<cudaStream_t>(stream);
  if (weight_dtype == 1) {
    pnm::edm_conditioning_kernel<float><<<B, 512, smem, st>>>(noise, freqs, extra, (const float*)w0, (const float*)b0, (const float*)w1,
                                                             (const float*)b1, out, C, E);
  } else if (weight_dtype == 0) {
    using bf = __nv_bfloat16;
    pnm::edm_conditioning_kernel<bf><<<B, 512, smem, st>>>(noise, freqs, extra, (const bf*)w0, (const bf*)b0, (const bf*)w1, (const bf*)b1,
                                                          out, C, E);
  } else {
    return -1;
  }
  return cudaGetLastError() == cudaSuccess ? 0 : -4;
}

// out = (a + b) * scale on bf16 tensors of n elements (n % 8 == 0, 16-byte aligned): the residual join of the diffusion
// U-Net blocks, one pass instead of an add and a multiply.  b may be null (out = a * scale).
namespace pnm {
__global__ void __launch_bounds__(256) add_scale_bf16_kernel(const uint4* __restrict__ a, const uint4* __restrict__ b, uint4* __restrict__ out,
                                                             long long nvec, float scale) {
  for (long long i = blockIdx.x * (long long)blockDim.x + threadIdx.x; i < nvec; i += (long long)gridDim.x * blockDim.x) {
    const uint4 ua = a[i];
    const uint32_t wa[4] = {ua.x, ua.y, ua.z, ua.w};
    uint32_t wo[4];
    if (b) {
      const uint4 ub = b[i];
      const uint32_t wb[4] = {ub.x, ub.y, ub.z, ub.w};
#pragma unroll
      for (int k = 0; k < 4; ++k) {
        const float2 x = unpack_bf16x2(wa[k]), y = unpack_bf16x2(wb[k]);
        wo[k] = pack_bf16x2((x.x + y.x) * scale, (x.y + y.y) * scale);
      }
    } else {
#pragma unroll
      for (int k = 0; k < 4; ++k) {
        const float2 x = unpack_bf16x2(wa[k]);
        wo[k] = pack_bf16x2(x.x * scale, x.y * scale);
      }
    }
    out[i] = make_uint4(wo[0], wo[1], wo[2], wo[3]);
  }
}
}  // namespace pnm

extern "C" int pnm_add_scale_bf16(const void* a, const void* b, void* out, long long n, float scale, void* stream) {
  if (!a || !out || n <= 0 || (n & 7)) return -2;
  const long long nvec = n >> 3;
  const long long blocks = (nvec + 255) / 256;
  pnm::add_scale_bf16_kernel<<<(unsigned)(blocks < 148 * 16 ? blocks : 148 * 16), 256, 0, (cudaStream_t)stream>>>(
      (const uint4*)a, (const uint4*)b, (uint4*)out, nvec, scale);
  return cudaGetLastError() == cudaSuccess ? 0 : -3;
}
