// Two memory-bound kernels at the tail of a patch-token model (AFNO, ModAFNO):
//
// pnm_unpatchify_bf16: head output tokens [B, h, w, p0 * p1 * C] (features ordered (i, j, c)) <-> image
// [B, C, h * p0, w * p1], in either direction (the reverse is the gradient).  A generic strided copy of this
// permutation moves 2-byte elements one at a time and reaches a fraction of the copy bandwidth; here a block stages the
// (j, c) features of one image row segment in shared memory, reads them with 16-byte vectors on the token side and
// writes 16-byte vectors along the image row (p1 a multiple of 8, p1 * C a multiple of 8), so both sides are coalesced.
//
// pnm_sq_err_sum / pnm_sq_err_grad: sum((pred - target)^2) * scale in one pass (fp32 accumulation, two-stage
// deterministic reduction) and its gradient 2 * scale * g * (pred - target) in one pass, for bf16 or fp32 predictions
// against bf16 or fp32 targets.  Replaces the cast / subtract / square / sum chain and its four backward kernels.
#include <cuda_bf16.h>
#include <cuda_runtime.h>
#include <stdint.h>

#include "common.cuh"
#include "pnm_api.h"

namespace pnm {

struct PatchGeom {
  int B, h, w, p0, p1, C;
  int wc;        // token columns per block
  int stride;    // shared-memory row stride in elements (even, odd number of 32-bit words)
};

// grid: (ceil(w / wc), h * p0, B); block: 256 threads.  to_image = true: tokens -> image, false: image -> tokens.
template <bool VEC>
__global__ void __launch_bounds__(256) unpatchify_kernel(const __nv_bfloat16* __restrict__ tokens_c, __nv_bfloat16* tokens_m,
                                                         const __nv_bfloat16* __restrict__ image_c, __nv_bfloat16* image_m,
                                                         PatchGeom g, int to_image) {
  extern __shared__ __align__(16) unsigned char smem_raw[];
  __nv_bfloat16* tile = reinterpret_cast<__nv_bfloat16*>(smem_raw);
  const int ww0 = blockIdx.x * g.wc;
  const int nw = min(g.wc, g.w - ww0);
  const int hh = blockIdx.y / g.p0, i = blockIdx.y % g.p0;
  const int b = blockIdx.z;
  const int feat = g.p1 * g.C;                                   // (j, c) features of one image row inside a token
  const long long tok_row = (long long)g.p0 * feat;              // features per token
  const long long tok0 = (((long long)b * g.h + hh) * g.w + ww0) * tok_row + (long long)i * feat;
  const int Hh = g.h * g.p0, Ww = g.w * g.p1;
  const long long img0 = ((long long)b * g.C * Hh + (hh * g.p0 + i)) * Ww + (long long)ww0 * g.p1;   // + c * Hh * Ww
  const long long plane = (long long)Hh * Ww;

  if (to_image) {
    // tokens -> tile[wl][k]
    if (VEC) {
      const int vrow = feat >> 3;
      for (int t = threadIdx.x; t < nw * vrow; t += blockDim.x) {
        const int wl = t / vrow, v = t - wl * vrow;
        const uint4 u = *reinterpret_cast<const uint4*>(tokens_c + tok0 + (long long)wl * tok_row + 8 * v);
        uint32_t* dst = reinterpret_cast<uint32_t*>(tile + wl * g.stride + 8 * v);
        dst[0] = u.x; dst[1] = u.y; dst[2] = u.z; dst[3] = u.w;
      }
    } else {
      for (int t = threadIdx.x; t < nw * feat; t += blockDim.x) {
        const int wl = t / feat, k = t - wl * feat;
        tile[wl * g.stride + k] = tokens_c[tok0 + (long long)wl * tok_row + k];
      }
    }
    __syncthreads();
    if (VEC) {
      const int jv = g.p1 >> 3;                                  // 16-byte vectors per token along the image row
      const int per_c = nw * jv;
      for (int t = threadIdx.x; t < g.C * per_c; t += blockDim.x) {
        const int c = t / per_c, r = t - c * per_c;              // r = wl * jv + v: consecutive lanes, consecutive bytes
        const int wl = r / jv, v = r - wl * jv;
        const __nv_bfloat16* src = tile + wl * g.stride + (8 * v) * g.C + c;
        uint32_t wo[4];
#pragma unroll
        for (int q = 0; q < 4; ++q) {
          const uint32_t lo = __bfloat16_as_ushort(src[(2 * q) * g.C]);
          const uint32_t hi = __bfloat16_as_ushort(src[(2 * q + 1) * g.C]);
          wo[q] = lo | (hi << 16);
        }
        *reinterpret_cast<uint4*>(image_m + img0 + c * plane + 8 * r) = make_uint4(wo[0], wo[1], wo[2], wo[3]);
      }
    } else {
      const int per_c = nw * g.p1;
      for (int t = threadIdx.x; t < g.C * per_c; t += blockDim.x) {
        const int c = t / per_c, r = t - c * per_c;
        const int wl = r / g.p1, j = r - wl * g.p1;
        image_m[img0 + c * plane + r] = tile[wl * g.stride + j * g.C + c];
      }
    }
  } else {
    // image -> tile[wl][k]
    if (VEC) {
      const int jv = g.p1 >> 3;
      const int per_c = nw * jv;
      for (int t = threadIdx.x; t < g.C * per_c; t += blockDim.x) {
        const int c = t / per_c, r = t - c * per_c;
        const int wl = r / jv, v = r - wl * jv;
        const uint4 u = *reinterpret_cast<const uint4*>(image_c + img0 + c * plane + 8 * r);
        __nv_bfloat16* dst = tile + wl * g.stride + (8 * v) * g.C + c;
        const uint32_t wi[4] = {u.x, u.y, u.z, u.w};
#pragma unroll
        for (int q = 0; q < 4; ++q) {
          dst[(2 * q) * g.C] = __ushort_as_bfloat16((unsigned short)(wi[q] & 0xffffu));
          dst[(2 * q + 1) * g.C] = __ushort_as_bfloat16((unsigned short)(wi[q] >> 16));
        }
      }
    } else {
      const int per_c = nw * g.p1;
      for (int t = threadIdx.x; t < g.C * per_c; t += blockDim.x) {
        const int c = t / per_c, r = t - c * per_c;
        const int wl = r / g.p1, j = r - wl * g.p1;
        tile[wl * g.stride + j * g.C + c] = image_c[img0 + c * plane + r];
      }
    }
    __syncthreads();
    if (VEC) {
      const int vrow = feat >> 3;
      for (int t = threadIdx.x; t < nw * vrow; t += blockDim.x) {
        const int wl = t / vrow, v = t - wl * vrow;
        const uint32_t* src = reinterpret_cast<const uint32_t*>(tile + wl * g.stride + 8 * v);
        *reinterpret_cast<uint4*>(tokens_m + tok0 + (long long)wl * tok_row + 8 * v) = make_uint4(src[0], src[1], src[2], src[3]);
      }
    } else {
      for (int t = threadIdx.x; t < nw * feat; t += blockDim.x) {
        const int wl = t / feat, k = t - wl * feat;
        tokens_m[tok0 + (long long)wl * tok_row + k] = tile[wl * g.stride + k];
      }
    }
  }
}

}  // namespace pnm

extern "C" int pnm_unpatchify_bf16(void* tokens, void* image, int B, int h, int w, int p0, int p1, int C, int to_image,
                                   void* stream) {
  if (!tokens || !image || B <= 0 || h <= 0 || w <= 0 || p0 <= 0 || p1 <= 0 || C <= 0) return -2;
  if ((long long)h * p0 > 65535 || B > 65535) return -2;
  pnm::PatchGeom g{B, h, w, p0, p1, C, 0, 0};
  const int feat = p1 * C;
  g.stride = (feat + 1) & ~1;                        // even number of elements ...
  if (((g.stride >> 1) & 1) == 0) g.stride += 2;     // ... and an odd number of 32-bit words: lanes over wl hit distinct banks
  const int budget = 24 * 1024;                      // elements per tile (48 KB)
  g.wc = budget / g.stride;
  if (g.wc < 1) return -2;
  if (g.wc > w) g.wc = w;
  if (g.wc >= 32) g.wc &= ~31;                       // whole warps of token columns
  const size_t smem = (size_t)g.wc * g.stride * sizeof(__nv_bfloat16);
  const bool vec = (p1 % 8 == 0) && (feat % 8 == 0) && ((uintptr_t)tokens % 16 == 0) && ((uintptr_t)image % 16 == 0);
  const dim3 grid((w + g.wc - 1) / g.wc, h * p0, B);
  auto* tk = (__nv_bfloat16*)tokens;
  auto* im = (__nv_bfloat16*)image;
  if (vec) {
    if (smem > 48 * 1024) cudaFuncSetAttribute(pnm::unpatchify_kernel<true>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
    pnm::unpatchify_kernel<true><<<grid, 256, smem, (cudaStream_t)stream>>>(tk, tk, im, im, g, to_image);
  } else {
    if (smem > 48 * 1024) cudaFuncSetAttribute(pnm::unpatchify_kernel<false>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
    pnm::unpatchify_kernel<false><<<grid, 256, smem, (cudaStream_t)stream>>>(tk, tk, im, im, g, to_image);
  }
  return cudaGetLastError() == cudaSuccess ? 0 : -3;
}

namespace pnm {

template <typename T> __device__ __forceinline__ void load8(const T* p, float* f);
template <> __device__ __forceinline__ void load8<__nv_bfloat16>(const __nv_bfloat16* p, float* f) {
  const uint4 u = *reinterpret_cast<const uint4*>(p);
  const uint32_t w[4] = {u.x, u.y, u.z, u.w};
#pragma unroll
  for (int q = 0; q < 4; ++q) {
    const float2 v = unpack_bf16x2(w[q]);
    f[2 * q] = v.x; f[2 * q + 1] = v.y;
  }
}
template <> __device__ __forceinline__ void load8<float>(const float* p, float* f) {
  const float4 a = *reinterpret_cast<const float4*>(p), b = *reinterpret_cast<const float4*>(p + 4);
  f[0] = a.x; f[1] = a.y; f[2] = a.z; f[3] = a.w; f[4] = b.x; f[5] = b.y; f[6] = b.z; f[7] = b.w;
}
template <typename T> __device__ __forceinline__ void store8(T* p, const float* f);
template <> __device__ __forceinline__ void store8<__nv_bfloat16>(__nv_bfloat16* p, const float* f) {
  *reinterpret_cast<uint4*>(p) = make_uint4(pack_bf16x2(f[0], f[1]), pack_bf16x2(f[2], f[3]), pack_bf16x2(f[4], f[5]),
                                            pack_bf16x2(f[6], f[7]));
}
template <> __device__ __forceinline__ void store8<float>(float* p, const float* f) {
  *reinterpret_cast<float4*>(p) = make_float4(f[0], f[1], f[2], f[3]);
  *reinterpret_cast<float4*>(p + 4) = make_float4(f[4], f[5], f[6], f[7]);
}
template <typename T> __device__ __forceinline__ float to_f(T v);
template <> __device__ __forceinline__ float to_f<float>(float v) { return v; }
template <> __device__ __forceinline__ float to_f<__nv_bfloat16>(__nv_bfloat16 v) { return __bfloat162float(v); }
template <typename T> __device__ __forceinline__ T from_f(float v);
template <> __device__ __forceinline__ float from_f<float>(float v) { return v; }
template <> __device__ __forceinline__ __nv_bfloat16 from_f<__nv_bfloat16>(float v) { return __float2bfloat16_rn(v); }

constexpr int kSqErrThreads = 256;

// stage 1: every block writes the sum over its grid-stride share to partial[blockIdx.x]
template <typename P, typename T>
__global__ void __launch_bounds__(kSqErrThreads) sq_err_partial_kernel(const P* __restrict__ pred, const T* __restrict__ tgt,
                                                                       long long n, float* __restrict__ partial) {
  const long long nvec = n >> 3;
  float acc = 0.f;
  for (long long v = (long long)blockIdx.x * blockDim.x + threadIdx.x; v < nvec; v += (long long)gridDim.x * blockDim.x) {
    float a[8], b[8];
    load8<P>(pred + 8 * v, a);
    load8<T>(tgt + 8 * v, b);
#pragma unroll
    for (int q = 0; q < 8; ++q) {
      const float d = a[q] - b[q];
      acc = fmaf(d, d, acc);
    }
  }
  if (blockIdx.x == 0) {                                          // ragged tail (n not a multiple of 8)
    for (long long e = (nvec << 3) + threadIdx.x; e < n; e += blockDim.x) {
      const float d = to_f<P>(pred[e]) - to_f<T>(tgt[e]);
      acc = fmaf(d, d, acc);
    }
  }
  __shared__ float warp_part[kSqErrThreads / 32];
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) acc += __shfl_xor_sync(0xffffffffu, acc, o);
  if ((threadIdx.x & 31) == 0) warp_part[threadIdx.x >> 5] = acc;
  __syncthreads();
  if (threadIdx.x == 0) {
    float s = 0.f;
    for (int k = 0; k < kSqErrThreads / 32; ++k) s += warp_part[k];
    partial[blockIdx.x] = s;
  }
}

// stage 2: one block folds the partials in double, in a fixed order
__global__ void __launch_bounds__(256) sq_err_finalize_kernel(const float* __restrict__ partial, int count, double scale,
                                                              float* __restrict__ out) {
  __shared__ double sh[256];
  double s = 0.0;
  for (int k = threadIdx.x; k < count; k += 256) s += (double)partial[k];
  sh[threadIdx.x] = s;
  __syncthreads();
  for (int o = 128; o > 0; o >>= 1) {
    if ((int)threadIdx.x < o) sh[threadIdx.x] += sh[threadIdx.x + o];
    __syncthreads();
  }
  if (threadIdx.x == 0) out[0] = (float)(sh[0] * scale);
}

// grad = coef * gout[0] * (pred - target)
template <typename P, typename T>
__global__ void __launch_bounds__(256) sq_err_grad_kernel(const P* __restrict__ pred, const T* __restrict__ tgt,
                                                          const float* __restrict__ gout, float coef, long long n,
                                                          P* __restrict__ grad) {
  const float s = coef * gout[0];
  const long long nvec = n >> 3;
  for (long long v = (long long)blockIdx.x * blockDim.x + threadIdx.x; v < nvec; v += (long long)gridDim.x * blockDim.x) {
    float a[8], b[8];
    load8<P>(pred + 8 * v, a);
    load8<T>(tgt + 8 * v, b);
#pragma unroll
    for (int q = 0; q < 8; ++q) a[q] = s * (a[q] - b[q]);
    store8<P>(grad + 8 * v, a);
  }
  if (blockIdx.x == 0) {
    for (long long e = (nvec << 3) + threadIdx.x; e < n; e += blockDim.x)
      grad[e] = from_f<P>(s * (to_f<P>(pred[e]) - to_f<T>(tgt[e])));
  }
}

inline int sq_err_grid(long long n) {
  const long long blocks = ((n >> 3) + 255) / 256;
  const long long cap = 148 * 8;
  return (int)(blocks < 1 ? 1 : (blocks < cap ? blocks : cap));
}

}  // namespace pnm

// dtype codes: 0 = fp32, 1 = bf16.  partial must hold pnm_sq_err_partials() floats.
extern "C" int pnm_sq_err_partials(void) { return 148 * 8; }

extern "C" int pnm_sq_err_sum(const void* pred, const void* tgt, long long n, int pred_dtype, int tgt_dtype, double scale,
                              float* partial, float* out, void* stream) {
  if (!pred || !tgt || !partial || !out || n <= 0) return -2;
  if (((uintptr_t)pred | (uintptr_t)tgt) & 15) return -2;
  const int grid = pnm::sq_err_grid(n);
  auto st = (cudaStream_t)stream;
  using bf = __nv_bfloat16;
  if (pred_dtype == 1 && tgt_dtype == 0)
    pnm::sq_err_partial_kernel<bf, float><<<grid, pnm::kSqErrThreads, 0, st>>>((const bf*)pred, (const float*)tgt, n, partial);
  else if (pred_dtype == 1 && tgt_dtype == 1)
    pnm::sq_err_partial_kernel<bf, bf><<<grid, pnm::kSqErrThreads, 0, st>>>((const bf*)pred, (const bf*)tgt, n, partial);
  else if (pred_dtype == 0 && tgt_dtype == 0)
    pnm::sq_err_partial_kernel<float, float><<<grid, pnm::kSqErrThreads, 0, st>>>((const float*)pred, (const float*)tgt, n, partial);
  else if (pred_dtype == 0 && tgt_dtype == 1)
    pnm::sq_err_partial_kernel<float, bf><<<grid, pnm::kSqErrThreads, 0, st>>>((const float*)pred, (const bf*)tgt, n, partial);
  else
    return -2;
  pnm::sq_err_finalize_kernel<<<1, 256, 0, st>>>(partial, grid, scale, out);
  return cudaGetLastError() == cudaSuccess ? 0 : -3;
}

extern "C" int pnm_sq_err_grad(const void* pred, const void* tgt, const float* gout, long long n, int pred_dtype, int tgt_dtype,
                               float coef, void* grad, void* stream) {
  if (!pred || !tgt || !gout || !grad || n <= 0) return -2;
  if (((uintptr_t)pred | (uintptr_t)tgt | (uintptr_t)grad) & 15) return -2;
  const int grid = pnm::sq_err_grid(n) * 2;
  auto st = (cudaStream_t)stream;
  using bf = __nv_bfloat16;
  if (pred_dtype == 1 && tgt_dtype == 0)
    pnm::sq_err_grad_kernel<bf, float><<<grid, 256, 0, st>>>((const bf*)pred, (const float*)tgt, gout, coef, n, (bf*)grad);
  else if (pred_dtype == 1 && tgt_dtype == 1)
    pnm::sq_err_grad_kernel<bf, bf><<<grid, 256, 0, st>>>((const bf*)pred, (const bf*)tgt, gout, coef, n, (bf*)grad);
  else if (pred_dtype == 0 && tgt_dtype == 0)
    pnm::sq_err_grad_kernel<float, float><<<grid, 256, 0, st>>>((const float*)pred, (const float*)tgt, gout, coef, n, (float*)grad);
  else if (pred_dtype == 0 && tgt_dtype == 1)
    pnm::sq_err_grad_kernel<float, bf><<<grid, 256, 0, st>>>((const float*)pred, (const bf*)tgt, gout, coef, n, (float*)grad);
  else
    return -2;
  return cudaGetLastError() == cudaSuccess ? 0 : -3;
}
