// Row softmax over long bf16 rows, forward and backward, for attention computed as two GEMMs around a materialised score
// matrix (head widths that the TMEM flash kernel does not cover, e.g. the single 512-wide head of the SongUNet bottleneck).
//
//   forward    P[r, :] = softmax(scale * S[r, :])  in place (bf16), lse[r] = log sum exp(scale * S[r, :])  (optional)
//   backward   dS[r, :] = scale * P[r, :] * (dP[r, :] - sum_j dP[r, j] P[r, j])  written over dP (bf16)
//
// One CTA per row; a row of up to 16384 values lives in registers between the passes (8 vectors of 8 per thread at 256
// threads), longer rows are re-read (they stay in L2).  fp32 arithmetic; L % 8 == 0, ld % 8 == 0.
#include <cuda_bf16.h>
#include <cuda_runtime.h>
#include <stdint.h>

#include "common.cuh"
#include "pnm_api.h"

namespace pnm {

constexpr int kSmThreads = 256;
constexpr int kSmVecs = 8;   // vectors of 8 kept in registers per thread

__device__ __forceinline__ float sm_block_max(float v, float* red) {
  for (int o = 16; o > 0; o >>= 1) v = fmaxf(v, __shfl_xor_sync(0xffffffffu, v, o));
  if ((threadIdx.x & 31) == 0) red[threadIdx.x >> 5] = v;
  __syncthreads();
  v = red[threadIdx.x & 7];
  for (int o = 4; o > 0; o >>= 1) v = fmaxf(v, __shfl_xor_sync(0xffffffffu, v, o));
  __syncthreads();
  return v;
}
__device__ __forceinline__ float sm_block_sum(float v, float* red) {
  for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
  if ((threadIdx.x & 31) == 0) red[threadIdx.x >> 5] = v;
  __syncthreads();
  v = red[threadIdx.x & 7];
  for (int o = 4; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
  __syncthreads();
  return v;
}
__device__ __forceinline__ void sm_unpack(const uint4& u, float* f) {
  float2 a;
  a = unpack_bf16x2(u.x); f[0] = a.x; f[1] = a.y;
  a = unpack_bf16x2(u.y); f[2] = a.x; f[3] = a.y;
  a = unpack_bf16x2(u.z); f[4] = a.x; f[5] = a.y;
  a = unpack_bf16x2(u.w); f[6] = a.x; f[7] = a.y;
}
__device__ __forceinline__ uint4 sm_pack(const float* f) {
  uint4 u;
  u.x = pack_bf16x2(f[0], f[1]); u.y = pack_bf16x2(f[2], f[3]);
  u.z = pack_bf16x2(f[4], f[5]); u.w = pack_bf16x2(f[6], f[7]);
  return u;
}

__global__ void __launch_bounds__(kSmThreads)
softmax_rows_fwd_kernel(__nv_bfloat16* __restrict__ S, long long ld, int L, float scale, float* __restrict__ lse) {
  __shared__ float red[8];
  __nv_bfloat16* row = S + (long long)blockIdx.x * ld;
  const int nvec = L >> 3;
  const bool in_regs = nvec <= kSmThreads * kSmVecs;
  float v[kSmVecs][8];
  float m = -3.0e38f;
  if (in_regs) {
#pragma unroll
    for (int k = 0; k < kSmVecs; ++k) {
      const int i = threadIdx.x + k * kSmThreads;
      if (i < nvec) {
        sm_unpack(*reinterpret_cast<const uint4*>(row + 8 * i), v[k]);
#pragma unroll
        for (int j = 0; j < 8; ++j) { v[k][j] *= scale; m = fmaxf(m, v[k][j]); }
      }
    }
  } else {
    for (int i = threadIdx.x; i < nvec; i += kSmThreads) {
      float f[8];
      sm_unpack(*reinterpret_cast<const uint4*>(row + 8 * i), f);
      for (int j = 0; j < 8; ++j) m = fmaxf(m, f[j] * scale);
    }
  }
  m = sm_block_max(m, red);
  float s = 0.f;
  if (in_regs) {
#pragma unroll
    for (int k = 0; k < kSmVecs; ++k) {
      const int i = threadIdx.x + k * kSmThreads;
      if (i < nvec) {
#pragma unroll
        for (int j = 0; j < 8; ++j) { v[k][j] = __expf(v[k][j] - m); s += v[k][j]; }
      }
    }
  } else {
    for (int i = threadIdx.x; i < nvec; i += kSmThreads) {
      float f[8];
      sm_unpack(*reinterpret_cast<const uint4*>(row + 8 * i), f);
      for (int j = 0; j < 8; ++j) s += __expf(f[j] * scale - m);
    }
  }
  s = sm_block_sum(s, red);
  const float inv = 1.f / s;
  if (in_regs) {
#pragma unroll
    for (int k = 0; k < kSmVecs; ++k) {
      const int i = threadIdx.x + k * kSmThreads;
      if (i < nvec) {
#pragma unroll
        for (int j = 0; j < 8; ++j) v[k][j] *= inv;
        *reinterpret_cast<uint4*>(row + 8 * i) = sm_pack(v[k]);
      }
    }
  } else {
    for (int i = threadIdx.x; i < nvec; i += kSmThreads) {
      float f[8];
      sm_unpack(*reinterpret_cast<const uint4*>(row + 8 * i), f);
      for (int j = 0; j < 8; ++j) f[j] = __expf(f[j] * scale - m) * inv;
      *reinterpret_cast<uint4*>(row + 8 * i) = sm_pack(f);
    }
  }
  if (lse && threadIdx.x == 0) lse[blockIdx.x] = m + __logf(s);
}

__global__ void __launch_bounds__(kSmThreads)
softmax_rows_bwd_kernel(const __nv_bfloat16* __restrict__ P, long long ldp, __nv_bfloat16* __restrict__ dP, long long ldd, int L,
                        float scale) {
  __shared__ float red[8];
  const __nv_bfloat16* prow = P + (long long)blockIdx.x * ldp;
  __nv_bfloat16* drow = dP + (long long)blockIdx.x * ldd;
  const int nvec = L >> 3;
  float dot = 0.f;
  for (int i = threadIdx.x; i < nvec; i += kSmThreads) {
    float p[8], d[8];
    sm_unpack(*reinterpret_cast<const uint4*>(prow + 8 * i), p);
    sm_unpack(*reinterpret_cast<const uint4*>(drow + 8 * i), d);
#pragma unroll
    for (int j = 0; j < 8; ++j) dot += p[j] * d[j];
  }
  dot = sm_block_sum(dot, red);
  for (int i = threadIdx.x; i < nvec; i += kSmThreads) {
    float p[8], d[8];
    sm_unpack(*reinterpret_cast<const uint4*>(prow + 8 * i), p);
    sm_unpack(*reinterpret_cast<const uint4*>(drow + 8 * i), d);
#pragma unroll
    for (int j = 0; j < 8; ++j) d[j] = scale * p[j] * (d[j] - dot);
    *reinterpret_cast<uint4*>(drow + 8 * i) = sm_pack(d);
  }
}

}  // namespace pnm

extern "C" {

int pnm_softmax_rows_fwd(void* S, long long ld, long long rows, int L, float scale, float* lse, void* stream) {
  if (rows <= 0 || L <= 0 || (L & 7) || (ld & 7) || rows > 0x7fffffffLL) return -2;
  pnm::softmax_rows_fwd_kernel<<<(unsigned)rows, pnm::kSmThreads, 0, (cudaStream_t)stream>>>((__nv_bfloat16*)S, ld, L, scale, lse);
  return cudaGetLastError() == cudaSuccess ? 0 : -3;
}

int pnm_softmax_rows_bwd(const void* P, long long ldp, void* dP, long long ldd, long long rows, int L, float scale, void* stream) {
  if (rows <= 0 || L <= 0 || (L & 7) || (ldp & 7) || (ldd & 7) || rows > 0x7fffffffLL) return -2;
  pnm::softmax_rows_bwd_kernel<<<(unsigned)rows, pnm::kSmThreads, 0, (cudaStream_t)stream>>>((const __nv_bfloat16*)P, ldp,
                                                                                           (__nv_bfloat16*)dP, ldd, L, scale);
  return cudaGetLastError() == cudaSuccess ? 0 : -3;
}

}  // extern "C"
