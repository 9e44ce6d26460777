// Graph primitives for message passing on bf16 feature rows (fp32 accumulation).
//
//   gather_rows  : out[e, :] = in[idx[e], :]                      (edge <- node)
//   segment_sum  : out[n, :] = (out[n, :] +) scale_n * sum_{k in [off[n], off[n+1])} in[perm[k], :]
//                  (node <- incident edges; edges pre-sorted by segment through `perm`,
//                   deterministic: no atomics, fixed summation order)
// Each 16-byte chunk (8 channels) of a row is owned by one thread; a row of C channels is
// covered by C/8 neighbouring lanes, so global accesses are coalesced 16-byte vectors.
#pragma once
#include "common.cuh"

namespace pnm {

__global__ void __launch_bounds__(256)
gather_rows_kernel(const __nv_bfloat16* __restrict__ in, int ldi, const int* __restrict__ idx,
                   __nv_bfloat16* __restrict__ out, int ldo, long long E, int C) {
  const int cpr = C >> 3;  // 16-byte chunks per row
  const long long total = E * cpr;
  for (long long t = (long long)blockIdx.x * blockDim.x + threadIdx.x; t < total;
       t += (long long)gridDim.x * blockDim.x) {
    const long long e = t / cpr;
    const int c = int(t - e * cpr) << 3;
    const long long src = idx ? (long long)__ldg(idx + e) : e;
    const uint4 v = *reinterpret_cast<const uint4*>(in + src * ldi + c);
    *reinterpret_cast<uint4*>(out + e * (long long)ldo + c) = v;
  }
}

// mode: 0 = sum, 1 = mean (divide by the segment length, empty segments give 0)
__global__ void __launch_bounds__(256)
segment_sum_kernel(const __nv_bfloat16* __restrict__ in, int ldi, const int* __restrict__ perm,
                   const int* __restrict__ offsets, __nv_bfloat16* __restrict__ out, int ldo, long long N, int C,
                   int accumulate, int mode) {
  const int cpr = C >> 3;
  const long long total = N * cpr;
  for (long long t = (long long)blockIdx.x * blockDim.x + threadIdx.x; t < total;
       t += (long long)gridDim.x * blockDim.x) {
    const long long n = t / cpr;
    const int c = int(t - n * cpr) << 3;
    const int k0 = __ldg(offsets + n), k1 = __ldg(offsets + n + 1);
    float acc[8] = {0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f};
    for (int k = k0; k < k1; ++k) {
      const long long row = perm ? (long long)__ldg(perm + k) : (long long)k;
      const uint4 v = *reinterpret_cast<const uint4*>(in + row * ldi + c);
      float2 f;
      f = unpack_bf16x2(v.x); acc[0] += f.x; acc[1] += f.y;
      f = unpack_bf16x2(v.y); acc[2] += f.x; acc[3] += f.y;
      f = unpack_bf16x2(v.z); acc[4] += f.x; acc[5] += f.y;
      f = unpack_bf16x2(v.w); acc[6] += f.x; acc[7] += f.y;
    }
    if (mode == 1 && k1 > k0) {
      const float inv = 1.f / float(k1 - k0);
#pragma unroll
      for (int j = 0; j < 8; ++j) acc[j] *= inv;
    }
    __nv_bfloat16* dst = out + n * (long long)ldo + c;
    if (accumulate) {
      const uint4 o = *reinterpret_cast<const uint4*>(dst);
      float2 f;
      f = unpack_bf16x2(o.x); acc[0] += f.x; acc[1] += f.y;
      f = unpack_bf16x2(o.y); acc[2] += f.x; acc[3] += f.y;
      f = unpack_bf16x2(o.z); acc[4] += f.x; acc[5] += f.y;
      f = unpack_bf16x2(o.w); acc[6] += f.x; acc[7] += f.y;
    }
    uint4 w;
    w.x = pack_bf16x2(acc[0], acc[1]); w.y = pack_bf16x2(acc[2], acc[3]);
    w.z = pack_bf16x2(acc[4], acc[5]); w.w = pack_bf16x2(acc[6], acc[7]);
    *reinterpret_cast<uint4*>(dst) = w;
  }
}

// gather with per-row scale (backward of mean aggregation): out[e,:] = in[idx[e],:] * scale[idx[e]]
__global__ void __launch_bounds__(256)
gather_rows_scaled_kernel(const __nv_bfloat16* __restrict__ in, int ldi, const int* __restrict__ idx,
                          const float* __restrict__ scale, __nv_bfloat16* __restrict__ out, int ldo, long long E,
                          int C) {
  const int cpr = C >> 3;
  const long long total = E * cpr;
  for (long long t = (long long)blockIdx.x * blockDim.x + threadIdx.x; t < total;
       t += (long long)gridDim.x * blockDim.x) {
    const long long e = t / cpr;
    const int c = int(t - e * cpr) << 3;
    const long long src = (long long)__ldg(idx + e);
    const float s = __ldg(scale + src);
    const uint4 v = *reinterpret_cast<const uint4*>(in + src * ldi + c);
    float2 a = unpack_bf16x2(v.x), b = unpack_bf16x2(v.y), cc = unpack_bf16x2(v.z), d = unpack_bf16x2(v.w);
    uint4 w;
    w.x = pack_bf16x2(a.x * s, a.y * s); w.y = pack_bf16x2(b.x * s, b.y * s);
    w.z = pack_bf16x2(cc.x * s, cc.y * s); w.w = pack_bf16x2(d.x * s, d.y * s);
    *reinterpret_cast<uint4*>(out + e * (long long)ldo + c) = w;
  }
}

inline int grid_for(long long work_items, int threads, int num_sms) {
  long long want = (work_items + threads - 1) / threads;
  long long cap = (long long)num_sms * 16;
  int g = (int)(want < cap ? want : cap);
  return g < 1 ? 1 : g;
}

inline int launch_gather_rows(const void* in, int ldi, const int* idx, const float* scale, void* out, int ldo,
                              long long E, int C, int num_sms, cudaStream_t st) {
  if (C % 8 || ldi % 8 || ldo % 8) return -40;
  if (E <= 0) return 0;
  const int grid = grid_for(E * (C >> 3), 256, num_sms);
  if (scale)
    gather_rows_scaled_kernel<<<grid, 256, 0, st>>>((const __nv_bfloat16*)in, ldi, idx, scale, (__nv_bfloat16*)out, ldo, E, C);
  else
    gather_rows_kernel<<<grid, 256, 0, st>>>((const __nv_bfloat16*)in, ldi, idx, (__nv_bfloat16*)out, ldo, E, C);
  return cudaGetLastError() == cudaSuccess ? 0 : -41;
}

inline int launch_segment_sum(const void* in, int ldi, const int* perm, const int* offsets, void* out, int ldo,
                              long long N, int C, int accumulate, int mode, int num_sms, cudaStream_t st) {
  if (C % 8 || ldi % 8 || ldo % 8) return -42;
  if (N <= 0) return 0;
  const int grid = grid_for(N * (C >> 3), 256, num_sms);
  segment_sum_kernel<<<grid, 256, 0, st>>>((const __nv_bfloat16*)in, ldi, perm, offsets, (__nv_bfloat16*)out, ldo, N, C,
                                           accumulate, mode);
  return cudaGetLastError() == cudaSuccess ? 0 : -43;
}

}  // namespace pnm
