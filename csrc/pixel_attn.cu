// Cross attention of grid pixels over their own variable-length lists of observation tokens, evaluated in token space.
//
// With K = tok Wk^T and V = tok Wv^T + b, the scores are tok . (Wk^T q) and the output is (sum_t w_t tok_t) Wv^T + b, so
// the two projections of every token are replaced by two dense GEMMs on the pixel side (done by the caller) and this
// kernel only sees   qk[P, H, Dt] (scaled),  tok[N, Dt],  cu[P + 1]   and returns   ctx[P, H, Dt] = softmax_t(tok qk^T) tok
// plus the log-sum-exp.  One warp owns one (pixel, block of 16 heads): the token tile is staged in shared memory once,
// lanes are tokens for the score / softmax phase and channels for the accumulation phase.  Dt = 32 * CPL, CPL <= 4.
// The backward recomputes the probabilities from the saved log-sum-exp and returns d qk and d tok (fp32, accumulated
// with atomics because the head blocks of a pixel run in different warps).
//
// Also here: the counting sort that groups observations by pixel (histogram, scan by the caller, scatter).

#include <cuda_bf16.h>
#include <cuda_runtime.h>
#include <math_constants.h>
#include <stdint.h>

#include "pnm_api.h"

namespace pnm {
namespace {

constexpr int kPaHeads = 16;     // heads per work item
constexpr int kPaTile = 32;      // tokens per tile (one per lane)
constexpr int kPaWarps = 4;      // warps per CTA

__device__ __forceinline__ float pa_warp_max(float v) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v = fmaxf(v, __shfl_xor_sync(0xffffffffu, v, o));
  return v;
}
__device__ __forceinline__ float pa_warp_sum(float v) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
  return v;
}
__device__ __forceinline__ float pa_f(float v) { return v; }
__device__ __forceinline__ float pa_f(__nv_bfloat16 v) { return __bfloat162float(v); }
template <typename T> __device__ __forceinline__ T pa_t(float v);
template <> __device__ __forceinline__ float pa_t<float>(float v) { return v; }
template <> __device__ __forceinline__ __nv_bfloat16 pa_t<__nv_bfloat16>(float v) { return __float2bfloat16(v); }

// per-warp shared memory: token tile [32][Dt + 1], head vectors [16][Dt] (x2 in the backward), weights [32][17] (x2)
template <int CPL> struct alignas(16) PaSmemFwd {
  float tile[kPaTile][32 * CPL + 1];
  alignas(16) float qk[kPaHeads][32 * CPL];
  alignas(16) float w[kPaTile][kPaHeads + 4];
};
template <int CPL> struct alignas(16) PaSmemBwd {
  float tile[kPaTile][32 * CPL + 1];
  alignas(16) float qk[kPaHeads][32 * CPL];
  alignas(16) float dc[kPaHeads][32 * CPL];
  alignas(16) float w[kPaTile][kPaHeads + 4];
  alignas(16) float ds[kPaTile][kPaHeads + 4];
};

template <typename T, int CPL>
__device__ __forceinline__ void stage_tokens(float (*tile)[32 * CPL + 1], const T* __restrict__ tok, int first, int n, int lane) {
  constexpr int Dt = 32 * CPL;
  for (int t = 0; t < n; ++t)
#pragma unroll
    for (int j = 0; j < CPL; ++j) tile[t][lane + 32 * j] = pa_f(tok[size_t(first + t) * Dt + lane + 32 * j]);
}

template <typename T, int CPL>
__global__ void __launch_bounds__(kPaWarps * 32)
pixel_attn_fwd_kernel(const T* __restrict__ qk, const T* __restrict__ tok, const int* __restrict__ cu, T* __restrict__ ctx,
                      float* __restrict__ lse, int P, int H) {
  constexpr int Dt = 32 * CPL;
  extern __shared__ __align__(16) unsigned char raw[];
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  PaSmemFwd<CPL>& s = reinterpret_cast<PaSmemFwd<CPL>*>(raw)[warp];
  const int blocks = (H + kPaHeads - 1) / kPaHeads;
  const long long items = (long long)P * blocks;
  for (long long it = (long long)blockIdx.x * kPaWarps + warp; it < items; it += (long long)gridDim.x * kPaWarps) {
    const int p = int(it / blocks), h0 = int(it % blocks) * kPaHeads;
    const int nh = min(kPaHeads, H - h0);
    const int start = cu[p], n = cu[p + 1] - start;
    for (int h = 0; h < kPaHeads; ++h)
#pragma unroll
      for (int j = 0; j < CPL; ++j)
        s.qk[h][lane + 32 * j] = h < nh ? pa_f(qk[(size_t(p) * H + h0 + h) * Dt + lane + 32 * j]) : 0.f;
    float m[kPaHeads], l[kPaHeads], acc[kPaHeads][CPL];
#pragma unroll
    for (int h = 0; h < kPaHeads; ++h) {
      m[h] = -CUDART_INF_F;
      l[h] = 0.f;
#pragma unroll
      for (int j = 0; j < CPL; ++j) acc[h][j] = 0.f;
    }
    for (int t0 = 0; t0 < n; t0 += kPaTile) {
      const int nt = min(kPaTile, n - t0);
      __syncwarp();
      stage_tokens<T, CPL>(s.tile, tok, start + t0, nt, lane);
      __syncwarp();
      // lanes = tokens: scores of this token against the 16 heads
      float sc[kPaHeads];
#pragma unroll
      for (int h = 0; h < kPaHeads; ++h) sc[h] = 0.f;
      if (lane < nt) {
        for (int c = 0; c < Dt; c += 4) {
          const float v0 = s.tile[lane][c], v1 = s.tile[lane][c + 1], v2 = s.tile[lane][c + 2], v3 = s.tile[lane][c + 3];
#pragma unroll
          for (int h = 0; h < kPaHeads; ++h) {
            const float4 q = *reinterpret_cast<const float4*>(&s.qk[h][c]);
            sc[h] = fmaf(v0, q.x, fmaf(v1, q.y, fmaf(v2, q.z, fmaf(v3, q.w, sc[h]))));
          }
        }
      }
#pragma unroll
      for (int h = 0; h < kPaHeads; ++h) {
        const float mine = lane < nt ? sc[h] : -CUDART_INF_F;
        const float mn = fmaxf(m[h], pa_warp_max(mine));
        const float corr = __expf(m[h] - mn);          // 0 on the first tile (m = -inf)
        const float w = lane < nt ? __expf(mine - mn) : 0.f;
        s.w[lane][h] = w;
        l[h] = l[h] * corr + w;                        // per-lane partial sum, reduced once at the end
        m[h] = mn;
#pragma unroll
        for (int j = 0; j < CPL; ++j) acc[h][j] *= corr;
      }
      __syncwarp();
      // lanes = channels: acc[h][c] += w[t][h] * tok[t][c]
      for (int t = 0; t < nt; ++t) {
        float v[CPL];
#pragma unroll
        for (int j = 0; j < CPL; ++j) v[j] = s.tile[t][lane + 32 * j];
#pragma unroll
        for (int h4 = 0; h4 < kPaHeads; h4 += 4) {
          const float4 w = *reinterpret_cast<const float4*>(&s.w[t][h4]);
#pragma unroll
          for (int j = 0; j < CPL; ++j) {
            acc[h4][j] = fmaf(w.x, v[j], acc[h4][j]);
            acc[h4 + 1][j] = fmaf(w.y, v[j], acc[h4 + 1][j]);
            acc[h4 + 2][j] = fmaf(w.z, v[j], acc[h4 + 2][j]);
            acc[h4 + 3][j] = fmaf(w.w, v[j], acc[h4 + 3][j]);
          }
        }
      }
    }
#pragma unroll
    for (int h = 0; h < kPaHeads; ++h) {
      const float tot = pa_warp_sum(l[h]);
      if (h < nh) {
        const float r = tot > 0.f ? 1.f / tot : 0.f;
#pragma unroll
        for (int j = 0; j < CPL; ++j) ctx[(size_t(p) * H + h0 + h) * Dt + lane + 32 * j] = pa_t<T>(acc[h][j] * r);
        if (lane == 0) lse[size_t(p) * H + h0 + h] = tot > 0.f ? m[h] + __logf(tot) : -CUDART_INF_F;
      }
    }
  }
}

template <typename T, int CPL, bool ATOMIC>
__global__ void __launch_bounds__(kPaWarps * 32)
pixel_attn_bwd_kernel(const T* __restrict__ qk, const T* __restrict__ tok, const int* __restrict__ cu, const T* __restrict__ dctx,
                      const float* __restrict__ lse, const float* __restrict__ delta, float* __restrict__ dqk,
                      float* __restrict__ dtok, int P, int H, long long N) {
  constexpr int Dt = 32 * CPL;
  extern __shared__ __align__(16) unsigned char raw[];
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  PaSmemBwd<CPL>& s = reinterpret_cast<PaSmemBwd<CPL>*>(raw)[warp];
  const int blocks = (H + kPaHeads - 1) / kPaHeads;
  const long long items = (long long)P * blocks;
  for (long long it = (long long)blockIdx.x * kPaWarps + warp; it < items; it += (long long)gridDim.x * kPaWarps) {
    const int p = int(it / blocks), h0 = int(it % blocks) * kPaHeads;
    const int nh = min(kPaHeads, H - h0);
    const int start = cu[p], n = cu[p + 1] - start;
    __syncwarp();
    for (int h = 0; h < kPaHeads; ++h)
#pragma unroll
      for (int j = 0; j < CPL; ++j) {
        const size_t g = (size_t(p) * H + h0 + h) * Dt + lane + 32 * j;
        s.qk[h][lane + 32 * j] = h < nh ? pa_f(qk[g]) : 0.f;
        s.dc[h][lane + 32 * j] = h < nh ? pa_f(dctx[g]) : 0.f;
      }
    float ls[kPaHeads], dl[kPaHeads], acc[kPaHeads][CPL];
#pragma unroll
    for (int h = 0; h < kPaHeads; ++h) {
      ls[h] = h < nh ? lse[size_t(p) * H + h0 + h] : 0.f;
      dl[h] = h < nh ? delta[size_t(p) * H + h0 + h] : 0.f;
#pragma unroll
      for (int j = 0; j < CPL; ++j) acc[h][j] = 0.f;
    }
    for (int t0 = 0; t0 < n; t0 += kPaTile) {
      const int nt = min(kPaTile, n - t0);
      __syncwarp();
      stage_tokens<T, CPL>(s.tile, tok, start + t0, nt, lane);
      __syncwarp();
      float sc[kPaHeads], dw[kPaHeads];
#pragma unroll
      for (int h = 0; h < kPaHeads; ++h) sc[h] = dw[h] = 0.f;
      if (lane < nt) {
        for (int c = 0; c < Dt; c += 4) {
          const float v0 = s.tile[lane][c], v1 = s.tile[lane][c + 1], v2 = s.tile[lane][c + 2], v3 = s.tile[lane][c + 3];
#pragma unroll
          for (int h = 0; h < kPaHeads; ++h) {
            const float4 q = *reinterpret_cast<const float4*>(&s.qk[h][c]);
            const float4 d = *reinterpret_cast<const float4*>(&s.dc[h][c]);
            sc[h] = fmaf(v0, q.x, fmaf(v1, q.y, fmaf(v2, q.z, fmaf(v3, q.w, sc[h]))));
            dw[h] = fmaf(v0, d.x, fmaf(v1, d.y, fmaf(v2, d.z, fmaf(v3, d.w, dw[h]))));
          }
        }
      }
#pragma unroll
      for (int h = 0; h < kPaHeads; ++h) {
        const float w = (lane < nt && h < nh) ? __expf(sc[h] - ls[h]) : 0.f;
        s.w[lane][h] = w;
        s.ds[lane][h] = w * (dw[h] - dl[h]);
      }
      __syncwarp();
      for (int t = 0; t < nt; ++t) {
        float v[CPL], g[CPL];
#pragma unroll
        for (int j = 0; j < CPL; ++j) {
          v[j] = s.tile[t][lane + 32 * j];
          g[j] = 0.f;
        }
#pragma unroll
        for (int h4 = 0; h4 < kPaHeads; h4 += 4) {
          const float4 w4 = *reinterpret_cast<const float4*>(&s.w[t][h4]);
          const float4 d4 = *reinterpret_cast<const float4*>(&s.ds[t][h4]);
          const float wv[4] = {w4.x, w4.y, w4.z, w4.w}, dv[4] = {d4.x, d4.y, d4.z, d4.w};
#pragma unroll
          for (int u = 0; u < 4; ++u)
#pragma unroll
            for (int j = 0; j < CPL; ++j) {
              acc[h4 + u][j] = fmaf(dv[u], v[j], acc[h4 + u][j]);
              g[j] = fmaf(wv[u], s.dc[h4 + u][lane + 32 * j], fmaf(dv[u], s.qk[h4 + u][lane + 32 * j], g[j]));
            }
        }
#pragma unroll
        for (int j = 0; j < CPL; ++j) {
          const size_t at = size_t(start + t0 + t) * Dt + lane + 32 * j;
          if (ATOMIC) atomicAdd(&dtok[at], g[j]);
          else dtok[size_t(h0 / kPaHeads) * size_t(N) * Dt + at] = g[j];     // one buffer per block of heads
        }
      }
    }
#pragma unroll
    for (int h = 0; h < kPaHeads; ++h)
      if (h < nh)
#pragma unroll
        for (int j = 0; j < CPL; ++j) dqk[(size_t(p) * H + h0 + h) * Dt + lane + 32 * j] = acc[h][j];
  }
}

__global__ void histogram_kernel(const int* __restrict__ idx, int* __restrict__ counts, long long n, int bins, int* __restrict__ bad) {
  for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += (long long)gridDim.x * blockDim.x) {
    const int b = idx[i];
    if (b < 0 || b >= bins) {
      atomicExch(bad, 1);
      continue;
    }
    atomicAdd(&counts[b], 1);
  }
}

__global__ void scatter_kernel(const int* __restrict__ idx, const int* __restrict__ offsets, int* __restrict__ cursor,
                               int* __restrict__ order, long long n, int bins) {
  for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += (long long)gridDim.x * blockDim.x) {
    const int b = idx[i];
    if (b < 0 || b >= bins) continue;
    order[offsets[b] + atomicAdd(&cursor[b], 1)] = int(i);
  }
}

int pa_grid(long long items) {
  int dev = 0, sms = 148;
  cudaGetDevice(&dev);
  cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev);
  const long long want = (items + kPaWarps - 1) / kPaWarps;
  const long long cap = (long long)sms * 8;
  return int(want < cap ? (want > 0 ? want : 1) : cap);
}

template <typename T, int CPL>
int launch_pa_fwd(const void* qk, const void* tok, const int* cu, void* ctx, float* lse, int P, int H, cudaStream_t st) {
  const size_t smem = sizeof(PaSmemFwd<CPL>) * kPaWarps;
  auto k = pixel_attn_fwd_kernel<T, CPL>;
  if (smem > 48 * 1024 && cudaFuncSetAttribute(k, cudaFuncAttributeMaxDynamicSharedMemorySize, int(smem)) != cudaSuccess) return -3;
  k<<<pa_grid((long long)P * ((H + kPaHeads - 1) / kPaHeads)), kPaWarps * 32, smem, st>>>((const T*)qk, (const T*)tok, cu, (T*)ctx, lse, P, H);
  return cudaGetLastError() == cudaSuccess ? 0 : -4;
}

template <typename T, int CPL>
int launch_pa_bwd(const void* qk, const void* tok, const int* cu, const void* dctx, const float* lse, const float* delta, float* dqk,
                  float* dtok, int P, int H, long long N, int atomic, cudaStream_t st) {
  const size_t smem = sizeof(PaSmemBwd<CPL>) * kPaWarps;
  auto k = atomic ? pixel_attn_bwd_kernel<T, CPL, true> : pixel_attn_bwd_kernel<T, CPL, false>;
  if (smem > 48 * 1024 && cudaFuncSetAttribute(k, cudaFuncAttributeMaxDynamicSharedMemorySize, int(smem)) != cudaSuccess) return -3;
  k<<<pa_grid((long long)P * ((H + kPaHeads - 1) / kPaHeads)), kPaWarps * 32, smem, st>>>((const T*)qk, (const T*)tok, cu, (const T*)dctx, lse,
                                                                                          delta, dqk, dtok, P, H, N);
  return cudaGetLastError() == cudaSuccess ? 0 : -4;
}

}  // namespace
}  // namespace pnm

#define PNM_PA_DISPATCH(FN, ...)                                                    \
  do {                                                                              \
    if (dtype == 0) {                                                               \
      if (Dt == 32) return pnm::FN<float, 1>(__VA_ARGS__);                          \
      if (Dt == 64) return pnm::FN<float, 2>(__VA_ARGS__);                          \
      if (Dt == 96) return pnm::FN<float, 3>(__VA_ARGS__);                          \
      if (Dt == 128) return pnm::FN<float, 4>(__VA_ARGS__);                         \
    } else if (dtype == 1) {                                                        \
      if (Dt == 32) return pnm::FN<__nv_bfloat16, 1>(__VA_ARGS__);                  \
      if (Dt == 64) return pnm::FN<__nv_bfloat16, 2>(__VA_ARGS__);                  \
      if (Dt == 96) return pnm::FN<__nv_bfloat16, 3>(__VA_ARGS__);                  \
      if (Dt == 128) return pnm::FN<__nv_bfloat16, 4>(__VA_ARGS__);                 \
    }                                                                               \
    return -1;                                                                      \
  } while (0)

// ctx[P, H, Dt] = softmax over the tokens cu[p] .. cu[p+1] of (tok qk[p, h]) applied to tok; lse[P, H] fp32 (-inf for empty pixels,
// whose ctx rows are zero).  dtype: 0 fp32, 1 bf16 (qk, tok, ctx).  Dt in {32, 64, 96, 128}.
extern "C" int pnm_pixel_attn_fwd(const void* qk, const void* tok, const int* cu, void* ctx, float* lse, int P, int H, int Dt, int dtype,
                                  void* stream) {
  if (!qk || !cu || !ctx || !lse || P <= 0 || H <= 0) return -1;
  cudaStream_t st = reinterpret_cast<cudaStream_t>(stream);
  PNM_PA_DISPATCH(launch_pa_fwd, qk, tok, cu, ctx, lse, P, H, st);
}

// dqk[P, H, Dt] (fp32, overwritten); delta[p, h] = sum_c dctx * ctx.  atomic = 1: dtok[N, Dt] fp32, zero on entry, accumulated with
// atomics; atomic = 0: dtok[ceil(H / 16), N, Dt] fp32, one slab per block of 16 heads, every element written once (the caller sums).
extern "C" int pnm_pixel_attn_bwd(const void* qk, const void* tok, const int* cu, const void* dctx, const float* lse, const float* delta,
                                  float* dqk, float* dtok, int P, int H, int Dt, long long N, int atomic, int dtype, void* stream) {
  if (!qk || !cu || !dctx || !lse || !delta || !dqk || !dtok || P <= 0 || H <= 0) return -1;
  cudaStream_t st = reinterpret_cast<cudaStream_t>(stream);
  PNM_PA_DISPATCH(launch_pa_bwd, qk, tok, cu, dctx, lse, delta, dqk, dtok, P, H, N, atomic, st);
}

// counts[bins] += histogram of idx[n] (int32); *bad is set to 1 when an index is outside [0, bins)
extern "C" int pnm_counting_histogram(const int* idx, int* counts, long long n, int bins, int* bad, void* stream) {
  if (!idx || !counts || !bad || n <= 0 || bins <= 0) return -1;
  const int grid = int((n + 255) / 256 < 148 * 8 ? (n + 255) / 256 : 148 * 8);
  pnm::histogram_kernel<<<grid, 256, 0, reinterpret_cast<cudaStream_t>(stream)>>>(idx, counts, n, bins, bad);
  return cudaGetLastError() == cudaSuccess ? 0 : -4;
}

// order[offsets[b] + k] = i for the k-th visited element i with idx[i] == b; cursor[bins] must be zero on entry
extern "C" int pnm_counting_scatter(const int* idx, const int* offsets, int* cursor, int* order, long long n, int bins, void* stream) {
  if (!idx || !offsets || !cursor || !order || n <= 0 || bins <= 0) return -1;
  const int grid = int((n + 255) / 256 < 148 * 8 ? (n + 255) / 256 : 148 * 8);
  pnm::scatter_kernel<<<grid, 256, 0, reinterpret_cast<cudaStream_t>(stream)>>>(idx, offsets, cursor, order, n, bins);
  return cudaGetLastError() == cudaSuccess ? 0 : -4;
}
