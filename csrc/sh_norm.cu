// Normalisation of spherical-harmonic feature grids [B, L, M, 2, C] (degree l, order m, real/imaginary, channel).
//
// One kernel family covers the three equivariant norms (RMS over all degrees, per-degree layer norm, and the tied
// variant with a plain layer norm on l = 0): degrees are partitioned into groups, every group g gets
//     S_g = (1 / C) * sum_{l in g} sum_m w[l, m] sum_r sum_c xc[l, m, r, c]^2 ,   inv_g = rsqrt(S_g + eps)
// where xc is the masked input with (optionally) the channel mean removed from the (l, m, r) = (0, 0, 0) row, and
//     y[l, m, r, c] = mask[l, m, r] * (xc * inv_{g(l)} * a[l, c] + [l = m = r = 0] * bias[c]).
// A CTA owns one sample at a time: the valid rows are read once into shared memory, the group statistics are
// reduced there, and the output is written once (masked rows are written as zeros and never read).  The backward
// kernel keeps x and dy of the sample in shared memory, and accumulates the affine-weight and bias gradients of all
// the samples a CTA visits in shared memory; one partial per CTA is written at the end.

#include <cuda_bf16.h>
#include <cuda_fp16.h>
#include <cuda_runtime.h>
#include <stdint.h>

#include "pnm_api.h"

namespace pnm {
namespace {

constexpr int kShThreads = 256;

__device__ __forceinline__ float warp_sum(float v) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
  return v;
}

__device__ __forceinline__ float to_f(float v) { return v; }
__device__ __forceinline__ float to_f(__nv_bfloat16 v) { return __bfloat162float(v); }
__device__ __forceinline__ float to_f(__half v) { return __half2float(v); }
template <typename T> __device__ __forceinline__ T from_f(float v);
template <> __device__ __forceinline__ float from_f<float>(float v) { return v; }
template <> __device__ __forceinline__ __nv_bfloat16 from_f<__nv_bfloat16>(float v) { return __float2bfloat16(v); }
template <> __device__ __forceinline__ __half from_f<__half>(float v) { return __float2half(v); }

// V consecutive elements as one access (V = 4: 16 bytes of float, 8 bytes of a 16-bit type; V = 1: scalar)
template <typename T, int V> struct alignas(sizeof(T) * V) Pack { T v[V]; };

template <typename T, int V>
__device__ __forceinline__ void load_row(const T* __restrict__ src, float* __restrict__ dst, int C, int lane) {
  for (int c = lane * V; c < C; c += 32 * V) {
    const Pack<T, V> p = *reinterpret_cast<const Pack<T, V>*>(src + c);
#pragma unroll
    for (int i = 0; i < V; ++i) dst[c + i] = to_f(p.v[i]);
  }
}

template <typename T, int V>
__device__ __forceinline__ void zero_row(T* __restrict__ dst, int C, int lane) {
  Pack<T, V> z;
#pragma unroll
  for (int i = 0; i < V; ++i) z.v[i] = from_f<T>(0.f);
  for (int c = lane * V; c < C; c += 32 * V) *reinterpret_cast<Pack<T, V>*>(dst + c) = z;
}

// loads the valid rows of one sample into xs, centres row 0, leaves sum_c xc^2 of every row in pos_sum
template <typename T, int V>
__device__ __forceinline__ void stage_sample(const T* __restrict__ xb, float* xs, float* pos_sum, const float* __restrict__ mask,
                                             int P, int C, int subtract_mean, int warp, int lane, int nw) {
  for (int p = warp; p < P; p += nw) {
    if (mask[p] == 0.f) {
      if (lane == 0) pos_sum[p] = 0.f;
      continue;
    }
    float* row = xs + size_t(p) * C;
    load_row<T, V>(xb + size_t(p) * C, row, C, lane);
    __syncwarp();
    float mean = 0.f;
    if (p == 0 && subtract_mean) {
      float s = 0.f;
      for (int c = lane; c < C; c += 32) s += row[c];
      mean = warp_sum(s) / float(C);
    }
    float q = 0.f;
    for (int c = lane; c < C; c += 32) {
      const float v = row[c] - mean;
      row[c] = v;
      q = fmaf(v, v, q);
    }
    q = warp_sum(q);
    if (lane == 0) pos_sum[p] = q;
  }
}

__device__ __forceinline__ void group_inverse(const float* pos_sum, float* inv, const float* __restrict__ wstat,
                                              const int* __restrict__ group, int L, int M, int C, float eps) {
  const int g = threadIdx.x;
  if (g < L) {
    float S = 0.f;
    for (int l = 0; l < L; ++l) {
      if (group[l] != g) continue;
      for (int m = 0; m < M; ++m) S += wstat[l * M + m] * (pos_sum[(l * M + m) * 2] + pos_sum[(l * M + m) * 2 + 1]);
    }
    inv[g] = rsqrtf(S / float(C) + eps);
  }
}

template <typename T, int V>
__global__ void __launch_bounds__(kShThreads)
sh_norm_fwd_kernel(const T* __restrict__ x, T* __restrict__ y, const float* __restrict__ aw, const float* __restrict__ bias,
                   const float* __restrict__ wstat, const float* __restrict__ mask, const int* __restrict__ group, long long B,
                   int L, int M, int C, float eps, int subtract_mean) {
  extern __shared__ float sm[];
  const int P = L * M * 2;
  float* xs = sm;
  float* pos_sum = xs + size_t(P) * C;
  float* inv = pos_sum + P;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31, nw = blockDim.x >> 5;
  for (long long b = blockIdx.x; b < B; b += gridDim.x) {
    const T* xb = x + size_t(b) * P * C;
    T* yb = y + size_t(b) * P * C;
    stage_sample<T, V>(xb, xs, pos_sum, mask, P, C, subtract_mean, warp, lane, nw);
    __syncthreads();
    group_inverse(pos_sum, inv, wstat, group, L, M, C, eps);
    __syncthreads();
    for (int p = warp; p < P; p += nw) {
      T* out = yb + size_t(p) * C;
      if (mask[p] == 0.f) {
        zero_row<T, V>(out, C, lane);
        continue;
      }
      const int l = p / (2 * M);
      const float s = inv[group[l]];
      const float* row = xs + size_t(p) * C;
      const float* a = aw + size_t(l) * C;
      const bool add_bias = (p == 0) && bias != nullptr;
      for (int c = lane * V; c < C; c += 32 * V) {
        Pack<T, V> o;
#pragma unroll
        for (int i = 0; i < V; ++i) {
          float v = row[c + i] * s * a[c + i];
          if (add_bias) v += bias[c + i];
          o.v[i] = from_f<T>(v);
        }
        *reinterpret_cast<Pack<T, V>*>(out + c) = o;
      }
    }
    __syncthreads();
  }
}

template <typename T, int V>
__global__ void __launch_bounds__(kShThreads)
sh_norm_bwd_kernel(const T* __restrict__ x, const T* __restrict__ dy, T* __restrict__ dx, const float* __restrict__ aw,
                   const float* __restrict__ wstat, const float* __restrict__ mask, const int* __restrict__ group,
                   float* __restrict__ daw_part, float* __restrict__ dbias_part, long long B, int L, int M, int C, float eps,
                   int subtract_mean) {
  extern __shared__ float sm[];
  const int P = L * M * 2;
  float* xs = sm;                          // centred input
  float* gs = xs + size_t(P) * C;          // dy, then dy * a
  float* daw_s = gs + size_t(P) * C;       // [L, C]
  float* dbias_s = daw_s + size_t(L) * C;  // [C]
  float* pos_sum = dbias_s + C;
  float* pos_dot = pos_sum + P;
  float* inv = pos_dot + P;
  float* dotg = inv + L;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31, nw = blockDim.x >> 5;
  for (int i = threadIdx.x; i < (L + 1) * C; i += blockDim.x) daw_s[i] = 0.f;   // daw_s and dbias_s are contiguous
  __syncthreads();
  for (long long b = blockIdx.x; b < B; b += gridDim.x) {
    const size_t off = size_t(b) * P * C;
    stage_sample<T, V>(x + off, xs, pos_sum, mask, P, C, subtract_mean, warp, lane, nw);
    for (int p = warp; p < P; p += nw)
      if (mask[p] != 0.f) load_row<T, V>(dy + off + size_t(p) * C, gs + size_t(p) * C, C, lane);
    __syncthreads();
    group_inverse(pos_sum, inv, wstat, group, L, M, C, eps);
    __syncthreads();
    // weight / bias gradients of this sample, g = dy * a, and sum_c g * xc per row
    for (int p = warp; p < P; p += nw) {
      if (mask[p] == 0.f) {
        if (lane == 0) pos_dot[p] = 0.f;
        continue;
      }
      const int l = p / (2 * M);
      const float s = inv[group[l]];
      const float* a = aw + size_t(l) * C;
      float dot = 0.f;
      for (int c = lane; c < C; c += 32) {
        const float d = gs[size_t(p) * C + c], v = xs[size_t(p) * C + c];
        atomicAdd(&daw_s[l * C + c], d * v * s);
        if (p == 0) dbias_s[c] += d;     // row 0 belongs to one warp of the CTA, lanes own distinct channels
        const float g = d * a[c];
        gs[size_t(p) * C + c] = g;
        dot = fmaf(g, v, dot);
      }
      dot = warp_sum(dot);
      if (lane == 0) pos_dot[p] = dot;
    }
    __syncthreads();
    if (threadIdx.x < L) {
      const int g = threadIdx.x;
      float D = 0.f;
      for (int l = 0; l < L; ++l)
        if (group[l] == g)
          for (int q = l * M * 2; q < (l + 1) * M * 2; ++q) D += pos_dot[q];
      dotg[g] = D;
    }
    __syncthreads();
    for (int p = warp; p < P; p += nw) {
      T* out = dx + off + size_t(p) * C;
      if (mask[p] == 0.f) {
        zero_row<T, V>(out, C, lane);
        continue;
      }
      const int l = p / (2 * M), m = (p / 2) % M;
      const int g = group[l];
      const float s = inv[g];
      const float k = wstat[l * M + m] * s * s * s * dotg[g] / float(C);
      float* grow = gs + size_t(p) * C;
      const float* row = xs + size_t(p) * C;
      float sum = 0.f;
      for (int c = lane; c < C; c += 32) {
        const float d = s * grow[c] - k * row[c];
        grow[c] = d;
        sum += d;
      }
      float mean = 0.f;
      if (p == 0 && subtract_mean) mean = warp_sum(sum) / float(C);
      __syncwarp();
      for (int c = lane * V; c < C; c += 32 * V) {
        Pack<T, V> o;
#pragma unroll
        for (int i = 0; i < V; ++i) o.v[i] = from_f<T>(grow[c + i] - mean);
        *reinterpret_cast<Pack<T, V>*>(out + c) = o;
      }
    }
    __syncthreads();
  }
  for (int i = threadIdx.x; i < L * C; i += blockDim.x) daw_part[size_t(blockIdx.x) * L * C + i] = daw_s[i];
  for (int i = threadIdx.x; i < C; i += blockDim.x) dbias_part[size_t(blockIdx.x) * C + i] = dbias_s[i];
}

// ---------------------------------------------------------------------------------------------------------------------
// Register-resident variants for C = 32 * CPL (CPL = 1, 2, 4) and at most R rows per warp: a warp always owns the same rows
// (p = warp + k * warps), a lane always owns the same CPL consecutive channels, so the sample lives in registers, all
// loads of a sample are issued before the first use, and the affine-weight / bias gradients accumulate in registers over
// all the samples a CTA visits (one shared-memory reduction per CTA at the end instead of one atomic per element).
constexpr int kShRows = 6;

template <typename T, int CPL>
__device__ __forceinline__ void load_chunk(const T* __restrict__ src, float (&dst)[CPL]) {
  const Pack<T, CPL> p = *reinterpret_cast<const Pack<T, CPL>*>(src);
#pragma unroll
  for (int i = 0; i < CPL; ++i) dst[i] = to_f(p.v[i]);
}

template <typename T, int CPL>
__device__ __forceinline__ void store_chunk(T* __restrict__ dst, const float (&src)[CPL]) {
  Pack<T, CPL> p;
#pragma unroll
  for (int i = 0; i < CPL; ++i) p.v[i] = from_f<T>(src[i]);
  *reinterpret_cast<Pack<T, CPL>*>(dst) = p;
}

// sum over the positions of each group of wpos[p] * val[p], evaluated redundantly by every warp (no broadcast barrier):
// lane l first sums the 2 M positions of degree l (L <= 32), then the degrees of one group are combined by a warp
// reduction per row of this warp (a single reduction when there is one group).  out[k] = sum for the group of row k.
template <int R>
__device__ __forceinline__ void group_sums(const float* val, const float* wpos, const int* gid, int L, int M, int G, int lane,
                                           const int (&gk)[R], float (&out)[R]) {
  float sl = 0.f;
  int gl = -2;
  if (lane < L) {
    gl = gid[lane * 2 * M];
    for (int q = lane * 2 * M; q < (lane + 1) * 2 * M; ++q) sl = fmaf(wpos[q], val[q], sl);
  }
  if (G == 1) {
    const float tot = warp_sum(sl);
#pragma unroll
    for (int k = 0; k < R; ++k) out[k] = tot;
    return;
  }
#pragma unroll
  for (int k = 0; k < R; ++k) out[k] = warp_sum(gl == gk[k] ? sl : 0.f);
}

template <typename T, int CPL>
__global__ void __launch_bounds__(512)
sh_norm_fwd_reg_kernel(const T* __restrict__ x, T* __restrict__ y, const float* __restrict__ aw, const float* __restrict__ bias,
                       const float* __restrict__ wstat, const float* __restrict__ mask, const int* __restrict__ group, long long B,
                       int L, int M, float eps, int subtract_mean) {
  constexpr int C = 32 * CPL;
  extern __shared__ float sm[];
  const int P = L * M * 2;
  float* pos_sum = sm;                       // [2][P], ping-pong over samples
  float* wpos = pos_sum + 2 * P;             // [P] statistic weight of the position
  int* gid = reinterpret_cast<int*>(wpos + P);
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31, nw = blockDim.x >> 5;
  const int c0 = lane * CPL;
  int G = 0;
  for (int l = 0; l < L; ++l) G = max(G, group[l] + 1);
  for (int p = threadIdx.x; p < P; p += blockDim.x) {
    wpos[p] = wstat[p / 2];
    gid[p] = group[p / (2 * M)];
  }
  bool valid[kShRows];
  int gk[kShRows];
#pragma unroll
  for (int k = 0; k < kShRows; ++k) {
    const int p = warp + k * nw;
    valid[k] = p < P && mask[p] != 0.f;
    gk[k] = p < P ? group[p / (2 * M)] : -1;
  }
  float bv[CPL];
#pragma unroll
  for (int i = 0; i < CPL; ++i) bv[i] = (bias != nullptr && warp == 0) ? bias[c0 + i] : 0.f;
  __syncthreads();
  int par = 0;
  for (long long b = blockIdx.x; b < B; b += gridDim.x, par ^= 1) {
    const T* xb = x + size_t(b) * P * C + c0;
    T* yb = y + size_t(b) * P * C + c0;
    float* ps = pos_sum + par * P;
    float xr[kShRows][CPL];
#pragma unroll
    for (int k = 0; k < kShRows; ++k)
      if (valid[k]) load_chunk<T, CPL>(xb + size_t(warp + k * nw) * C, xr[k]);
#pragma unroll
    for (int k = 0; k < kShRows; ++k) {
      const int p = warp + k * nw;
      if (p >= P) continue;
      float q = 0.f;
      if (valid[k]) {
        if (p == 0 && subtract_mean) {
          float s = 0.f;
#pragma unroll
          for (int i = 0; i < CPL; ++i) s += xr[k][i];
          const float mean = warp_sum(s) / float(C);
#pragma unroll
          for (int i = 0; i < CPL; ++i) xr[k][i] -= mean;
        }
#pragma unroll
        for (int i = 0; i < CPL; ++i) q = fmaf(xr[k][i], xr[k][i], q);
        q = warp_sum(q);
      }
      if (lane == 0) ps[p] = q;
    }
    // one barrier per sample: the other half of pos_sum is only rewritten after the next barrier
    __syncthreads();
    float S[kShRows];
#pragma unroll
    for (int k = 0; k < kShRows; ++k) S[k] = 0.f;
    group_sums<kShRows>(ps, wpos, gid, L, M, G, lane, gk, S);
#pragma unroll
    for (int k = 0; k < kShRows; ++k) {
      const int p = warp + k * nw;
      if (p >= P) continue;
      float o[CPL];
      if (valid[k]) {
        const float sc = rsqrtf(S[k] / float(C) + eps);
        float a[CPL];
        load_chunk<float, CPL>(aw + (p / (2 * M)) * C + c0, a);
#pragma unroll
        for (int i = 0; i < CPL; ++i) o[i] = xr[k][i] * sc * a[i] + (p == 0 ? bv[i] : 0.f);
      } else {
#pragma unroll
        for (int i = 0; i < CPL; ++i) o[i] = 0.f;
      }
      store_chunk<T, CPL>(yb + size_t(p) * C, o);
    }
  }
}

template <typename T, int CPL>
__global__ void __launch_bounds__(512)
sh_norm_bwd_reg_kernel(const T* __restrict__ x, const T* __restrict__ dy, T* __restrict__ dx, const float* __restrict__ aw,
                       const float* __restrict__ wstat, const float* __restrict__ mask, const int* __restrict__ group,
                       float* __restrict__ daw_part, float* __restrict__ dbias_part, long long B, int L, int M, float eps,
                       int subtract_mean) {
  constexpr int C = 32 * CPL;
  extern __shared__ float sm[];
  const int P = L * M * 2;
  float* daw_s = sm;                       // [L, C] then [C] for the bias
  float* pos_sum = daw_s + size_t(L + 1) * C;   // [2][P]
  float* pos_dot = pos_sum + 2 * P;             // [2][P]
  float* wpos = pos_dot + 2 * P;                // [P]
  float* ones = wpos + P;                       // [P]
  int* gid = reinterpret_cast<int*>(ones + P);
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31, nw = blockDim.x >> 5;
  const int c0 = lane * CPL;
  for (int i = threadIdx.x; i < (L + 1) * C; i += blockDim.x) daw_s[i] = 0.f;
  int G = 0;
  for (int l = 0; l < L; ++l) G = max(G, group[l] + 1);
  for (int p = threadIdx.x; p < P; p += blockDim.x) {
    wpos[p] = wstat[p / 2];
    ones[p] = 1.f;
    gid[p] = group[p / (2 * M)];
  }
  bool valid[kShRows];
  int gk[kShRows];
  float a[kShRows][CPL], dacc[kShRows][CPL], bacc[CPL];
#pragma unroll
  for (int k = 0; k < kShRows; ++k) {
    const int p = warp + k * nw;
    valid[k] = p < P && mask[p] != 0.f;
    const int l = p < P ? p / (2 * M) : 0;
    gk[k] = p < P ? group[l] : -1;
#pragma unroll
    for (int i = 0; i < CPL; ++i) {
      a[k][i] = aw[l * C + c0 + i];
      dacc[k][i] = 0.f;
    }
  }
#pragma unroll
  for (int i = 0; i < CPL; ++i) bacc[i] = 0.f;
  __syncthreads();
  int par = 0;
  for (long long b = blockIdx.x; b < B; b += gridDim.x, par ^= 1) {
    const size_t off = size_t(b) * P * C + c0;
    float* ps = pos_sum + par * P;
    float* pd = pos_dot + par * P;
    float xr[kShRows][CPL], gr[kShRows][CPL];
#pragma unroll
    for (int k = 0; k < kShRows; ++k)
      if (valid[k]) {
        load_chunk<T, CPL>(x + off + size_t(warp + k * nw) * C, xr[k]);
        load_chunk<T, CPL>(dy + off + size_t(warp + k * nw) * C, gr[k]);
      }
#pragma unroll
    for (int k = 0; k < kShRows; ++k) {
      const int p = warp + k * nw;
      if (p >= P) continue;
      float q = 0.f;
      if (valid[k]) {
        if (p == 0 && subtract_mean) {
          float s = 0.f;
#pragma unroll
          for (int i = 0; i < CPL; ++i) s += xr[k][i];
          const float mean = warp_sum(s) / float(C);
#pragma unroll
          for (int i = 0; i < CPL; ++i) xr[k][i] -= mean;
        }
#pragma unroll
        for (int i = 0; i < CPL; ++i) q = fmaf(xr[k][i], xr[k][i], q);
        q = warp_sum(q);
      }
      if (lane == 0) ps[p] = q;
    }
    __syncthreads();
    float S[kShRows], D[kShRows];
#pragma unroll
    for (int k = 0; k < kShRows; ++k) S[k] = D[k] = 0.f;
    group_sums<kShRows>(ps, wpos, gid, L, M, G, lane, gk, S);
#pragma unroll
    for (int k = 0; k < kShRows; ++k) {
      const int p = warp + k * nw;
      if (p >= P) continue;
      float dot = 0.f;
      if (valid[k]) {
        const float sc = rsqrtf(S[k] / float(C) + eps);
        S[k] = sc;
#pragma unroll
        for (int i = 0; i < CPL; ++i) {
          const float d = gr[k][i], v = xr[k][i];
          dacc[k][i] = fmaf(d * v, sc, dacc[k][i]);
          if (p == 0) bacc[i] += d;
          const float g = d * a[k][i];
          gr[k][i] = g;
          dot = fmaf(g, v, dot);
        }
        dot = warp_sum(dot);
      }
      if (lane == 0) pd[p] = dot;
    }
    __syncthreads();
    group_sums<kShRows>(pd, ones, gid, L, M, G, lane, gk, D);
#pragma unroll
    for (int k = 0; k < kShRows; ++k) {
      const int p = warp + k * nw;
      if (p >= P) continue;
      float o[CPL];
      if (valid[k]) {
        const float sc = S[k];
        const float kc = wpos[p] * sc * sc * sc * D[k] / float(C);
        float sum = 0.f;
#pragma unroll
        for (int i = 0; i < CPL; ++i) {
          o[i] = sc * gr[k][i] - kc * xr[k][i];
          sum += o[i];
        }
        if (p == 0 && subtract_mean) {
          const float mean = warp_sum(sum) / float(C);
#pragma unroll
          for (int i = 0; i < CPL; ++i) o[i] -= mean;
        }
      } else {
#pragma unroll
        for (int i = 0; i < CPL; ++i) o[i] = 0.f;
      }
      store_chunk<T, CPL>(dx + off + size_t(p) * C, o);
    }
  }
  __syncthreads();
#pragma unroll
  for (int k = 0; k < kShRows; ++k) {
    const int p = warp + k * nw;
    if (p < P && valid[k]) {
      const int l = p / (2 * M);
#pragma unroll
      for (int i = 0; i < CPL; ++i) atomicAdd(&daw_s[l * C + c0 + i], dacc[k][i]);
    }
  }
  if (warp == 0) {
#pragma unroll
    for (int i = 0; i < CPL; ++i) daw_s[L * C + c0 + i] = bacc[i];
  }
  __syncthreads();
  for (int i = threadIdx.x; i < L * C; i += blockDim.x) daw_part[size_t(blockIdx.x) * L * C + i] = daw_s[i];
  for (int i = threadIdx.x; i < C; i += blockDim.x) dbias_part[size_t(blockIdx.x) * C + i] = daw_s[L * C + i];
}

// threads of the register-resident variants (0: not applicable)
int reg_threads(int L, int M, int C) {
  const int P = L * M * 2;
  if ((C != 32 && C != 64 && C != 128) || L > 32) return 0;
  if (P <= 8 * kShRows) return 256;
  if (P <= 16 * kShRows) return 512;
  return 0;
}
size_t reg_fwd_smem(int L, int M) { return size_t(L) * M * 2 * 4 * sizeof(float); }
size_t reg_bwd_smem(int L, int M, int C) { return (size_t(L + 1) * C + size_t(L) * M * 2 * 7) * sizeof(float); }

int reg_grid(int threads, int ctas_per_sm, long long B) {
  int dev = 0, sms = 148;
  cudaGetDevice(&dev);
  cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev);
  const long long g = (long long)sms * ctas_per_sm;
  return int(g < B ? g : B);
}

size_t fwd_smem(int L, int M, int C) { return (size_t(L) * M * 2 * C + size_t(L) * M * 2 + L) * sizeof(float); }
size_t bwd_smem(int L, int M, int C) {
  return (size_t(L) * M * 2 * C * 2 + size_t(L + 1) * C + size_t(L) * M * 2 * 2 + 2 * L) * sizeof(float);
}
constexpr size_t kMaxSmem = 200 * 1024;

int grid_for(size_t smem, long long B) {
  int dev = 0, sms = 148;
  cudaGetDevice(&dev);
  cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev);
  int per_sm = int((220 * 1024) / (smem + 1024));
  per_sm = per_sm < 1 ? 1 : (per_sm > 8 ? 8 : per_sm);
  long long g = (long long)sms * per_sm;
  return int(g < B ? g : B);
}

template <typename T>
int launch_fwd(const void* x, void* y, const float* aw, const float* bias, const float* wstat, const float* mask, const int* group,
               long long B, int L, int M, int C, float eps, int sub, cudaStream_t st) {
  if (const int threads = reg_threads(L, M, C)) {
    const size_t smem = reg_fwd_smem(L, M);
    auto kern = C == 128 ? sh_norm_fwd_reg_kernel<T, 4> : (C == 64 ? sh_norm_fwd_reg_kernel<T, 2> : sh_norm_fwd_reg_kernel<T, 1>);
    int per_sm = 1;
    if (cudaOccupancyMaxActiveBlocksPerMultiprocessor(&per_sm, kern, threads, smem) != cudaSuccess || per_sm < 1) per_sm = 1;
    kern<<<reg_grid(threads, per_sm, B), threads, smem, st>>>((const T*)x, (T*)y, aw, bias, wstat, mask, group, B, L, M, eps, sub);
    return cudaGetLastError() == cudaSuccess ? 0 : -4;
  }
  const size_t smem = fwd_smem(L, M, C);
  const int grid = grid_for(smem, B);
  auto k4 = sh_norm_fwd_kernel<T, 4>;
  auto k1 = sh_norm_fwd_kernel<T, 1>;
  auto k = (C % 4 == 0) ? k4 : k1;
  if (smem > 48 * 1024 && cudaFuncSetAttribute(k, cudaFuncAttributeMaxDynamicSharedMemorySize, int(smem)) != cudaSuccess) return -3;
  k<<<grid, kShThreads, smem, st>>>((const T*)x, (T*)y, aw, bias, wstat, mask, group, B, L, M, C, eps, sub);
  return cudaGetLastError() == cudaSuccess ? 0 : -4;
}

template <typename T>
int launch_bwd(const void* x, const void* dy, void* dx, const float* aw, const float* wstat, const float* mask, const int* group,
               float* daw_part, float* dbias_part, long long B, int L, int M, int C, float eps, int sub, int grid, cudaStream_t st) {
  if (const int threads = reg_threads(L, M, C)) {
    const size_t smem = reg_bwd_smem(L, M, C);
    if (C == 128)
      sh_norm_bwd_reg_kernel<T, 4><<<grid, threads, smem, st>>>((const T*)x, (const T*)dy, (T*)dx, aw, wstat, mask, group, daw_part,
                                                                 dbias_part, B, L, M, eps, sub);
    else if (C == 64)
      sh_norm_bwd_reg_kernel<T, 2><<<grid, threads, smem, st>>>((const T*)x, (const T*)dy, (T*)dx, aw, wstat, mask, group, daw_part,
                                                                 dbias_part, B, L, M, eps, sub);
    else
      sh_norm_bwd_reg_kernel<T, 1><<<grid, threads, smem, st>>>((const T*)x, (const T*)dy, (T*)dx, aw, wstat, mask, group, daw_part,
                                                                 dbias_part, B, L, M, eps, sub);
    return cudaGetLastError() == cudaSuccess ? 0 : -4;
  }
  const size_t smem = bwd_smem(L, M, C);
  auto k4 = sh_norm_bwd_kernel<T, 4>;
  auto k1 = sh_norm_bwd_kernel<T, 1>;
  auto k = (C % 4 == 0) ? k4 : k1;
  if (smem > 48 * 1024 && cudaFuncSetAttribute(k, cudaFuncAttributeMaxDynamicSharedMemorySize, int(smem)) != cudaSuccess) return -3;
  k<<<grid, kShThreads, smem, st>>>((const T*)x, (const T*)dy, (T*)dx, aw, wstat, mask, group, daw_part, dbias_part, B, L, M, C, eps,
                                    sub);
  return cudaGetLastError() == cudaSuccess ? 0 : -4;
}

}  // namespace
}  // namespace pnm

// 1 when the sample of one (L, M, C) grid fits the shared memory of the forward (which = 0) or backward (1) kernel
extern "C" int pnm_sh_norm_fits(int L, int M, int C, int which) {
  if (L <= 0 || M <= 0 || C <= 0 || L > pnm::kShThreads) return 0;
  return (which ? pnm::bwd_smem(L, M, C) : pnm::fwd_smem(L, M, C)) <= pnm::kMaxSmem ? 1 : 0;
}

// number of CTAs of the backward launch = leading extent of the two partial-gradient buffers
extern "C" int pnm_sh_norm_bwd_grid(long long B, int L, int M, int C) {
  if (!pnm_sh_norm_fits(L, M, C, 1) || B <= 0) return 0;
  if (const int threads = pnm::reg_threads(L, M, C)) return pnm::reg_grid(threads, threads == 256 ? 2 : 1, B);
  return pnm::grid_for(pnm::bwd_smem(L, M, C), B);
}

// dtype: 0 float32, 1 bfloat16, 2 float16 (x / y); every parameter table is float32, group is int32
extern "C" int pnm_sh_norm_fwd(const void* x, void* y, const float* aw, const float* bias, const float* wstat, const float* mask,
                               const int* group, long long B, int L, int M, int C, float eps, int subtract_mean, int dtype,
                               void* stream) {
  if (!x || !y || !aw || !wstat || !mask || !group || B <= 0 || !pnm_sh_norm_fits(L, M, C, 0)) return -1;
  cudaStream_t st = reinterpret_cast<cudaStream_t>(stream);
  if (dtype == 0) return pnm::launch_fwd<float>(x, y, aw, bias, wstat, mask, group, B, L, M, C, eps, subtract_mean, st);
  if (dtype == 1) return pnm::launch_fwd<__nv_bfloat16>(x, y, aw, bias, wstat, mask, group, B, L, M, C, eps, subtract_mean, st);
  if (dtype == 2) return pnm::launch_fwd<__half>(x, y, aw, bias, wstat, mask, group, B, L, M, C, eps, subtract_mean, st);
  return -1;
}

extern "C" int pnm_sh_norm_bwd(const void* x, const void* dy, void* dx, const float* aw, const float* wstat, const float* mask,
                               const int* group, float* daw_part, float* dbias_part, long long B, int L, int M, int C, float eps,
                               int subtract_mean, int dtype, int grid, void* stream) {
  if (!x || !dy || !dx || !aw || !wstat || !mask || !group || !daw_part || !dbias_part || B <= 0 || grid <= 0 ||
      !pnm_sh_norm_fits(L, M, C, 1))
    return -1;
  cudaStream_t st = reinterpret_cast<cudaStream_t>(stream);
  if (dtype == 0)
    return pnm::launch_bwd<float>(x, dy, dx, aw, wstat, mask, group, daw_part, dbias_part, B, L, M, C, eps, subtract_mean, grid, st);
  if (dtype == 1)
    return pnm::launch_bwd<__nv_bfloat16>(x, dy, dx, aw, wstat, mask, group, daw_part, dbias_part, B, L, M, C, eps, subtract_mean, grid,
                                         st);
  if (dtype == 2)
    return pnm::launch_bwd<__half>(x, dy, dx, aw, wstat, mask, group, daw_part, dbias_part, B, L, M, C, eps, subtract_mean, grid, st);
  return -1;
}
