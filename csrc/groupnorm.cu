// GroupNorm with an optional fused SiLU, forward and backward, for (B, C, *spatial) tensors in either memory format:
// layout 0 = channels-first (spatial contiguous), layout 1 = channels-last (channels contiguous).  bf16 or fp32 I/O,
// fp32 statistics.  The spatial extent is split into S slices so that small batches still fill the GPU:
//
//   forward   1) slice partials (sum, sum of squares) per (b, slice, group)
//             2) mean / rstd from the S partials, y = act((x - mean) * rstd * gamma + beta)
//   backward  1) slice partials per (b, slice, channel): sum of dz * xhat and of dz, dz = dy * act'(z)
//             2) per-batch channel sums, per-group sums A = sum gamma dz, B = sum gamma dz xhat, dgamma / dbeta
//             3) dx = rstd * (gamma dz - A/n - xhat B/n)
//
// Row-sharded images (channels-last only): the "_sh" entry points take the moments over the whole image.  The
// statistics kernel's last block folds this rank's partials into (B, G) sums, leaves them in the rank's symmetric
// buffer and raises one flag per peer; the normalising kernel waits (bounded) for every rank's flag in its prologue
// and adds the P short vectors with direct peer loads, so no collective call sits between the two passes.  The
// backward does the same with the two per-group sums of the input gradient.
//
// Every access is a 16-byte vector of 8 (bf16) or 4 (fp32) elements.  In the channels-last kernels a thread owns a
// fixed vector of channels and walks down the pixels, so gamma / beta / scale / shift live in registers.
#include <cuda_bf16.h>
#include <cuda_runtime.h>
#include <stdint.h>

#include "pnm_api.h"
#include "pnm_internal.h"

namespace pnm {

template <typename T> struct Vec;
template <> struct Vec<__nv_bfloat16> {
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
};
template <> struct Vec<float> {
  static constexpr int N = 4;
  static __device__ __forceinline__ void load(const float* p, float* f) {
    const float4 u = *reinterpret_cast<const float4*>(p);
    f[0] = u.x; f[1] = u.y; f[2] = u.z; f[3] = u.w;
  }
  static __device__ __forceinline__ void store(float* p, const float* f) {
    *reinterpret_cast<float4*>(p) = make_float4(f[0], f[1], f[2], f[3]);
  }
};

__device__ __forceinline__ float gn_silu(float z) { return z / (1.f + __expf(-z)); }
__device__ __forceinline__ float gn_silu_grad(float z) {
  const float s = 1.f / (1.f + __expf(-z));
  return s * (1.f + z * (1.f - s));
}

__device__ __forceinline__ float2 block_sum2(float a, float b) {
  __shared__ float2 red[32];
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) { a += __shfl_xor_sync(0xffffffffu, a, o); b += __shfl_xor_sync(0xffffffffu, b, o); }
  const int w = threadIdx.x >> 5, l = threadIdx.x & 31;
  __syncthreads();
  if (l == 0) red[w] = make_float2(a, b);
  __syncthreads();
  const int nw = (blockDim.x + 31) >> 5;
  float2 v = l < nw ? red[l] : make_float2(0.f, 0.f);
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) { v.x += __shfl_xor_sync(0xffffffffu, v.x, o); v.y += __shfl_xor_sync(0xffffffffu, v.y, o); }
  return v;
}

struct GNShape { int B, C, G, cpg, S; long long HW; };

// ---------------- channels-first ----------------------------------------------------------------------------------
// grid (S, B*C): one channel slice per CTA; partial[b][s][c] = (sum x, sum x^2)
template <typename T>
__global__ void __launch_bounds__(256) gn_stats_cf(const T* __restrict__ x, float2* __restrict__ partial, GNShape sh) {
  constexpr int V = Vec<T>::N;
  const int s = blockIdx.x, bc = blockIdx.y, b = bc / sh.C, c = bc % sh.C;
  const long long nvec = sh.HW / V, per = (nvec + sh.S - 1) / sh.S, v0 = s * per, v1 = min(nvec, v0 + per);
  const T* base = x + (long long)bc * sh.HW;
  float a = 0.f, q = 0.f, f[V];
  for (long long v = v0 + threadIdx.x; v < v1; v += blockDim.x) {
    Vec<T>::load(base + v * V, f);
#pragma unroll
    for (int i = 0; i < V; ++i) { a += f[i]; q += f[i] * f[i]; }
  }
  const float2 r = block_sum2(a, q);
  if (threadIdx.x == 0) partial[((long long)b * sh.S + s) * sh.C + c] = r;
}

// mean / rstd of group g of batch b from the channel partials (call with all threads; result valid in all threads)
__device__ __forceinline__ float2 group_moments(const float2* __restrict__ partial, const GNShape& sh, int b, int g, float eps) {
  float a = 0.f, q = 0.f;
  const int n = sh.S * sh.cpg;
  for (int i = threadIdx.x; i < n; i += blockDim.x) {
    const float2 p = partial[((long long)b * sh.S + i / sh.cpg) * sh.C + g * sh.cpg + i % sh.cpg];
    a += p.x; q += p.y;
  }
  const float2 r = block_sum2(a, q);
  const float cnt = (float)sh.cpg * (float)sh.HW;
  const float mean = r.x / cnt;
  return make_float2(mean, rsqrtf(fmaxf(r.y / cnt - mean * mean, 0.f) + eps));
}

template <typename T, bool kSilu>
__global__ void __launch_bounds__(256) gn_apply_cf(const T* __restrict__ x, const float2* __restrict__ partial,
                                                    const float* __restrict__ gamma, const float* __restrict__ beta,
                                                    T* __restrict__ y, float* __restrict__ mean_out, float* __restrict__ rstd_out,
                                                    GNShape sh, float eps) {
  constexpr int V = Vec<T>::N;
  const int s = blockIdx.x, bc = blockIdx.y, b = bc / sh.C, c = bc % sh.C, g = c / sh.cpg;
  const float2 m = group_moments(partial, sh, b, g, eps);
  if (s == 0 && c % sh.cpg == 0 && threadIdx.x == 0) { mean_out[b * sh.G + g] = m.x; rstd_out[b * sh.G + g] = m.y; }
  const float scale = m.y * gamma[c], shift = beta[c] - m.x * scale;
  const long long nvec = sh.HW / V, per = (nvec + sh.S - 1) / sh.S, v0 = s * per, v1 = min(nvec, v0 + per);
  const T* xi = x + (long long)bc * sh.HW;
  T* yo = y + (long long)bc * sh.HW;
  float f[V];
  for (long long v = v0 + threadIdx.x; v < v1; v += blockDim.x) {
    Vec<T>::load(xi + v * V, f);
#pragma unroll
    for (int i = 0; i < V; ++i) { const float z = f[i] * scale + shift; f[i] = kSilu ? gn_silu(z) : z; }
    Vec<T>::store(yo + v * V, f);
  }
}

// backward partials: pc[b][s][c] = (sum dz xhat, sum dz)
template <typename T, bool kSilu>
__global__ void __launch_bounds__(256) gn_bwd_stats_cf(const T* __restrict__ x, const T* __restrict__ dy,
                                                        const float* __restrict__ gamma, const float* __restrict__ beta,
                                                        const float* __restrict__ mean, const float* __restrict__ rstd,
                                                        float2* __restrict__ pc, GNShape sh) {
  constexpr int V = Vec<T>::N;
  const int s = blockIdx.x, bc = blockIdx.y, b = bc / sh.C, c = bc % sh.C, g = c / sh.cpg;
  const float mu = mean[b * sh.G + g], rs = rstd[b * sh.G + g], ga = gamma[c], be = beta[c];
  const long long nvec = sh.HW / V, per = (nvec + sh.S - 1) / sh.S, v0 = s * per, v1 = min(nvec, v0 + per);
  const T* xi = x + (long long)bc * sh.HW;
  const T* di = dy + (long long)bc * sh.HW;
  float a = 0.f, d = 0.f, f[V], e[V];
  for (long long v = v0 + threadIdx.x; v < v1; v += blockDim.x) {
    Vec<T>::load(xi + v * V, f);
    Vec<T>::load(di + v * V, e);
#pragma unroll
    for (int i = 0; i < V; ++i) {
      const float xh = (f[i] - mu) * rs;
      const float dz = kSilu ? e[i] * gn_silu_grad(xh * ga + be) : e[i];
      a += dz * xh; d += dz;
    }
  }
  const float2 r = block_sum2(a, d);
  if (threadIdx.x == 0) pc[((long long)b * sh.S + s) * sh.C + c] = r;
}

template <typename T, bool kSilu>
__global__ void __launch_bounds__(256) gn_bwd_apply_cf(const T* __restrict__ x, const T* __restrict__ dy,
                                                        const float* __restrict__ gamma, const float* __restrict__ beta,
                                                        const float* __restrict__ mean, const float* __restrict__ rstd,
                                                        const float2* __restrict__ group_ab, T* __restrict__ dx, GNShape sh) {
  constexpr int V = Vec<T>::N;
  const int s = blockIdx.x, bc = blockIdx.y, b = bc / sh.C, c = bc % sh.C, g = c / sh.cpg;
  const float mu = mean[b * sh.G + g], rs = rstd[b * sh.G + g], ga = gamma[c], be = beta[c];
  const float inv_n = 1.f / ((float)sh.cpg * (float)sh.HW);
  const float2 ab = group_ab[b * sh.G + g];
  const float A = ab.x * inv_n, Bq = ab.y * inv_n;
  const long long nvec = sh.HW / V, per = (nvec + sh.S - 1) / sh.S, v0 = s * per, v1 = min(nvec, v0 + per);
  const T* xi = x + (long long)bc * sh.HW;
  const T* di = dy + (long long)bc * sh.HW;
  T* o = dx + (long long)bc * sh.HW;
  float f[V], e[V];
  for (long long v = v0 + threadIdx.x; v < v1; v += blockDim.x) {
    Vec<T>::load(xi + v * V, f);
    Vec<T>::load(di + v * V, e);
#pragma unroll
    for (int i = 0; i < V; ++i) {
      const float xh = (f[i] - mu) * rs;
      const float dz = kSilu ? e[i] * gn_silu_grad(xh * ga + be) : e[i];
      f[i] = rs * (ga * dz - A - xh * Bq);
    }
    Vec<T>::store(o + v * V, f);
  }
}

// ---------------- channels-last -----------------------------------------------------------------------------------
// grid (S, B); a thread owns channels [c0, c0 + V) and every (blockDim / tpp)-th pixel of the slice
struct CLThread { int c0, lane_pix, ppi; bool active; long long p0, p1; };

template <int V>
__device__ __forceinline__ CLThread cl_thread(const GNShape& sh, int s) {
  CLThread t;
  const int tpp = sh.C / V;
  t.ppi = blockDim.x / tpp;
  t.active = (int)threadIdx.x < t.ppi * tpp;
  t.c0 = ((int)threadIdx.x % tpp) * V;
  t.lane_pix = (int)threadIdx.x / tpp;
  const long long per = (sh.HW + sh.S - 1) / sh.S;
  t.p0 = s * per;
  t.p1 = min(sh.HW, t.p0 + per);
  return t;
}

// One counter per batch item (zero between launches: the CTA that folds resets it).  Forward and backward keep apart.
__device__ unsigned int g_gn_fwd_counter[65536];
__device__ unsigned int g_gn_bwd_counter[65536];

// Called by every CTA of the (S, B) grid after it wrote its group partials part[b][s][0..G): the CTA that arrives last at
// the batch item's counter sums part[b][0..S)[g] in a fixed order (one warp per group, lanes over slices, shuffle tree)
// into out[b][g].  The channels-last kernels use hundreds of slices so that a batch of one still fills the machine; this
// keeps the fold off every consumer CTA's prologue and out of a launch of its own.
__device__ __forceinline__ void cl_fold_slices(const float2* part, float2* out, unsigned int* counter, const GNShape& sh, int b) {
  __shared__ int last;
  __threadfence();
  __syncthreads();
  if (threadIdx.x == 0) last = atomicAdd(counter + b, 1u) == gridDim.x - 1;
  __syncthreads();
  if (!last) return;
  __threadfence();
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31, nw = blockDim.x >> 5;
  for (int g = warp; g < sh.G; g += nw) {
    float a = 0.f, q = 0.f;
#pragma unroll 4
    for (int sl = lane; sl < sh.S; sl += 32) {
      const float2 v = __ldcg(part + ((long long)b * sh.S + sl) * sh.G + g);
      a += v.x; q += v.y;
    }
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) { a += __shfl_xor_sync(0xffffffffu, a, o); q += __shfl_xor_sync(0xffffffffu, q, o); }
    if (lane == 0) out[b * sh.G + g] = make_float2(a, q);
  }
  if (threadIdx.x == 0) counter[b] = 0;
}

// part[b][s][g] = (sum x, sum x^2) of slice s; gsum[b][g] = their sum over the slices (written by the last CTA of item b)
template <typename T>
__global__ void __launch_bounds__(256) gn_stats_cl(const T* __restrict__ x, float2* __restrict__ part, float2* __restrict__ gsum,
                                                    GNShape sh) {
  constexpr int V = Vec<T>::N;
  extern __shared__ float smem[];                        // [C][2]
  const int s = blockIdx.x, b = blockIdx.y;
  for (int i = threadIdx.x; i < 2 * sh.C; i += blockDim.x) smem[i] = 0.f;
  __syncthreads();
  const CLThread t = cl_thread<V>(sh, s);
  float a[V], q[V], f[V];
#pragma unroll
  for (int i = 0; i < V; ++i) a[i] = q[i] = 0.f;
  if (t.active) {
    const T* base = x + (long long)b * sh.HW * sh.C + t.c0;
#pragma unroll 4
    for (long long p = t.p0 + t.lane_pix; p < t.p1; p += t.ppi) {
      Vec<T>::load(base + p * sh.C, f);
#pragma unroll
      for (int i = 0; i < V; ++i) { a[i] += f[i]; q[i] += f[i] * f[i]; }
    }
#pragma unroll
    for (int i = 0; i < V; ++i) { atomicAdd(&smem[2 * (t.c0 + i)], a[i]); atomicAdd(&smem[2 * (t.c0 + i) + 1], q[i]); }
  }
  __syncthreads();
  for (int g = threadIdx.x; g < sh.G; g += blockDim.x) {
    float a2 = 0.f, q2 = 0.f;
    for (int k = 0; k < sh.cpg; ++k) { a2 += smem[2 * (g * sh.cpg + k)]; q2 += smem[2 * (g * sh.cpg + k) + 1]; }
    part[((long long)b * sh.S + s) * sh.G + g] = make_float2(a2, q2);
  }
  cl_fold_slices(part, gsum, g_gn_fwd_counter, sh, b);
}

// fills smem mom[g] = (mean, rstd) for all groups of batch item b from the folded sums
__device__ __forceinline__ void all_group_moments(const float2* __restrict__ gsum, const GNShape& sh, int b, float eps,
                                                  float2* mom) {
  const float cnt = (float)sh.cpg * (float)sh.HW;
  for (int g = threadIdx.x; g < sh.G; g += blockDim.x) {
    const float2 v = gsum[b * sh.G + g];
    const float mean = v.x / cnt;
    mom[g] = make_float2(mean, rsqrtf(fmaxf(v.y / cnt - mean * mean, 0.f) + eps));
  }
  __syncthreads();
}

// ---- sharded statistics ---------------------------------------------------------------------------------------------
// grid (B): the folded sums[b][g] = (sum x, sum x^2) of this rank's rows go to stage A of the symmetric buffer at float
// offset 2 * (b * G + g); the block that finishes last raises the flags.
__global__ void __launch_bounds__(256) gn_publish_moments(const float2* __restrict__ gsum, GNShape sh, PeerArgs peer,
                                                           unsigned int* counter) {
  const uint32_t epoch = peer_epoch(peer);
  float2* dst = reinterpret_cast<float2*>(peer_data(peer, peer.rank, epoch & 1, 0));
  const int b = blockIdx.x;
  for (int g = threadIdx.x; g < sh.G; g += blockDim.x) dst[b * sh.G + g] = gsum[b * sh.G + g];
  __threadfence_system();
  __syncthreads();
  if (threadIdx.x == 0 && atomicAdd(counter, 1u) == gridDim.x - 1) {
    *counter = 0;
    peer_small_publish(peer, epoch);
  }
}

// grid (B): like gn_bwd_reduce, then publishes group_ab[b][g] = (sum gamma dz, sum gamma dz xhat) of this rank's rows
__global__ void __launch_bounds__(256) gn_publish_ab(const float2* __restrict__ group_ab, GNShape sh, PeerArgs peer,
                                                      unsigned int* counter) {
  const uint32_t epoch = peer_epoch(peer);
  float2* dst = reinterpret_cast<float2*>(peer_data(peer, peer.rank, epoch & 1, 0));
  const int b = blockIdx.x;
  for (int g = threadIdx.x; g < sh.G; g += blockDim.x) dst[b * sh.G + g] = group_ab[b * sh.G + g];
  __threadfence_system();
  __syncthreads();
  if (threadIdx.x == 0 && atomicAdd(counter, 1u) == gridDim.x - 1) {
    *counter = 0;
    peer_small_publish(peer, epoch);
  }
}

template <typename T, bool kSilu>
__global__ void __launch_bounds__(256) gn_apply_cl_sh(const T* __restrict__ x, const float* __restrict__ gamma,
                                                       const float* __restrict__ beta, T* __restrict__ y,
                                                       float* __restrict__ mean_out, float* __restrict__ rstd_out, GNShape sh,
                                                       float eps, float count_global, PeerArgs peer, int* err) {
  constexpr int V = Vec<T>::N;
  extern __shared__ float smem[];
  float2* mom = reinterpret_cast<float2*>(smem);         // [G]
  __shared__ int sh_ok;
  const int s = blockIdx.x, b = blockIdx.y;
  const uint32_t epoch = peer_epoch(peer);
  const bool ok = peer_small_wait(peer, epoch, err, &sh_ok);
  for (int g = threadIdx.x; g < sh.G; g += blockDim.x) {
    float a = __int_as_float(0x7fc00000), q = a;         // a time-out shows as NaN in the output
    if (ok) {
      a = peer_small_sum(peer, epoch, 2 * (b * sh.G + g));
      q = peer_small_sum(peer, epoch, 2 * (b * sh.G + g) + 1);
    }
    const float mean = a / count_global;
    mom[g] = make_float2(mean, rsqrtf(fmaxf(q / count_global - mean * mean, 0.f) + eps));
  }
  __syncthreads();
  if (s == 0)
    for (int g = threadIdx.x; g < sh.G; g += blockDim.x) { mean_out[b * sh.G + g] = mom[g].x; rstd_out[b * sh.G + g] = mom[g].y; }
  const CLThread t = cl_thread<V>(sh, s);
  if (!t.active) return;
  float scale[V], shift[V], f[V];
#pragma unroll
  for (int i = 0; i < V; ++i) {
    const int c = t.c0 + i;
    const float2 m = mom[c / sh.cpg];
    scale[i] = m.y * gamma[c];
    shift[i] = beta[c] - m.x * scale[i];
  }
  const long long off = (long long)b * sh.HW * sh.C + t.c0;
#pragma unroll 4
  for (long long p = t.p0 + t.lane_pix; p < t.p1; p += t.ppi) {
    Vec<T>::load(x + off + p * sh.C, f);
#pragma unroll
    for (int i = 0; i < V; ++i) { const float z = f[i] * scale[i] + shift[i]; f[i] = kSilu ? gn_silu(z) : z; }
    Vec<T>::store(y + off + p * sh.C, f);
  }
}

template <typename T, bool kSilu>
__global__ void __launch_bounds__(256) gn_bwd_apply_cl_sh(const T* __restrict__ x, const T* __restrict__ dy,
                                                           const float* __restrict__ gamma, const float* __restrict__ beta,
                                                           const float* __restrict__ mean, const float* __restrict__ rstd,
                                                           T* __restrict__ dx, GNShape sh, float count_global, PeerArgs peer,
                                                           int* err) {
  constexpr int V = Vec<T>::N;
  extern __shared__ float smem[];
  float2* gab = reinterpret_cast<float2*>(smem);         // [G]
  __shared__ int sh_ok;
  const int s = blockIdx.x, b = blockIdx.y;
  const uint32_t epoch = peer_epoch(peer);
  const bool ok = peer_small_wait(peer, epoch, err, &sh_ok);
  for (int g = threadIdx.x; g < sh.G; g += blockDim.x) {
    float a = __int_as_float(0x7fc00000), q = a;
    if (ok) {
      a = peer_small_sum(peer, epoch, 2 * (b * sh.G + g));
      q = peer_small_sum(peer, epoch, 2 * (b * sh.G + g) + 1);
    }
    gab[g] = make_float2(a, q);
  }
  __syncthreads();
  const CLThread t = cl_thread<V>(sh, s);
  if (!t.active) return;
  const float inv_n = 1.f / count_global;
  float mu[V], rs[V], ga[V], be[V], A[V], Bq[V], f[V], e[V];
#pragma unroll
  for (int i = 0; i < V; ++i) {
    const int c = t.c0 + i, g = c / sh.cpg;
    mu[i] = mean[b * sh.G + g]; rs[i] = rstd[b * sh.G + g]; ga[i] = gamma[c]; be[i] = beta[c];
    A[i] = gab[g].x * inv_n; Bq[i] = gab[g].y * inv_n;
  }
  const long long off = (long long)b * sh.HW * sh.C + t.c0;
#pragma unroll 2
  for (long long p = t.p0 + t.lane_pix; p < t.p1; p += t.ppi) {
    Vec<T>::load(x + off + p * sh.C, f);
    Vec<T>::load(dy + off + p * sh.C, e);
#pragma unroll
    for (int i = 0; i < V; ++i) {
      const float xh = (f[i] - mu[i]) * rs[i];
      const float dz = kSilu ? e[i] * gn_silu_grad(xh * ga[i] + be[i]) : e[i];
      f[i] = rs[i] * (ga[i] * dz - A[i] - xh * Bq[i]);
    }
    Vec<T>::store(dx + off + p * sh.C, f);
  }
}

template <typename T, bool kSilu>
__global__ void __launch_bounds__(256) gn_apply_cl(const T* __restrict__ x, const float2* __restrict__ partial,
                                                    const float* __restrict__ gamma, const float* __restrict__ beta,
                                                    T* __restrict__ y, float* __restrict__ mean_out, float* __restrict__ rstd_out,
                                                    GNShape sh, float eps) {
  constexpr int V = Vec<T>::N;
  extern __shared__ float smem[];
  float2* mom = reinterpret_cast<float2*>(smem);         // [G]
  const int s = blockIdx.x, b = blockIdx.y;
  all_group_moments(partial, sh, b, eps, mom);
  if (s == 0)
    for (int g = threadIdx.x; g < sh.G; g += blockDim.x) { mean_out[b * sh.G + g] = mom[g].x; rstd_out[b * sh.G + g] = mom[g].y; }
  const CLThread t = cl_thread<V>(sh, s);
  if (!t.active) return;
  float scale[V], shift[V], f[V];
#pragma unroll
  for (int i = 0; i < V; ++i) {
    const int c = t.c0 + i;
    const float2 m = mom[c / sh.cpg];
    scale[i] = m.y * gamma[c];
    shift[i] = beta[c] - m.x * scale[i];
  }
  const long long off = (long long)b * sh.HW * sh.C + t.c0;
#pragma unroll 4
  for (long long p = t.p0 + t.lane_pix; p < t.p1; p += t.ppi) {
    Vec<T>::load(x + off + p * sh.C, f);
#pragma unroll
    for (int i = 0; i < V; ++i) { const float z = f[i] * scale[i] + shift[i]; f[i] = kSilu ? gn_silu(z) : z; }
    Vec<T>::store(y + off + p * sh.C, f);
  }
}

template <typename T, bool kSilu>
__global__ void __launch_bounds__(256) gn_bwd_stats_cl(const T* __restrict__ x, const T* __restrict__ dy,
                                                        const float* __restrict__ gamma, const float* __restrict__ beta,
                                                        const float* __restrict__ mean, const float* __restrict__ rstd,
                                                        float2* __restrict__ part, float2* __restrict__ group_ab,
                                                        float* __restrict__ dgamma, float* __restrict__ dbeta, GNShape sh) {
  constexpr int V = Vec<T>::N;
  extern __shared__ float smem[];                        // [C][2]
  const int s = blockIdx.x, b = blockIdx.y;
  for (int i = threadIdx.x; i < 2 * sh.C; i += blockDim.x) smem[i] = 0.f;
  __syncthreads();
  const CLThread t = cl_thread<V>(sh, s);
  if (t.active) {
    float mu[V], rs[V], ga[V], be[V], a[V], d[V], f[V], e[V];
#pragma unroll
    for (int i = 0; i < V; ++i) {
      const int c = t.c0 + i, g = c / sh.cpg;
      mu[i] = mean[b * sh.G + g]; rs[i] = rstd[b * sh.G + g]; ga[i] = gamma[c]; be[i] = beta[c];
      a[i] = d[i] = 0.f;
    }
    const long long off = (long long)b * sh.HW * sh.C + t.c0;
#pragma unroll 2
    for (long long p = t.p0 + t.lane_pix; p < t.p1; p += t.ppi) {
      Vec<T>::load(x + off + p * sh.C, f);
      Vec<T>::load(dy + off + p * sh.C, e);
#pragma unroll
      for (int i = 0; i < V; ++i) {
        const float xh = (f[i] - mu[i]) * rs[i];
        const float dz = kSilu ? e[i] * gn_silu_grad(xh * ga[i] + be[i]) : e[i];
        a[i] += dz * xh; d[i] += dz;
      }
    }
#pragma unroll
    for (int i = 0; i < V; ++i) { atomicAdd(&smem[2 * (t.c0 + i)], a[i]); atomicAdd(&smem[2 * (t.c0 + i) + 1], d[i]); }
  }
  __syncthreads();
  // parameter gradients: every slice adds its channel sums (dgamma / dbeta are zeroed by the caller)
  for (int c = threadIdx.x; c < sh.C; c += blockDim.x) {
    atomicAdd(&dgamma[c], smem[2 * c]);
    atomicAdd(&dbeta[c], smem[2 * c + 1]);
  }
  // group sums for dx: A = sum gamma * (sum dz), B = sum gamma * (sum dz xhat), folded over the slices by the last CTA
  for (int g = threadIdx.x; g < sh.G; g += blockDim.x) {
    float A = 0.f, Bq = 0.f;
    for (int k = 0; k < sh.cpg; ++k) {
      const int c = g * sh.cpg + k;
      A += gamma[c] * smem[2 * c + 1];
      Bq += gamma[c] * smem[2 * c];
    }
    part[((long long)b * sh.S + s) * sh.G + g] = make_float2(A, Bq);
  }
  cl_fold_slices(part, group_ab, g_gn_bwd_counter, sh, b);
}

template <typename T, bool kSilu>
__global__ void __launch_bounds__(256) gn_bwd_apply_cl(const T* __restrict__ x, const T* __restrict__ dy,
                                                        const float* __restrict__ gamma, const float* __restrict__ beta,
                                                        const float* __restrict__ mean, const float* __restrict__ rstd,
                                                        const float2* __restrict__ group_ab, T* __restrict__ dx, GNShape sh) {
  constexpr int V = Vec<T>::N;
  const int s = blockIdx.x, b = blockIdx.y;
  const CLThread t = cl_thread<V>(sh, s);
  if (!t.active) return;
  const float inv_n = 1.f / ((float)sh.cpg * (float)sh.HW);
  float mu[V], rs[V], ga[V], be[V], A[V], Bq[V], f[V], e[V];
#pragma unroll
  for (int i = 0; i < V; ++i) {
    const int c = t.c0 + i, g = c / sh.cpg;
    mu[i] = mean[b * sh.G + g]; rs[i] = rstd[b * sh.G + g]; ga[i] = gamma[c]; be[i] = beta[c];
    const float2 ab = group_ab[b * sh.G + g];
    A[i] = ab.x * inv_n; Bq[i] = ab.y * inv_n;
  }
  const long long off = (long long)b * sh.HW * sh.C + t.c0;
#pragma unroll 2
  for (long long p = t.p0 + t.lane_pix; p < t.p1; p += t.ppi) {
    Vec<T>::load(x + off + p * sh.C, f);
    Vec<T>::load(dy + off + p * sh.C, e);
#pragma unroll
    for (int i = 0; i < V; ++i) {
      const float xh = (f[i] - mu[i]) * rs[i];
      const float dz = kSilu ? e[i] * gn_silu_grad(xh * ga[i] + be[i]) : e[i];
      f[i] = rs[i] * (ga[i] * dz - A[i] - xh * Bq[i]);
    }
    Vec<T>::store(dx + off + p * sh.C, f);
  }
}

// per batch item: channel sums over slices, group sums A = sum gamma * dbeta_c, B = sum gamma * dgamma_c, and the
// parameter gradients accumulated over the batch with atomics (dgamma / dbeta zeroed by the caller).  grid (B)
__global__ void __launch_bounds__(256) gn_bwd_reduce(const float2* __restrict__ pc, const float* __restrict__ gamma,
                                                      float2* __restrict__ group_ab, float* __restrict__ dgamma,
                                                      float* __restrict__ dbeta, GNShape sh) {
  extern __shared__ float smem[];                        // [G][2]
  const int b = blockIdx.x;
  for (int i = threadIdx.x; i < 2 * sh.G; i += blockDim.x) smem[i] = 0.f;
  __syncthreads();
  for (int c = threadIdx.x; c < sh.C; c += blockDim.x) {
    float a = 0.f, d = 0.f;
    for (int s = 0; s < sh.S; ++s) { const float2 p = pc[((long long)b * sh.S + s) * sh.C + c]; a += p.x; d += p.y; }
    atomicAdd(&dgamma[c], a);
    atomicAdd(&dbeta[c], d);
    const int g = c / sh.cpg;
    atomicAdd(&smem[2 * g], gamma[c] * d);
    atomicAdd(&smem[2 * g + 1], gamma[c] * a);
  }
  __syncthreads();
  for (int g = threadIdx.x; g < sh.G; g += blockDim.x) group_ab[b * sh.G + g] = make_float2(smem[2 * g], smem[2 * g + 1]);
}

template <typename T>
int gn_forward(const void* x, const float* gamma, const float* beta, void* y, float* mean, float* rstd, float* scratch,
               GNShape sh, int layout, int act, float eps, cudaStream_t st) {
  float2* partial = reinterpret_cast<float2*>(scratch);
  const T* xi = static_cast<const T*>(x);
  T* yo = static_cast<T*>(y);
  if (layout == 0) {
    const dim3 grid(sh.S, sh.B * sh.C);
    gn_stats_cf<T><<<grid, 256, 0, st>>>(xi, partial, sh);
    if (act) gn_apply_cf<T, true><<<grid, 256, 0, st>>>(xi, partial, gamma, beta, yo, mean, rstd, sh, eps);
    else gn_apply_cf<T, false><<<grid, 256, 0, st>>>(xi, partial, gamma, beta, yo, mean, rstd, sh, eps);
  } else {
    const dim3 grid(sh.S, sh.B);
    float2* gsum = partial + (long long)sh.B * sh.S * sh.G;
    gn_stats_cl<T><<<grid, 256, 2 * sh.C * sizeof(float), st>>>(xi, partial, gsum, sh);
    if (act) gn_apply_cl<T, true><<<grid, 256, sh.G * sizeof(float2), st>>>(xi, gsum, gamma, beta, yo, mean, rstd, sh, eps);
    else gn_apply_cl<T, false><<<grid, 256, sh.G * sizeof(float2), st>>>(xi, gsum, gamma, beta, yo, mean, rstd, sh, eps);
  }
  return (int)cudaGetLastError();
}

template <typename T>
int gn_backward(const void* x, const void* dy, const float* gamma, const float* beta, const float* mean, const float* rstd,
                void* dx, float* dgamma, float* dbeta, float* scratch, GNShape sh, int layout, int act, cudaStream_t st) {
  float2* pc = reinterpret_cast<float2*>(scratch);
  float2* ab = pc + (long long)sh.B * sh.S * (layout == 0 ? sh.C : sh.G);
  const T* xi = static_cast<const T*>(x);
  const T* di = static_cast<const T*>(dy);
  T* o = static_cast<T*>(dx);
  const dim3 grid = layout == 0 ? dim3(sh.S, sh.B * sh.C) : dim3(sh.S, sh.B);
  const size_t sm = layout == 0 ? 0 : 2 * sh.C * sizeof(float);
  if (layout == 0) {
    if (act) gn_bwd_stats_cf<T, true><<<grid, 256, 0, st>>>(xi, di, gamma, beta, mean, rstd, pc, sh);
    else gn_bwd_stats_cf<T, false><<<grid, 256, 0, st>>>(xi, di, gamma, beta, mean, rstd, pc, sh);
    gn_bwd_reduce<<<sh.B, 256, 2 * sh.G * sizeof(float), st>>>(pc, gamma, ab, dgamma, dbeta, sh);
  } else {
    if (act) gn_bwd_stats_cl<T, true><<<grid, 256, sm, st>>>(xi, di, gamma, beta, mean, rstd, pc, ab, dgamma, dbeta, sh);
    else gn_bwd_stats_cl<T, false><<<grid, 256, sm, st>>>(xi, di, gamma, beta, mean, rstd, pc, ab, dgamma, dbeta, sh);
  }
  if (layout == 0) {
    if (act) gn_bwd_apply_cf<T, true><<<grid, 256, 0, st>>>(xi, di, gamma, beta, mean, rstd, ab, o, sh);
    else gn_bwd_apply_cf<T, false><<<grid, 256, 0, st>>>(xi, di, gamma, beta, mean, rstd, ab, o, sh);
  } else {
    if (act) gn_bwd_apply_cl<T, true><<<grid, 256, 0, st>>>(xi, di, gamma, beta, mean, rstd, ab, o, sh);
    else gn_bwd_apply_cl<T, false><<<grid, 256, 0, st>>>(xi, di, gamma, beta, mean, rstd, ab, o, sh);
  }
  return (int)cudaGetLastError();
}

template <typename T>
int gn_forward_sh(const void* x, const float* gamma, const float* beta, void* y, float* mean, float* rstd, float* scratch,
                  GNShape sh, int act, float eps, float count_global, const PeerArgs& peer, unsigned int* counter, int* err,
                  cudaStream_t st) {
  float2* partial = reinterpret_cast<float2*>(scratch);
  const T* xi = static_cast<const T*>(x);
  T* yo = static_cast<T*>(y);
  const dim3 grid(sh.S, sh.B);
  float2* gsum = partial + (long long)sh.B * sh.S * sh.G;
  gn_stats_cl<T><<<grid, 256, 2 * sh.C * sizeof(float), st>>>(xi, partial, gsum, sh);
  gn_publish_moments<<<sh.B, 256, 0, st>>>(gsum, sh, peer, counter);
  if (act) gn_apply_cl_sh<T, true><<<grid, 256, sh.G * sizeof(float2), st>>>(xi, gamma, beta, yo, mean, rstd, sh, eps, count_global, peer, err);
  else gn_apply_cl_sh<T, false><<<grid, 256, sh.G * sizeof(float2), st>>>(xi, gamma, beta, yo, mean, rstd, sh, eps, count_global, peer, err);
  return (int)cudaGetLastError();
}

template <typename T>
int gn_backward_sh(const void* x, const void* dy, const float* gamma, const float* beta, const float* mean, const float* rstd,
                   void* dx, float* dgamma, float* dbeta, float* scratch, GNShape sh, int act, float count_global,
                   const PeerArgs& peer, unsigned int* counter, int* err, cudaStream_t st) {
  float2* pc = reinterpret_cast<float2*>(scratch);
  float2* ab = pc + (long long)sh.B * sh.S * sh.G;
  const T* xi = static_cast<const T*>(x);
  const T* di = static_cast<const T*>(dy);
  T* o = static_cast<T*>(dx);
  const dim3 grid(sh.S, sh.B);
  const size_t sm = 2 * sh.C * sizeof(float);
  if (act) gn_bwd_stats_cl<T, true><<<grid, 256, sm, st>>>(xi, di, gamma, beta, mean, rstd, pc, ab, dgamma, dbeta, sh);
  else gn_bwd_stats_cl<T, false><<<grid, 256, sm, st>>>(xi, di, gamma, beta, mean, rstd, pc, ab, dgamma, dbeta, sh);
  gn_publish_ab<<<sh.B, 256, 0, st>>>(ab, sh, peer, counter);
  if (act) gn_bwd_apply_cl_sh<T, true><<<grid, 256, sh.G * sizeof(float2), st>>>(xi, di, gamma, beta, mean, rstd, o, sh, count_global, peer, err);
  else gn_bwd_apply_cl_sh<T, false><<<grid, 256, sh.G * sizeof(float2), st>>>(xi, di, gamma, beta, mean, rstd, o, sh, count_global, peer, err);
  return (int)cudaGetLastError();
}

static bool gn_supported(const GNShape& sh, int layout, int dtype) {
  const int V = dtype == 0 ? 8 : 4;
  if (sh.B <= 0 || sh.C <= 0 || sh.G <= 0 || sh.C % sh.G || sh.S <= 0 || sh.HW <= 0) return false;
  if (layout == 0) return sh.HW % V == 0 && (long long)sh.B * sh.C <= 65535;
  return sh.C % V == 0 && sh.C / V <= 256 && sh.B <= 65535 && 2 * sh.C * sizeof(float) <= 48 * 1024;
}

}  // namespace pnm

extern "C" {

// floats of scratch needed by forward / backward for a given slice count
long long pnm_groupnorm_scratch_floats(int B, int C, int G, int S) { return 2LL * B * S * C + 2LL * B * G; }

// dtype: 0 bf16, 1 fp32.  layout: 0 channels-first, 1 channels-last.  act: 0 none, 1 SiLU.  Returns -1 if the shape is
// outside what the kernels cover (the caller then uses another path), else the CUDA error code.
int pnm_groupnorm_fwd(const void* x, const float* gamma, const float* beta, void* y, float* mean, float* rstd, float* scratch,
                      int B, int C, long long HW, int G, int S, int layout, int dtype, int act, float eps, void* stream) {
  pnm::GNShape sh{B, C, G, G > 0 ? C / G : 0, S, HW};
  if (!pnm::gn_supported(sh, layout, dtype)) return -1;
  cudaStream_t st = (cudaStream_t)stream;
  return dtype == 0 ? pnm::gn_forward<__nv_bfloat16>(x, gamma, beta, y, mean, rstd, scratch, sh, layout, act, eps, st)
                    : pnm::gn_forward<float>(x, gamma, beta, y, mean, rstd, scratch, sh, layout, act, eps, st);
}

int pnm_groupnorm_bwd(const void* x, const void* dy, const float* gamma, const float* beta, const float* mean,
                      const float* rstd, void* dx, float* dgamma, float* dbeta, float* scratch, int B, int C, long long HW,
                      int G, int S, int layout, int dtype, int act, void* stream) {
  pnm::GNShape sh{B, C, G, G > 0 ? C / G : 0, S, HW};
  if (!pnm::gn_supported(sh, layout, dtype)) return -1;
  cudaStream_t st = (cudaStream_t)stream;
  return dtype == 0 ? pnm::gn_backward<__nv_bfloat16>(x, dy, gamma, beta, mean, rstd, dx, dgamma, dbeta, scratch, sh, layout, act, st)
                    : pnm::gn_backward<float>(x, dy, gamma, beta, mean, rstd, dx, dgamma, dbeta, scratch, sh, layout, act, st);
}

// Row-sharded variants (channels-last, layout 1): the moments span all ranks' rows.  hw_global = pixels per image over the
// whole (unsharded) extent; `counter` is one device uint32 that is zero before the first call (the kernels reset it).  2 * B * G floats must fit into one stage of the symmetric buffer.  Peer arguments as in
// pnm_peer_allreduce.
int pnm_groupnorm_fwd_sharded(const void* x, const float* gamma, const float* beta, void* y, float* mean, float* rstd,
                              float* scratch, int B, int C, long long HW, long long hw_global, int G, int S, int dtype, int act,
                              float eps, const void* const* bases, int rank, int world, unsigned int epoch,
                              long long capacity_floats, double budget_s, const void* epoch_base, void* counter, void* stream) {
  pnm::GNShape sh{B, C, G, G > 0 ? C / G : 0, S, HW};
  if (!pnm::gn_supported(sh, 1, dtype) || world < 1 || world > pnm::kPeerMaxRanks || 2LL * B * G > capacity_floats || !counter) return -1;
  int* err = pnm::error_word_ptr();
  if (!err) return -2;
  const pnm::PeerArgs p = pnm::make_peer_args(bases, rank, world, epoch, capacity_floats, budget_s, epoch_base);
  const float cnt = (float)sh.cpg * (float)hw_global;
  cudaStream_t st = (cudaStream_t)stream;
  return dtype == 0 ? pnm::gn_forward_sh<__nv_bfloat16>(x, gamma, beta, y, mean, rstd, scratch, sh, act, eps, cnt, p, (unsigned int*)counter, err, st)
                    : pnm::gn_forward_sh<float>(x, gamma, beta, y, mean, rstd, scratch, sh, act, eps, cnt, p, (unsigned int*)counter, err, st);
}

int pnm_groupnorm_bwd_sharded(const void* x, const void* dy, const float* gamma, const float* beta, const float* mean,
                              const float* rstd, void* dx, float* dgamma, float* dbeta, float* scratch, int B, int C,
                              long long HW, long long hw_global, int G, int S, int dtype, int act, const void* const* bases,
                              int rank, int world, unsigned int epoch, long long capacity_floats, double budget_s,
                              const void* epoch_base, void* counter, void* stream) {
  pnm::GNShape sh{B, C, G, G > 0 ? C / G : 0, S, HW};
  if (!pnm::gn_supported(sh, 1, dtype) || world < 1 || world > pnm::kPeerMaxRanks || 2LL * B * G > capacity_floats || !counter) return -1;
  int* err = pnm::error_word_ptr();
  if (!err) return -2;
  const pnm::PeerArgs p = pnm::make_peer_args(bases, rank, world, epoch, capacity_floats, budget_s, epoch_base);
  const float cnt = (float)sh.cpg * (float)hw_global;
  cudaStream_t st = (cudaStream_t)stream;
  return dtype == 0 ? pnm::gn_backward_sh<__nv_bfloat16>(x, dy, gamma, beta, mean, rstd, dx, dgamma, dbeta, scratch, sh, act, cnt, p, (unsigned int*)counter, err, st)
                    : pnm::gn_backward_sh<float>(x, dy, gamma, beta, mean, rstd, dx, dgamma, dbeta, scratch, sh, act, cnt, p, (unsigned int*)counter, err, st);
}

}  // extern "C"
