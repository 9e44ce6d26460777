// Neighbourhood attention, 1-3 spatial dimensions, forward and backward.
//
// Tensors are [B, L, H, D] with L the flattened spatial extent (row-major over up to three axes).  Every query attends
// to a kernel_size window per axis, centred on it and shifted (not truncated) at the borders; with dilation d the
// window lives on the sub-lattice of positions congruent to the query modulo d.
//
// One warp per (batch, position, head).  Scores: lane j owns neighbour j (rows of K are read as contiguous vectors
// against the query held in shared memory); softmax across lanes; output: lane d owns channels d, d+32, ... and walks
// the neighbours (coalesced rows of V).  Backward recomputes the probabilities, then dQ is gathered the same way and
// dK / dV are scattered with fp32 atomics into accumulators that the caller casts back.
#include <cuda_bf16.h>
#include <cuda_runtime.h>
#include <float.h>
#include <stdint.h>

#include "pnm_api.h"

namespace pnm {

constexpr int kNaWarps = 4;
constexpr int kNaMaxK = 512;
constexpr int kNaMaxD = 256;

__host__ __device__ __forceinline__ size_t na_align16(size_t v) { return (v + 15) & ~(size_t)15; }

struct NaGeom { int nd; int n[3]; int k[3]; int dil[3]; int K; long long L; };

__device__ __forceinline__ float na_ld(const float* p) { return *p; }
__device__ __forceinline__ float na_ld(const __nv_bfloat16* p) { return __bfloat162float(*p); }
__device__ __forceinline__ void na_st(float* p, float v) { *p = v; }
__device__ __forceinline__ void na_st(__nv_bfloat16* p, float v) { *p = __float2bfloat16(v); }

// first window position along one axis and its stride
__device__ __forceinline__ void na_axis(int i, int n, int k, int d, int& first, int& step) {
  if (d == 1) { first = min(max(i - k / 2, 0), n - k); step = 1; return; }
  const int phase = i % d, pos = i / d, count = (n - phase + d - 1) / d;
  first = min(max(pos - k / 2, 0), count - k) * d + phase;
  step = d;
}

// linear index of neighbour j of the query at flat position l
__device__ __forceinline__ long long na_neighbour(const NaGeom& g, const int* first, const int* step, int j) {
  long long idx = 0;
  int rem = j;
  int t[3] = {0, 0, 0};
  for (int a = g.nd - 1; a >= 0; --a) { t[a] = rem % g.k[a]; rem /= g.k[a]; }
  for (int a = 0; a < g.nd; ++a) idx = idx * g.n[a] + first[a] + t[a] * step[a];
  return idx;
}

template <typename T>
struct NaWarp {
  float* sq;        // [D] query * scale (forward) / plain query (backward)
  float* sp;        // [K] probabilities
  float* sx;        // [D] dO (backward)
  float* sd;        // [K] ds (backward)
  long long* sn;    // [K] neighbour rows
};

template <typename T>
__device__ __forceinline__ float na_row_dot(const float* s, const T* row, int D) {
  float acc = 0.f;
  for (int d = 0; d < D; ++d) acc += s[d] * na_ld(row + d);
  return acc;
}
template <>
__device__ __forceinline__ float na_row_dot<__nv_bfloat16>(const float* s, const __nv_bfloat16* row, int D) {
  float acc = 0.f;
  int d = 0;
  if ((reinterpret_cast<uintptr_t>(row) & 15) == 0)
    for (; d + 8 <= D; d += 8) {
      const uint4 u = *reinterpret_cast<const uint4*>(row + d);
      const __nv_bfloat162* h = reinterpret_cast<const __nv_bfloat162*>(&u);
#pragma unroll
      for (int i = 0; i < 4; ++i) { const float2 v = __bfloat1622float2(h[i]); acc += s[d + 2 * i] * v.x + s[d + 2 * i + 1] * v.y; }
    }
  for (; d < D; ++d) acc += s[d] * __bfloat162float(row[d]);
  return acc;
}

__device__ __forceinline__ float warp_max(float v) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v = fmaxf(v, __shfl_xor_sync(0xffffffffu, v, o));
  return v;
}
__device__ __forceinline__ float warp_sum(float v) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
  return v;
}

// decodes the warp's query, fills sn[] and returns false if the warp has no work
template <typename T>
__device__ __forceinline__ bool na_setup(const NaGeom& g, int H, long long total, long long& row, long long* sn, int lane,
                                         long long& b) {
  const long long wq = blockIdx.x * (long long)kNaWarps + (threadIdx.x >> 5);
  if (wq >= total) return false;
  row = wq;                                             // (b, l, h) flattened in memory order
  const int h = (int)(wq % H);
  const long long bl = wq / H, l = bl % g.L;
  b = bl / g.L;
  int first[3], step[3], coord[3];
  long long rem = l;
  for (int a = g.nd - 1; a >= 0; --a) { coord[a] = (int)(rem % g.n[a]); rem /= g.n[a]; }
  for (int a = 0; a < g.nd; ++a) na_axis(coord[a], g.n[a], g.k[a], g.dil[a], first[a], step[a]);
  for (int j = lane; j < g.K; j += 32) sn[j] = ((b * g.L + na_neighbour(g, first, step, j)) * H + h);
  return true;
}

template <typename T>
__global__ void __launch_bounds__(kNaWarps * 32) natten_fwd_kernel(const T* __restrict__ q, const T* __restrict__ k,
                                                                    const T* __restrict__ v, T* __restrict__ out, NaGeom g,
                                                                    int H, int D, long long total, float scale) {
  extern __shared__ __align__(16) unsigned char smem_raw[];
  const int w = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const size_t per_warp = na_align16((size_t)(D + g.K) * sizeof(float) + (size_t)g.K * sizeof(long long));
  unsigned char* base = smem_raw + w * per_warp;
  long long* sn = reinterpret_cast<long long*>(base);
  float* sq = reinterpret_cast<float*>(base + (size_t)g.K * sizeof(long long));
  float* sp = sq + D;
  long long row, b;
  if (!na_setup<T>(g, H, total, row, sn, lane, b)) return;
  for (int d = lane; d < D; d += 32) sq[d] = na_ld(q + row * D + d) * scale;
  __syncwarp();
  float mx = -FLT_MAX;
  for (int j = lane; j < g.K; j += 32) { const float s = na_row_dot<T>(sq, k + sn[j] * D, D); sp[j] = s; mx = fmaxf(mx, s); }
  mx = warp_max(mx);
  float sum = 0.f;
  for (int j = lane; j < g.K; j += 32) { const float e = __expf(sp[j] - mx); sp[j] = e; sum += e; }
  sum = warp_sum(sum);
  __syncwarp();
  const float inv = 1.f / sum;
  for (int d = lane; d < D; d += 32) {
    float acc = 0.f;
    for (int j = 0; j < g.K; ++j) acc += sp[j] * na_ld(v + sn[j] * D + d);
    na_st(out + row * D + d, acc * inv);
  }
}

template <typename T>
__global__ void __launch_bounds__(kNaWarps * 32) natten_bwd_kernel(const T* __restrict__ q, const T* __restrict__ k,
                                                                    const T* __restrict__ v, const T* __restrict__ dout,
                                                                    T* __restrict__ dq, float* __restrict__ dk,
                                                                    float* __restrict__ dv, NaGeom g, int H, int D,
                                                                    long long total, float scale) {
  extern __shared__ __align__(16) unsigned char smem_raw[];
  const int w = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const size_t per_warp = na_align16((size_t)(2 * D + 2 * g.K) * sizeof(float) + (size_t)g.K * sizeof(long long));
  unsigned char* base = smem_raw + w * per_warp;
  long long* sn = reinterpret_cast<long long*>(base);
  float* sq = reinterpret_cast<float*>(base + (size_t)g.K * sizeof(long long));
  float* sx = sq + D;
  float* sp = sx + D;
  float* sd = sp + g.K;
  long long row, b;
  if (!na_setup<T>(g, H, total, row, sn, lane, b)) return;
  for (int d = lane; d < D; d += 32) { sq[d] = na_ld(q + row * D + d); sx[d] = na_ld(dout + row * D + d); }
  __syncwarp();
  float mx = -FLT_MAX;
  for (int j = lane; j < g.K; j += 32) {
    const float s = na_row_dot<T>(sq, k + sn[j] * D, D) * scale;
    sp[j] = s; mx = fmaxf(mx, s);
    sd[j] = na_row_dot<T>(sx, v + sn[j] * D, D);                 // dP_j = dO . v_j
  }
  mx = warp_max(mx);
  float sum = 0.f;
  for (int j = lane; j < g.K; j += 32) { const float e = __expf(sp[j] - mx); sp[j] = e; sum += e; }
  sum = warp_sum(sum);
  const float inv = 1.f / sum;
  float delta = 0.f;
  for (int j = lane; j < g.K; j += 32) { sp[j] *= inv; delta += sp[j] * sd[j]; }
  delta = warp_sum(delta);
  for (int j = lane; j < g.K; j += 32) sd[j] = sp[j] * (sd[j] - delta) * scale;   // dS_j
  __syncwarp();
  for (int d = lane; d < D; d += 32) {
    float acc = 0.f;
    const float qd = sq[d], od = sx[d];
    for (int j = 0; j < g.K; ++j) {
      const long long r = sn[j] * D + d;
      acc += sd[j] * na_ld(k + r);
      atomicAdd(dk + r, sd[j] * qd);
      atomicAdd(dv + r, sp[j] * od);
    }
    na_st(dq + row * D + d, acc);
  }
}

static int na_geom(NaGeom& g, int nd, const int* shape, const int* kernel, const int* dilation) {
  if (nd < 1 || nd > 3) return -1;
  g.nd = nd; g.K = 1; g.L = 1;
  for (int a = 0; a < 3; ++a) { g.n[a] = 1; g.k[a] = 1; g.dil[a] = 1; }
  for (int a = 0; a < nd; ++a) {
    g.n[a] = shape[a]; g.k[a] = kernel[a]; g.dil[a] = dilation[a];
    if (g.k[a] < 1 || g.dil[a] < 1 || (long long)g.k[a] * g.dil[a] > g.n[a] + g.dil[a] - 1 || g.k[a] > g.n[a]) return -1;
    if (g.dil[a] > 1 && g.k[a] > g.n[a] / g.dil[a]) return -1;   // every sub-lattice must hold a full window
    g.K *= g.k[a]; g.L *= g.n[a];
  }
  return g.K <= kNaMaxK ? 0 : -1;
}

}  // namespace pnm

extern "C" {

// dtype 0 bf16, 1 fp32.  Returns -1 for geometry outside the kernel's limits (K <= 512 neighbours, D <= 256).
int pnm_natten_fwd(const void* q, const void* k, const void* v, void* out, int B, int H, int D, int nd, const int* shape,
                   const int* kernel, const int* dilation, float scale, int dtype, void* stream) {
  pnm::NaGeom g;
  if (pnm::na_geom(g, nd, shape, kernel, dilation) || D > pnm::kNaMaxD || D < 1) return -1;
  const long long total = (long long)B * g.L * H;
  if (total <= 0) return 0;
  const size_t smem = pnm::kNaWarps * pnm::na_align16((size_t)(D + g.K) * sizeof(float) + (size_t)g.K * sizeof(long long));
  const unsigned grid = (unsigned)((total + pnm::kNaWarps - 1) / pnm::kNaWarps);
  cudaStream_t st = (cudaStream_t)stream;
  if (dtype == 0)
    pnm::natten_fwd_kernel<__nv_bfloat16><<<grid, pnm::kNaWarps * 32, smem, st>>>(
        (const __nv_bfloat16*)q, (const __nv_bfloat16*)k, (const __nv_bfloat16*)v, (__nv_bfloat16*)out, g, H, D, total, scale);
  else
    pnm::natten_fwd_kernel<float><<<grid, pnm::kNaWarps * 32, smem, st>>>((const float*)q, (const float*)k, (const float*)v,
                                                                         (float*)out, g, H, D, total, scale);
  return (int)cudaGetLastError();
}

// dk / dv: fp32 accumulators [B, L, H, D], zeroed by the caller
int pnm_natten_bwd(const void* q, const void* k, const void* v, const void* dout, void* dq, float* dk, float* dv, int B, int H,
                   int D, int nd, const int* shape, const int* kernel, const int* dilation, float scale, int dtype,
                   void* stream) {
  pnm::NaGeom g;
  if (pnm::na_geom(g, nd, shape, kernel, dilation) || D > pnm::kNaMaxD || D < 1) return -1;
  const long long total = (long long)B * g.L * H;
  if (total <= 0) return 0;
  const size_t smem = pnm::kNaWarps * pnm::na_align16((size_t)(2 * D + 2 * g.K) * sizeof(float) + (size_t)g.K * sizeof(long long));
  const unsigned grid = (unsigned)((total + pnm::kNaWarps - 1) / pnm::kNaWarps);
  cudaStream_t st = (cudaStream_t)stream;
  if (dtype == 0)
    pnm::natten_bwd_kernel<__nv_bfloat16><<<grid, pnm::kNaWarps * 32, smem, st>>>(
        (const __nv_bfloat16*)q, (const __nv_bfloat16*)k, (const __nv_bfloat16*)v, (const __nv_bfloat16*)dout,
        (__nv_bfloat16*)dq, dk, dv, g, H, D, total, scale);
  else
    pnm::natten_bwd_kernel<float><<<grid, pnm::kNaWarps * 32, smem, st>>>((const float*)q, (const float*)k, (const float*)v,
                                                                         (const float*)dout, (float*)dq, dk, dv, g, H, D,
                                                                         total, scale);
  return (int)cudaGetLastError();
}

}  // extern "C"
