// Neighbour queries on point clouds: fixed-radius search over a cell list, brute-force k-nearest
// neighbours with shared-memory tiles, and farthest point sampling.
//
// Radius search: the host sorts the points by cell of a uniform grid (cell edge >= radius) and
// passes [cell_start, cell_end) per cell; a query visits the 27 cells around its own.  The ragged
// form is count -> (host-side prefix sum) -> fill; the capped form keeps the `max_points` nearest
// hits of a query, sorted by distance, in that query's own output row.
#include <cuda_runtime.h>
#include <float.h>
#include <stdint.h>

#include "pnm_api.h"

namespace pnm {

struct CellGrid {
  float lo[3];
  float inv_cell;
  int n[3];
};

__device__ __forceinline__ int clampi(int v, int lo, int hi) { return v < lo ? lo : (v > hi ? hi : v); }

template <typename F>
__device__ __forceinline__ void for_each_candidate(const CellGrid& g, const int* __restrict__ cell_start,
                                                   const int* __restrict__ cell_end, float qx, float qy, float qz, F&& f) {
  // cells of the query, possibly outside the grid: visit the overlap of [c-1, c+1] with the grid
  const int cx = (int)floorf((qx - g.lo[0]) * g.inv_cell), cy = (int)floorf((qy - g.lo[1]) * g.inv_cell),
            cz = (int)floorf((qz - g.lo[2]) * g.inv_cell);
  const int x0 = max(cx - 1, 0), x1 = min(cx + 1, g.n[0] - 1);
  const int y0 = max(cy - 1, 0), y1 = min(cy + 1, g.n[1] - 1);
  const int z0 = max(cz - 1, 0), z1 = min(cz + 1, g.n[2] - 1);
  for (int x = x0; x <= x1; ++x)
    for (int y = y0; y <= y1; ++y)
      for (int z = z0; z <= z1; ++z) {
        const int cell = (x * g.n[1] + y) * g.n[2] + z;
        for (int k = cell_start[cell]; k < cell_end[cell]; ++k) f(k);
      }
}

__global__ void radius_count_kernel(const float* __restrict__ pts, const int* __restrict__ cell_start,
                                    const int* __restrict__ cell_end, const float* __restrict__ queries,
                                    int* __restrict__ counts, const __grid_constant__ CellGrid g, int nq, float r2) {
  const int q = blockIdx.x * blockDim.x + threadIdx.x;
  if (q >= nq) return;
  const float qx = queries[3 * q], qy = queries[3 * q + 1], qz = queries[3 * q + 2];
  int c = 0;
  for_each_candidate(g, cell_start, cell_end, qx, qy, qz, [&](int k) {
    const float dx = pts[3 * k] - qx, dy = pts[3 * k + 1] - qy, dz = pts[3 * k + 2] - qz;
    c += (dx * dx + dy * dy + dz * dz <= r2) ? 1 : 0;
  });
  counts[q] = c;
}

// pairs: [2, total] (row 0 = query index, row 1 = original point index)
__global__ void radius_fill_kernel(const float* __restrict__ pts, const int* __restrict__ order,
                                   const int* __restrict__ cell_start, const int* __restrict__ cell_end,
                                   const float* __restrict__ queries, const long long* __restrict__ offsets,
                                   long long* __restrict__ pairs, long long total, const __grid_constant__ CellGrid g,
                                   int nq, float r2) {
  const int q = blockIdx.x * blockDim.x + threadIdx.x;
  if (q >= nq) return;
  const float qx = queries[3 * q], qy = queries[3 * q + 1], qz = queries[3 * q + 2];
  long long at = offsets[q];
  const long long end = offsets[q + 1];
  for_each_candidate(g, cell_start, cell_end, qx, qy, qz, [&](int k) {
    const float dx = pts[3 * k] - qx, dy = pts[3 * k + 1] - qy, dz = pts[3 * k + 2] - qz;
    if (dx * dx + dy * dy + dz * dz <= r2 && at < end) {
      pairs[at] = q;
      pairs[total + at] = order[k];
      ++at;
    }
  });
}

// idx: [nq, K] (int64, -1 = empty), d2: [nq, K]; rows sorted by distance.
__global__ void radius_topk_kernel(const float* __restrict__ pts, const int* __restrict__ order,
                                   const int* __restrict__ cell_start, const int* __restrict__ cell_end,
                                   const float* __restrict__ queries, long long* __restrict__ idx, float* __restrict__ d2out,
                                   const __grid_constant__ CellGrid g, int nq, int K, float r2) {
  const int q = blockIdx.x * blockDim.x + threadIdx.x;
  if (q >= nq) return;
  const float qx = queries[3 * q], qy = queries[3 * q + 1], qz = queries[3 * q + 2];
  long long* row = idx + (long long)q * K;
  float* drow = d2out + (long long)q * K;
  int have = 0;
  for_each_candidate(g, cell_start, cell_end, qx, qy, qz, [&](int k) {
    const float dx = pts[3 * k] - qx, dy = pts[3 * k + 1] - qy, dz = pts[3 * k + 2] - qz;
    const float d = dx * dx + dy * dy + dz * dz;
    if (d > r2) return;
    if (have == K && d >= drow[K - 1]) return;
    int pos = have < K ? have : K - 1;
    const long long id = order[k];
    // ties are broken by the smaller point index so that the result does not depend on the visiting order
    while (pos > 0 && (drow[pos - 1] > d || (drow[pos - 1] == d && row[pos - 1] > id))) {
      drow[pos] = drow[pos - 1];
      row[pos] = row[pos - 1];
      --pos;
    }
    drow[pos] = d;
    row[pos] = id;
    if (have < K) ++have;
  });
  for (int j = have; j < K; ++j) { row[j] = -1; drow[j] = 0.f; }
}

// ------------------------------------------------------------------ brute-force kNN
constexpr int kKnnTile = 1024;
constexpr int kKnnThreads = 128;

template <int D, int KMAX>
__global__ void __launch_bounds__(kKnnThreads)
knn_kernel(const float* __restrict__ pts, const float* __restrict__ queries, long long* __restrict__ idx,
           float* __restrict__ dist, int np, int nq, int K) {
  __shared__ float tile[kKnnTile * D];
  const int q = blockIdx.x * blockDim.x + threadIdx.x;
  float qc[D];
#pragma unroll
  for (int a = 0; a < D; ++a) qc[a] = q < nq ? queries[(long long)q * D + a] : 0.f;
  float bd[KMAX];
  int bi[KMAX];
#pragma unroll
  for (int j = 0; j < KMAX; ++j) { bd[j] = FLT_MAX; bi[j] = -1; }
  for (int base = 0; base < np; base += kKnnTile) {
    const int cnt = min(kKnnTile, np - base);
    __syncthreads();
    for (int t = threadIdx.x; t < cnt * D; t += blockDim.x) tile[t] = pts[(long long)base * D + t];
    __syncthreads();
    if (q < nq) {
      for (int t = 0; t < cnt; ++t) {
        float d = 0.f;
#pragma unroll
        for (int a = 0; a < D; ++a) { const float e = tile[t * D + a] - qc[a]; d += e * e; }
        if (d < bd[K - 1]) {
          // insertion with a fixed trip count keeps the list in registers
          float cd = d;
          int ci = base + t;
#pragma unroll
          for (int j = 0; j < KMAX; ++j) {
            if (j < K && cd < bd[j]) {
              const float td = bd[j]; const int ti = bi[j];
              bd[j] = cd; bi[j] = ci;
              cd = td; ci = ti;
            }
          }
        }
      }
    }
  }
  if (q < nq) {
#pragma unroll
    for (int j = 0; j < KMAX; ++j)
      if (j < K) { idx[(long long)q * K + j] = bi[j]; dist[(long long)q * K + j] = sqrtf(bd[j]); }
  }
}

// ------------------------------------------------------------------ farthest point sampling
constexpr int kFpsThreads = 1024;

// pts: [B, N, 3]; mind: [B, N] scratch; out: [B, S] int64 with column 0 preset to the first sample.  One CTA per cloud.
__global__ void __launch_bounds__(kFpsThreads)
fps_kernel(const float* __restrict__ pts, float* __restrict__ mind, long long* __restrict__ out, int N, int S) {
  const int b = blockIdx.x;
  const float* P = pts + (long long)b * N * 3;
  float* md = mind + (long long)b * N;
  __shared__ float sval[kFpsThreads / 32];
  __shared__ int sidx[kFpsThreads / 32];
  __shared__ int cur;
  for (int i = threadIdx.x; i < N; i += blockDim.x) md[i] = FLT_MAX;
  if (threadIdx.x == 0) cur = (int)out[(long long)b * S];  // the host chooses the first sample
  __syncthreads();
  for (int s = 1; s < S; ++s) {
    const int c = cur;
    const float cx = P[3 * c], cy = P[3 * c + 1], cz = P[3 * c + 2];
    float best = -1.f;
    int bi = 0;
    for (int i = threadIdx.x; i < N; i += blockDim.x) {
      const float dx = P[3 * i] - cx, dy = P[3 * i + 1] - cy, dz = P[3 * i + 2] - cz;
      const float d = fminf(md[i], dx * dx + dy * dy + dz * dz);
      md[i] = d;
      if (d > best) { best = d; bi = i; }   // smallest index wins ties within a thread (ascending i)
    }
    for (int o = 16; o; o >>= 1) {
      const float ov = __shfl_down_sync(0xffffffffu, best, o);
      const int oi = __shfl_down_sync(0xffffffffu, bi, o);
      if (ov > best || (ov == best && oi < bi)) { best = ov; bi = oi; }
    }
    if ((threadIdx.x & 31) == 0) { sval[threadIdx.x >> 5] = best; sidx[threadIdx.x >> 5] = bi; }
    __syncthreads();
    if (threadIdx.x < 32) {
      best = threadIdx.x < kFpsThreads / 32 ? sval[threadIdx.x] : -2.f;
      bi = threadIdx.x < kFpsThreads / 32 ? sidx[threadIdx.x] : 0x7fffffff;
      for (int o = 16; o; o >>= 1) {
        const float ov = __shfl_down_sync(0xffffffffu, best, o);
        const int oi = __shfl_down_sync(0xffffffffu, bi, o);
        if (ov > best || (ov == best && oi < bi)) { best = ov; bi = oi; }
      }
      if (threadIdx.x == 0) { cur = bi; out[(long long)b * S + s] = bi; }
    }
    __syncthreads();
  }
}

}  // namespace pnm

template <int D>
static int knn_launch(const float* pts, const float* q, long long* idx, float* dist, int np, int nq, int K, cudaStream_t st) {
  const unsigned blocks = (nq + pnm::kKnnThreads - 1) / pnm::kKnnThreads;
  if (K <= 8) pnm::knn_kernel<D, 8><<<blocks, pnm::kKnnThreads, 0, st>>>(pts, q, idx, dist, np, nq, K);
  else if (K <= 16) pnm::knn_kernel<D, 16><<<blocks, pnm::kKnnThreads, 0, st>>>(pts, q, idx, dist, np, nq, K);
  else if (K <= 32) pnm::knn_kernel<D, 32><<<blocks, pnm::kKnnThreads, 0, st>>>(pts, q, idx, dist, np, nq, K);
  else pnm::knn_kernel<D, 64><<<blocks, pnm::kKnnThreads, 0, st>>>(pts, q, idx, dist, np, nq, K);
  return (int)cudaGetLastError();
}

extern "C" {

static pnm::CellGrid make_grid(const float* lo, float cell, const int* n) {
  pnm::CellGrid g;
  for (int a = 0; a < 3; ++a) { g.lo[a] = lo[a]; g.n[a] = n[a]; }
  g.inv_cell = 1.f / cell;
  return g;
}

int pnm_radius_count(const float* pts_sorted, const int* cell_start, const int* cell_end, const float* queries,
                     int* counts, const float* lo, float cell, const int* n, int nq, float radius, void* stream) {
  if (nq <= 0) return 0;
  pnm::radius_count_kernel<<<(nq + 127) / 128, 128, 0, (cudaStream_t)stream>>>(
      pts_sorted, cell_start, cell_end, queries, counts, make_grid(lo, cell, n), nq, radius * radius);
  return (int)cudaGetLastError();
}

int pnm_radius_fill(const float* pts_sorted, const int* order, const int* cell_start, const int* cell_end,
                    const float* queries, const long long* offsets, long long* pairs, long long total, const float* lo,
                    float cell, const int* n, int nq, float radius, void* stream) {
  if (nq <= 0 || total <= 0) return 0;
  pnm::radius_fill_kernel<<<(nq + 127) / 128, 128, 0, (cudaStream_t)stream>>>(
      pts_sorted, order, cell_start, cell_end, queries, offsets, pairs, total, make_grid(lo, cell, n), nq, radius * radius);
  return (int)cudaGetLastError();
}

int pnm_radius_topk(const float* pts_sorted, const int* order, const int* cell_start, const int* cell_end,
                    const float* queries, long long* idx, float* d2, const float* lo, float cell, const int* n, int nq,
                    int K, float radius, void* stream) {
  if (nq <= 0 || K <= 0) return 0;
  pnm::radius_topk_kernel<<<(nq + 127) / 128, 128, 0, (cudaStream_t)stream>>>(
      pts_sorted, order, cell_start, cell_end, queries, idx, d2, make_grid(lo, cell, n), nq, K, radius * radius);
  return (int)cudaGetLastError();
}

int pnm_knn_max_k() { return 64; }

int pnm_knn(const float* pts, const float* queries, long long* idx, float* dist, int np, int nq, int D, int K, void* stream) {
  if (nq <= 0) return 0;
  if (K < 1 || K > 64 || K > np) return -1;
  cudaStream_t st = (cudaStream_t)stream;
  switch (D) {
    case 1: return knn_launch<1>(pts, queries, idx, dist, np, nq, K, st);
    case 2: return knn_launch<2>(pts, queries, idx, dist, np, nq, K, st);
    case 3: return knn_launch<3>(pts, queries, idx, dist, np, nq, K, st);
    default: return -2;
  }
}

int pnm_fps(const float* pts, float* scratch, long long* out, int B, int N, int S, void* stream) {
  if (B <= 0 || S <= 0) return 0;
  if (S > N) return -1;
  pnm::fps_kernel<<<B, pnm::kFpsThreads, 0, (cudaStream_t)stream>>>(pts, scratch, out, N, S);
  return (int)cudaGetLastError();
}

}  // extern "C"
