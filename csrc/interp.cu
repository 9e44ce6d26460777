// Grid <-> point interpolation on uniform 1-3-D grids.
//
// For a query point the stencil is the stride^D block of grid nodes around it (stride 1 nearest,
// 2 linear / smooth-step, 5 Gaussian).  `gather` evaluates out[p, c] = sum_j w_j grid[c, node_j];
// `scatter` is its transpose, grid[c, node_j] += w_j vals[p, c] (atomics).  Nodes outside the grid
// contribute zero (the grid is treated as zero-padded).  One thread per (point, channel).
#include <cuda_runtime.h>
#include <stdint.h>

#include "pnm_api.h"

namespace pnm {

struct InterpGrid {
  float x0[3], dx[3];
  int n[3];
  int dims;
  int type;  // 0 nearest, 1 linear, 2 smooth_step_1, 3 smooth_step_2, 4 gaussian
};

__device__ __forceinline__ float step_fn(int type, float x) {
  x = fminf(fmaxf(x, 0.f), 1.f);
  if (type == 2) return x * x * (3.f - 2.f * x);
  if (type == 3) return x * x * x * (x * (6.f * x - 15.f) + 10.f);
  return x;
}

// Per-axis stencil of one point: first node index (may be out of range), node count, weights.
struct AxisStencil {
  int first;
  float w[5];
};

__device__ __forceinline__ void axis_stencil(const InterpGrid& g, int a, float q, int stride, AxisStencil& s) {
  const float t = (q - g.x0[a]) / g.dx[a];
  if (stride == 1) {
    s.first = (int)floorf(t + 0.5f);
    s.w[0] = 1.f;
  } else if (stride == 2) {
    const float fl = floorf(t);
    s.first = (int)fl;
    const float lower = t - fl;           // distance to the lower node, in cells
    s.w[0] = step_fn(g.type, 1.f - lower);
    s.w[1] = step_fn(g.type, lower);
  } else {
    const int c = (int)floorf(t + 0.5f);
    s.first = c - 2;
#pragma unroll
    for (int j = 0; j < 5; ++j) {
      const float d = (t - float(c - 2 + j)) * 2.f;  // distance / sigma, sigma = dx / 2
      s.w[j] = __expf(-0.5f * d * d);
    }
  }
}

template <bool SCATTER>
__global__ void __launch_bounds__(256)
interp_kernel(const float* __restrict__ pts, const float* __restrict__ src, float* __restrict__ dst,
              const __grid_constant__ InterpGrid g, long long npts, int C) {
  const long long tid = blockIdx.x * (long long)blockDim.x + threadIdx.x;
  if (tid >= npts * C) return;
  const long long p = tid / C;
  const int c = int(tid % C);
  const int stride = g.type == 0 ? 1 : (g.type == 4 ? 5 : 2);
  AxisStencil s[3];
#pragma unroll
  for (int a = 0; a < 3; ++a) {
    if (a < g.dims) axis_stencil(g, a, pts[p * g.dims + a], stride, s[a]);
    else { s[a].first = 0; s[a].w[0] = 1.f; }
  }
  const int m0 = stride, m1 = g.dims > 1 ? stride : 1, m2 = g.dims > 2 ? stride : 1;
  const long long n1 = g.dims > 1 ? g.n[1] : 1, n2 = g.dims > 2 ? g.n[2] : 1;
  const long long cells = (long long)g.n[0] * n1 * n2;
  float norm = 1.f;
  if (g.type == 4) {  // Gaussian weights are normalised over the whole (padded) block
    float s0 = 0.f, s1 = 0.f, s2 = 0.f;
    for (int j = 0; j < m0; ++j) s0 += s[0].w[j];
    for (int j = 0; j < m1; ++j) s1 += s[1].w[j];
    for (int j = 0; j < m2; ++j) s2 += s[2].w[j];
    norm = 1.f / (s0 * s1 * s2);
  }
  const float val = SCATTER ? src[p * C + c] : 0.f;
  float acc = 0.f;
  for (int j0 = 0; j0 < m0; ++j0) {
    const int i0 = s[0].first + j0;
    if (i0 < 0 || i0 >= g.n[0]) continue;
    for (int j1 = 0; j1 < m1; ++j1) {
      const int i1 = s[1].first + j1;
      if (i1 < 0 || i1 >= n1) continue;
      for (int j2 = 0; j2 < m2; ++j2) {
        const int i2 = s[2].first + j2;
        if (i2 < 0 || i2 >= n2) continue;
        const float w = s[0].w[j0] * s[1].w[j1] * s[2].w[j2] * norm;
        const long long node = c * cells + ((long long)i0 * n1 + i1) * n2 + i2;
        if (SCATTER) atomicAdd(&dst[node], w * val);
        else acc += w * src[node];
      }
    }
  }
  if (!SCATTER) dst[p * C + c] = acc;
}

}  // namespace pnm

extern "C" {

// grid_desc: host array [x0_0..2, dx_0..2] floats; n: host int[3]. scatter == 0: src = grid [C, *n], dst = out [npts, C];
// scatter != 0: src = vals [npts, C], dst = grid [C, *n] (accumulated into).
int pnm_interp(const float* pts, const float* src, float* dst, const float* grid_desc, const int* n, int dims, int type,
               long long npts, int C, int scatter, void* stream) {
  if (npts <= 0 || C <= 0) return 0;
  if (dims < 1 || dims > 3 || type < 0 || type > 4) return -1;
  pnm::InterpGrid g;
  for (int a = 0; a < 3; ++a) { g.x0[a] = grid_desc[a]; g.dx[a] = grid_desc[3 + a]; g.n[a] = n[a]; }
  g.dims = dims;
  g.type = type;
  const long long work = npts * C;
  const unsigned blocks = (unsigned)((work + 255) / 256);
  if (scatter) pnm::interp_kernel<true><<<blocks, 256, 0, (cudaStream_t)stream>>>(pts, src, dst, g, npts, C);
  else pnm::interp_kernel<false><<<blocks, 256, 0, (cudaStream_t)stream>>>(pts, src, dst, g, npts, C);
  return (int)cudaGetLastError();
}

}  // extern "C"
