// Darcy-flow data generator: random piecewise-constant permeability and the multigrid Jacobi pressure solve.
//
// The whole solve of a batch is ONE cooperative launch: a persistent grid walks the multigrid levels
// (coarse -> fine), runs Jacobi sweeps separated by grid-wide barriers, checks the max-norm update every
// `check_every` sweeps on the device (all CTAs read the same reduced value, so the exit decision is uniform)
// and prolongates to the next level - no host round trip inside the solve.
//
//   -div(k grad u) = 1 on the unit square, u = 0 on the boundary; nodes (b, x, y), x,y in [0, L), L = res + 1.
#include <cooperative_groups.h>
#include <cuda_runtime.h>
#include <stdint.h>

#include "pnm_api.h"

namespace cg = cooperative_groups;

namespace pnm {

__device__ __forceinline__ float at_zero(const float* a, long long base, int x, int y, int L) {
  return (x < 0 || y < 0 || x >= L || y >= L) ? 0.f : a[base + (long long)x * L + y];
}
__device__ __forceinline__ float at_clamp(const float* a, long long base, int x, int y, int L) {
  x = min(max(x, 0), L - 1);
  y = min(max(y, 0), L - 1);
  return a[base + (long long)x * L + y];
}

// k[b, x, y] = (sum_ij f0 sin sin + f1 cos sin + f2 sin cos + f3 cos cos) / nf^2 < 0 ? kmin : kmax
__global__ void darcy_permeability_kernel(const float* __restrict__ fourier, float* __restrict__ perm, int B, int L,
                                          int res, int nf, float kmin, float kmax) {
  const long long tid = blockIdx.x * (long long)blockDim.x + threadIdx.x;
  const long long total = (long long)B * L * L;
  if (tid >= total) return;
  const int y = int(tid % L), x = int((tid / L) % L), b = int(tid / ((long long)L * L));
  const float rx = 6.28318f / float(res) * float(x), ry = 6.28318f / float(res) * float(y);
  const long long plane = (long long)B * nf * nf;
  float acc = 0.f;
  for (int i = 0; i < nf; ++i) {
    float si, ci;
    __sincosf(float(i) * rx, &si, &ci);
    for (int j = 0; j < nf; ++j) {
      float sj, cj;
      __sincosf(float(j) * ry, &sj, &cj);
      const long long o = ((long long)b * nf + i) * nf + j;
      acc += fourier[o] * si * sj + fourier[plane + o] * ci * sj + fourier[2 * plane + o] * si * cj +
             fourier[3 * plane + o] * ci * cj;
    }
  }
  perm[tid] = (acc / float(nf * nf)) < 0.f ? kmin : kmax;
}

struct DarcyArgs {
  float* u0;
  float* u1;
  const float* perm;
  unsigned int* residual;  // two words: [0] running max (float bits), [1] sweeps done (for reporting)
  int B, L, res, levels, max_iterations, check_every;
  float dx, threshold;
};

__global__ void __launch_bounds__(256)
darcy_multigrid_kernel(const DarcyArgs a) {
  cg::grid_group grid = cg::this_grid();
  const long long nthreads = (long long)gridDim.x * blockDim.x;
  const long long t0 = blockIdx.x * (long long)blockDim.x + threadIdx.x;
  const int L = a.L;
  float* cur = a.u0;
  float* nxt = a.u1;
  unsigned int sweeps_total = 0;
  for (int level = 0; level < a.levels; ++level) {
    const int f = 1 << (a.levels - level - 1);       // grid reduction factor of this level
    const int n = f > 1 ? a.res / f : L;             // nodes per side on this level
    const long long work = (long long)a.B * n * n;
    const float gdx = a.dx * float(f);
    const float inv_dx2 = 1.f / (gdx * gdx);
    const int chunks = a.max_iterations / a.check_every;
    for (int c = 0; c < chunks; ++c) {
      for (int s = 0; s < a.check_every; ++s) {
        for (long long w = t0; w < work; w += nthreads) {
          const int y = int(w % n), x = int((w / n) % n), b = int(w / ((long long)n * n));
          const int gx = f * x + (f - 1), gy = f * y + (f - 1);
          const long long base = (long long)b * L * L;
          const float d01 = at_zero(cur, base, gx - f, gy, L), d21 = at_zero(cur, base, gx + f, gy, L);
          const float d10 = at_zero(cur, base, gx, gy - f, L), d12 = at_zero(cur, base, gx, gy + f, L);
          const float p11 = at_clamp(a.perm, base, gx, gy, L);
          const float p01 = at_clamp(a.perm, base, gx - f, gy, L), p21 = at_clamp(a.perm, base, gx + f, gy, L);
          const float p10 = at_clamp(a.perm, base, gx, gy - f, L), p12 = at_clamp(a.perm, base, gx, gy + f, L);
          const float t1 = p11 * (d01 + d21 + d10 + d12) * inv_dx2;
          const float t2 = (p21 - p01) * (d21 - d01) / (2.f * gdx);
          const float t3 = (p12 - p10) * (d12 - d10) / (2.f * gdx);
          nxt[base + (long long)gx * L + gy] = (t1 + t2 + t3 + 1.f) / (p11 * 4.f * inv_dx2);
        }
        grid.sync();
        float* tmp = cur; cur = nxt; nxt = tmp;
      }
      sweeps_total += a.check_every;
      // max-norm of the last update over the level's nodes
      float local = 0.f;
      for (long long w = t0; w < work; w += nthreads) {
        const int y = int(w % n), x = int((w / n) % n), b = int(w / ((long long)n * n));
        const long long idx = (long long)b * L * L + (long long)(f * x + f - 1) * L + (f * y + f - 1);
        local = fmaxf(local, fabsf(cur[idx] - nxt[idx]));
      }
      for (int o = 16; o; o >>= 1) local = fmaxf(local, __shfl_xor_sync(0xffffffffu, local, o));
      if ((threadIdx.x & 31) == 0 && local > 0.f) atomicMax(a.residual, __float_as_uint(local));
      grid.sync();
      const float res_now = __uint_as_float(*((volatile unsigned int*)a.residual));
      grid.sync();
      if (t0 == 0) a.residual[0] = 0u;
      grid.sync();
      if (res_now < a.threshold * float(f)) break;
    }
    if (f > 1) {
      // prolongation: fill every fine node by bilinear interpolation of this level's nodes (out of place)
      const long long fine = (long long)a.B * L * L;
      for (long long w = t0; w < fine; w += nthreads) {
        const int y = int(w % L), x = int((w / L) % L), b = int(w / ((long long)L * L));
        const long long base = (long long)b * L * L;
        const int rx = (x + 1) % f, ry = (y + 1) % f;
        const int x0 = x - rx, x1 = x + rx, y0 = y - ry, y1 = y + ry;
        const float d00 = at_zero(cur, base, x0, y0, L), d10 = at_zero(cur, base, x1, y0, L);
        const float d01 = at_zero(cur, base, x0, y1, L), d11 = at_zero(cur, base, x1, y1, L);
        const float fx = float(x - x0) / float(f), fy = float(y - y0) / float(f);
        nxt[w] = (1.f - fy) * ((1.f - fx) * d00 + fx * d10) + fy * ((1.f - fx) * d01 + fx * d11);
      }
      grid.sync();
      float* tmp = cur; cur = nxt; nxt = tmp;
    }
  }
  // the caller reads the solution from u0
  if (cur != a.u0) {
    const long long fine = (long long)a.B * L * L;
    for (long long w = t0; w < fine; w += nthreads) a.u0[w] = cur[w];
  }
  if (t0 == 0) a.residual[1] = sweeps_total;
}

}  // namespace pnm

extern "C" {

int pnm_darcy_permeability(const float* fourier, float* perm, int B, int res, int nf, float kmin, float kmax, void* stream) {
  const int L = res + 1;
  const long long total = (long long)B * L * L;
  if (total <= 0) return 0;
  pnm::darcy_permeability_kernel<<<(unsigned)((total + 255) / 256), 256, 0, (cudaStream_t)stream>>>(fourier, perm, B, L, res,
                                                                                                nf, kmin, kmax);
  return (int)cudaGetLastError();
}

// u0, u1: [B, res+1, res+1] zero-initialised work arrays (solution returned in u0); residual: 2 zeroed words.
int pnm_darcy_solve(float* u0, float* u1, const float* perm, unsigned int* residual, int B, int res, int levels,
                    int max_iterations, int check_every, float threshold, void* stream) {
  if (B <= 0) return 0;
  if (levels < 1 || check_every < 1 || (res % (1 << (levels - 1))) != 0) return -1;
  pnm::DarcyArgs a;
  a.u0 = u0; a.u1 = u1; a.perm = perm; a.residual = residual;
  a.B = B; a.L = res + 1; a.res = res; a.levels = levels;
  a.max_iterations = max_iterations; a.check_every = check_every;
  a.dx = 1.f / float(res + 1); a.threshold = threshold;
  int dev = 0, sms = 0, per_sm = 0;
  cudaGetDevice(&dev);
  cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev);
  cudaOccupancyMaxActiveBlocksPerMultiprocessor(&per_sm, pnm::darcy_multigrid_kernel, 256, 0);
  if (per_sm < 1) return -2;
  const long long fine = (long long)B * a.L * a.L;
  long long blocks = (long long)sms * per_sm;
  blocks = blocks < (fine + 255) / 256 ? blocks : (fine + 255) / 256;
  void* params[] = {&a};
  return (int)cudaLaunchCooperativeKernel((void*)pnm::darcy_multigrid_kernel, dim3((unsigned)blocks), dim3(256), params, 0,
                                          (cudaStream_t)stream);
}

}  // extern "C"
