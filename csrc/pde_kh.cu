// Kelvin-Helmholtz data generator: 2-D compressible Euler, second-order MUSCL-Hancock finite volumes with a
// Rusanov flux on a periodic square.
//
// One cooperative launch integrates a whole batch through all snapshots.  A time step is two grid-wide phases:
//   A  per cell: primitives of the cell and its four neighbours (from the conserved state), central slopes,
//      half-step predictor, extrapolation to the four faces            -> faces[16][B,N,N]
//   B  per cell: Rusanov fluxes through its four faces (the two "minus" faces are recomputed from the
//      neighbours' face states instead of being stored) and the conservative update.
// Snapshots of (rho, v, p) are written from the conserved state at the start of every snapshot interval.
#include <cooperative_groups.h>
#include <cuda_runtime.h>
#include <stdint.h>

#include "pnm_api.h"

namespace cg = cooperative_groups;

namespace pnm {

struct Prim { float r, u, v, p; };

struct KhArgs {
  float* cons;         // [4][B,N,N]: mass, mom_x, mom_y, energy (cell totals)
  float* faces;        // [16][B,N,N]: (r,u,v,p) x (xl, xr, yl, yr)
  const float* w;      // [B, nfreq] perturbation amplitudes
  float* snap_rho;     // [S,B,N,N]
  float* snap_vel;     // [S,B,N,N,2]
  float* snap_p;       // [S,B,N,N]
  int B, N, nfreq, snapshots, steps_per_snapshot;
  float gamma, dx, dt, vol, sigma;
};

__device__ __forceinline__ int pwrap(int i, int n) { return i < 0 ? i + n : (i >= n ? i - n : i); }

__device__ __forceinline__ Prim to_prim(const float* cons, long long plane, long long idx, float gamma, float vol) {
  const float m = cons[idx], mx = cons[plane + idx], my = cons[2 * plane + idx], e = cons[3 * plane + idx];
  Prim q;
  q.r = m / vol;
  q.u = mx / q.r / vol;
  q.v = my / q.r / vol;
  q.p = (e / vol - 0.5f * q.r * (q.u * q.u + q.v * q.v)) * (gamma - 1.f);
  return q;
}

// Rusanov flux along the face normal; (un, ut) are normal / tangential velocities. Returns mass, mom_n, mom_t, energy.
__device__ __forceinline__ float4 rusanov(float rl, float rr, float unl, float unr, float utl, float utr, float pl, float pr,
                                          float gamma) {
  const float el = pl / (gamma - 1.f) + 0.5f * rl * (unl * unl + utl * utl);
  const float er = pr / (gamma - 1.f) + 0.5f * rr * (unr * unr + utr * utr);
  const float ra = 0.5f * (rl + rr), mn = 0.5f * (rl * unl + rr * unr), mt = 0.5f * (rl * utl + rr * utr);
  const float ea = 0.5f * (el + er);
  const float pa = (gamma - 1.f) * (ea - 0.5f * (mn * mn + mt * mt) / ra);
  const float c = fmaxf(sqrtf(gamma * pl / rl) + fabsf(unl), sqrtf(gamma * pr / rr) + fabsf(unr));
  float4 f;
  f.x = mn - c * 0.5f * (rl - rr);
  f.y = mn * mn / ra + pa - c * 0.5f * (rl * unl - rr * unr);
  f.z = mn * mt / ra - c * 0.5f * (rl * utl - rr * utr);
  f.w = (ea + pa) * mn / ra - c * 0.5f * (el - er);
  return f;
}

__global__ void __launch_bounds__(256)
kh_simulate_kernel(const KhArgs a) {
  cg::grid_group grid = cg::this_grid();
  const long long nthreads = (long long)gridDim.x * blockDim.x;
  const long long t0 = blockIdx.x * (long long)blockDim.x + threadIdx.x;
  const int N = a.N;
  const long long plane = (long long)a.B * N * N;
  // ---- initial condition (primitive) -> conserved
  for (long long c = t0; c < plane; c += nthreads) {
    const int j = int(c % N), i = int((c / N) % N), b = int(c / ((long long)N * N));
    const float x = float(i) / float(N), y = float(j) / float(N);
    const bool band = fabsf(y - 0.5f) < 0.25f;
    const float ux = band ? 0.5f : -0.5f, r = band ? 2.f : 1.f;
    const float s2 = 2.f * a.sigma * a.sigma;
    const float env = __expf(-(y - 0.25f) * (y - 0.25f) / s2) + __expf(-(y - 0.75f) * (y - 0.75f) / s2);
    float uy = 0.f;
    for (int f = 0; f < a.nfreq; ++f) {
      const float ff = float(f + 1);
      uy += ff * a.w[b * a.nfreq + f] * __sinf(4.f * 3.14159f * x * ff) * env;
    }
    const float p = 2.5f;
    a.cons[c] = r * a.vol;
    a.cons[plane + c] = ux * r * a.vol;
    a.cons[2 * plane + c] = uy * r * a.vol;
    a.cons[3 * plane + c] = (p / (a.gamma - 1.f) + 0.5f * r * (ux * ux + uy * uy)) * a.vol;
  }
  grid.sync();
  const float hdx = 0.5f * a.dx, inv2dx = 1.f / (2.f * a.dx);
  for (int s = 0; s < a.snapshots; ++s) {
    for (long long c = t0; c < plane; c += nthreads) {
      const Prim q = to_prim(a.cons, plane, c, a.gamma, a.vol);
      const long long o = (long long)s * plane + c;
      a.snap_rho[o] = q.r;
      a.snap_vel[2 * o] = q.u;
      a.snap_vel[2 * o + 1] = q.v;
      a.snap_p[o] = q.p;
    }
    for (int it = 0; it < a.steps_per_snapshot; ++it) {
      // ---------------------------------------------------------------- phase A
      for (long long c = t0; c < plane; c += nthreads) {
        const int j = int(c % N), i = int((c / N) % N);
        const long long base = c - ((long long)i * N + j);
        auto at = [&](int ii, int jj) { return base + (long long)pwrap(ii, N) * N + pwrap(jj, N); };
        const Prim q = to_prim(a.cons, plane, c, a.gamma, a.vol);
        const Prim xe = to_prim(a.cons, plane, at(i + 1, j), a.gamma, a.vol), xw = to_prim(a.cons, plane, at(i - 1, j), a.gamma, a.vol);
        const Prim yn = to_prim(a.cons, plane, at(i, j + 1), a.gamma, a.vol), ys = to_prim(a.cons, plane, at(i, j - 1), a.gamma, a.vol);
        const float rdx = (xe.r - xw.r) * inv2dx, rdy = (yn.r - ys.r) * inv2dx;
        const float udx = (xe.u - xw.u) * inv2dx, udy = (yn.u - ys.u) * inv2dx;
        const float vdx = (xe.v - xw.v) * inv2dx, vdy = (yn.v - ys.v) * inv2dx;
        const float pdx = (xe.p - xw.p) * inv2dx, pdy = (yn.p - ys.p) * inv2dx;
        const float h = 0.5f * a.dt;
        const float r1 = q.r - h * (q.u * rdx + q.r * udx + q.v * rdy + q.r * vdy);
        const float u1 = q.u - h * (q.u * udx + q.v * udy + pdx / q.r);
        const float v1 = q.v - h * (q.u * vdx + q.v * vdy + pdy / q.r);
        const float p1 = q.p - h * (a.gamma * q.p * (udx + vdy) + q.u * pdx + q.v * pdy);
        float* F = a.faces;
        // order: var-major (r,u,v,p), face-minor (xl, xr, yl, yr)
        F[0 * plane + c] = r1 - rdx * hdx;  F[1 * plane + c] = r1 + rdx * hdx;  F[2 * plane + c] = r1 - rdy * hdx;  F[3 * plane + c] = r1 + rdy * hdx;
        F[4 * plane + c] = u1 - udx * hdx;  F[5 * plane + c] = u1 + udx * hdx;  F[6 * plane + c] = u1 - udy * hdx;  F[7 * plane + c] = u1 + udy * hdx;
        F[8 * plane + c] = v1 - vdx * hdx;  F[9 * plane + c] = v1 + vdx * hdx;  F[10 * plane + c] = v1 - vdy * hdx; F[11 * plane + c] = v1 + vdy * hdx;
        F[12 * plane + c] = p1 - pdx * hdx; F[13 * plane + c] = p1 + pdx * hdx; F[14 * plane + c] = p1 - pdy * hdx; F[15 * plane + c] = p1 + pdy * hdx;
      }
      grid.sync();
      // ---------------------------------------------------------------- phase B
      for (long long c = t0; c < plane; c += nthreads) {
        const int j = int(c % N), i = int((c / N) % N);
        const long long base = c - ((long long)i * N + j);
        const long long xe = base + (long long)pwrap(i + 1, N) * N + j, xw = base + (long long)pwrap(i - 1, N) * N + j;
        const long long yn = base + (long long)i * N + pwrap(j + 1, N), ys = base + (long long)i * N + pwrap(j - 1, N);
        const float* F = a.faces;
        // face between cell and its +x neighbour: left state = neighbour's xl, right state = own xr (reference convention)
        const float4 fxp = rusanov(F[0 * plane + xe], F[1 * plane + c], F[4 * plane + xe], F[5 * plane + c], F[8 * plane + xe],
                                   F[9 * plane + c], F[12 * plane + xe], F[13 * plane + c], a.gamma);
        const float4 fxm = rusanov(F[0 * plane + c], F[1 * plane + xw], F[4 * plane + c], F[5 * plane + xw], F[8 * plane + c],
                                   F[9 * plane + xw], F[12 * plane + c], F[13 * plane + xw], a.gamma);
        const float4 fyp = rusanov(F[2 * plane + yn], F[3 * plane + c], F[10 * plane + yn], F[11 * plane + c], F[6 * plane + yn],
                                   F[7 * plane + c], F[14 * plane + yn], F[15 * plane + c], a.gamma);
        const float4 fym = rusanov(F[2 * plane + c], F[3 * plane + ys], F[10 * plane + c], F[11 * plane + ys], F[6 * plane + c],
                                   F[7 * plane + ys], F[14 * plane + c], F[15 * plane + ys], a.gamma);
        const float k = a.dt * a.dx;
        a.cons[c] += k * (-fxp.x + fxm.x - fyp.x + fym.x);
        a.cons[plane + c] += k * (-fxp.y + fxm.y - fyp.z + fym.z);
        a.cons[2 * plane + c] += k * (-fxp.z + fxm.z - fyp.y + fym.y);
        a.cons[3 * plane + c] += k * (-fxp.w + fxm.w - fyp.w + fym.w);
      }
      grid.sync();
    }
  }
}

}  // namespace pnm

extern "C" {

int pnm_kh_simulate(float* cons, float* faces, const float* w, float* snap_rho, float* snap_vel, float* snap_p, int B, int N,
                    int nfreq, int snapshots, int steps_per_snapshot, float gamma, float dx, float dt, float sigma, void* stream) {
  if (B <= 0 || N <= 0 || snapshots <= 0) return 0;
  pnm::KhArgs a;
  a.cons = cons; a.faces = faces; a.w = w; a.snap_rho = snap_rho; a.snap_vel = snap_vel; a.snap_p = snap_p;
  a.B = B; a.N = N; a.nfreq = nfreq; a.snapshots = snapshots; a.steps_per_snapshot = steps_per_snapshot;
  a.gamma = gamma; a.dx = dx; a.dt = dt; a.vol = dx * dx; a.sigma = sigma;
  int dev = 0, sms = 0, per_sm = 0;
  cudaGetDevice(&dev);
  cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev);
  cudaOccupancyMaxActiveBlocksPerMultiprocessor(&per_sm, pnm::kh_simulate_kernel, 256, 0);
  if (per_sm < 1) return -2;
  const long long cells = (long long)B * N * N;
  long long blocks = (long long)sms * per_sm;
  blocks = blocks < (cells + 255) / 256 ? blocks : (cells + 255) / 256;
  void* params[] = {&a};
  return (int)cudaLaunchCooperativeKernel((void*)pnm::kh_simulate_kernel, dim3((unsigned)blocks), dim3(256), params, 0,
                                          (cudaStream_t)stream);
}

}  // extern "C"
