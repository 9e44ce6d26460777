// Mesh gradient reconstructions: weighted least squares over ragged neighbourhoods and
// Green-Gauss over simplex cells.  One thread per entity / cell; values are [n, C] fp32.
//
// LSQ: g_i = M_i^{-1} sum_j w_ij r_ij (v_j - v_i),  M_i = sum_j w_ij r_ij r_ij^T,  w = |r|^-p.
// The transposed pass (gradient with respect to the values) scatters with atomics.
#include <cuda_runtime.h>
#include <stdint.h>

#include "pnm_api.h"

namespace pnm {

template <int D>
__device__ __forceinline__ bool invert_sym(const float* m, float* inv) {
  if (D == 1) {
    if (fabsf(m[0]) < 1e-30f) return false;
    inv[0] = 1.f / m[0];
    return true;
  }
  if (D == 2) {
    const float det = m[0] * m[3] - m[1] * m[2];
    if (fabsf(det) < 1e-30f) return false;
    const float r = 1.f / det;
    inv[0] = m[3] * r; inv[1] = -m[1] * r; inv[2] = -m[2] * r; inv[3] = m[0] * r;
    return true;
  }
  const float c00 = m[4] * m[8] - m[5] * m[7], c01 = m[5] * m[6] - m[3] * m[8], c02 = m[3] * m[7] - m[4] * m[6];
  const float det = m[0] * c00 + m[1] * c01 + m[2] * c02;
  if (fabsf(det) < 1e-30f) return false;
  const float r = 1.f / det;
  inv[0] = c00 * r; inv[1] = (m[2] * m[7] - m[1] * m[8]) * r; inv[2] = (m[1] * m[5] - m[2] * m[4]) * r;
  inv[3] = c01 * r; inv[4] = (m[0] * m[8] - m[2] * m[6]) * r; inv[5] = (m[2] * m[3] - m[0] * m[5]) * r;
  inv[6] = c02 * r; inv[7] = (m[1] * m[6] - m[0] * m[7]) * r; inv[8] = (m[0] * m[4] - m[1] * m[3]) * r;
  return true;
}

template <int D>
__device__ __forceinline__ bool lsq_setup(const float* __restrict__ pts, const long long* __restrict__ offs,
                                          const long long* __restrict__ nbr, long long i, float half_power, float eps,
                                          int min_neighbors, float* inv, long long& lo, long long& hi) {
  lo = offs[i];
  hi = offs[i + 1];
  if (hi - lo < min_neighbors || hi == lo) return false;
  float m[D * D];
#pragma unroll
  for (int k = 0; k < D * D; ++k) m[k] = 0.f;
  for (long long e = lo; e < hi; ++e) {
    const long long j = nbr[e];
    float r[D], d2 = 0.f;
#pragma unroll
    for (int a = 0; a < D; ++a) { r[a] = pts[j * D + a] - pts[i * D + a]; d2 += r[a] * r[a]; }
    const float w = __powf(fmaxf(d2, eps), -half_power);
#pragma unroll
    for (int a = 0; a < D; ++a)
#pragma unroll
      for (int b = 0; b < D; ++b) m[a * D + b] += w * r[a] * r[b];
  }
  return invert_sym<D>(m, inv);
}

// out: [n, D, C]
template <int D>
__global__ void lsq_gradient_fwd_kernel(const float* __restrict__ pts, const float* __restrict__ vals,
                                        const long long* __restrict__ offs, const long long* __restrict__ nbr,
                                        float* __restrict__ out, long long n, int C, float half_power, float eps,
                                        int min_neighbors) {
  const long long i = blockIdx.x * (long long)blockDim.x + threadIdx.x;
  if (i >= n) return;
  float inv[D * D];
  long long lo, hi;
  const bool ok = lsq_setup<D>(pts, offs, nbr, i, half_power, eps, min_neighbors, inv, lo, hi);
  for (int c = 0; c < C; ++c) {
    float rhs[D];
#pragma unroll
    for (int a = 0; a < D; ++a) rhs[a] = 0.f;
    if (ok) {
      const float vi = vals[i * C + c];
      for (long long e = lo; e < hi; ++e) {
        const long long j = nbr[e];
        float r[D], d2 = 0.f;
#pragma unroll
        for (int a = 0; a < D; ++a) { r[a] = pts[j * D + a] - pts[i * D + a]; d2 += r[a] * r[a]; }
        const float w = __powf(fmaxf(d2, eps), -half_power) * (vals[j * C + c] - vi);
#pragma unroll
        for (int a = 0; a < D; ++a) rhs[a] += w * r[a];
      }
    }
#pragma unroll
    for (int a = 0; a < D; ++a) {
      float g = 0.f;
#pragma unroll
      for (int b = 0; b < D; ++b) g += inv[a * D + b] * rhs[b];
      out[(i * D + a) * C + c] = ok ? g : 0.f;
    }
  }
}

// dvals[j] += w r . (M^-1 gout_i); dvals[i] -= the same (dvals zero-initialised by the caller)
template <int D>
__global__ void lsq_gradient_bwd_values_kernel(const float* __restrict__ pts, const float* __restrict__ gout,
                                               const long long* __restrict__ offs, const long long* __restrict__ nbr,
                                               float* __restrict__ dvals, long long n, int C, float half_power,
                                               float eps, int min_neighbors) {
  const long long i = blockIdx.x * (long long)blockDim.x + threadIdx.x;
  if (i >= n) return;
  float inv[D * D];
  long long lo, hi;
  if (!lsq_setup<D>(pts, offs, nbr, i, half_power, eps, min_neighbors, inv, lo, hi)) return;
  for (int c = 0; c < C; ++c) {
    float q[D];  // M^-T gout = M^-1 gout (symmetric)
#pragma unroll
    for (int a = 0; a < D; ++a) {
      q[a] = 0.f;
#pragma unroll
      for (int b = 0; b < D; ++b) q[a] += inv[a * D + b] * gout[(i * D + b) * C + c];
    }
    float self = 0.f;
    for (long long e = lo; e < hi; ++e) {
      const long long j = nbr[e];
      float r[D], d2 = 0.f, dot = 0.f;
#pragma unroll
      for (int a = 0; a < D; ++a) { r[a] = pts[j * D + a] - pts[i * D + a]; d2 += r[a] * r[a]; dot += r[a] * q[a]; }
      const float t = __powf(fmaxf(d2, eps), -half_power) * dot;
      atomicAdd(&dvals[j * C + c], t);
      self += t;
    }
    atomicAdd(&dvals[i * C + c], -self);
  }
}

// Green-Gauss coefficients per cell face: coeff[cell, face, D] = outward area normal / cell volume.
template <int D>
__global__ void green_gauss_coeff_kernel(const float* __restrict__ pts, const long long* __restrict__ cells,
                                         float* __restrict__ coeff, long long n_cells) {
  constexpr int F = D + 1;
  const long long c = blockIdx.x * (long long)blockDim.x + threadIdx.x;
  if (c >= n_cells) return;
  float p[F][D], cen[D];
#pragma unroll
  for (int a = 0; a < D; ++a) cen[a] = 0.f;
#pragma unroll
  for (int v = 0; v < F; ++v)
#pragma unroll
    for (int a = 0; a < D; ++a) { p[v][a] = pts[cells[c * F + v] * D + a]; cen[a] += p[v][a] / F; }
  float vol;
  if (D == 2) {
    vol = 0.5f * fabsf((p[1][0] - p[0][0]) * (p[2][1] - p[0][1]) - (p[1][1] - p[0][1]) * (p[2][0] - p[0][0]));
  } else {
    const float a0 = p[1][0] - p[0][0], a1 = p[1][1] - p[0][1], a2 = p[1][2 % D] - p[0][2 % D];
    const float b0 = p[2][0] - p[0][0], b1 = p[2][1] - p[0][1], b2 = p[2][2 % D] - p[0][2 % D];
    const float c0 = p[F - 1][0] - p[0][0], c1 = p[F - 1][1] - p[0][1], c2 = p[F - 1][2 % D] - p[0][2 % D];
    vol = fabsf(a0 * (b1 * c2 - b2 * c1) + a1 * (b2 * c0 - b0 * c2) + a2 * (b0 * c1 - b1 * c0)) / 6.f;
  }
  vol = fmaxf(vol, 1e-12f);
#pragma unroll
  for (int f = 0; f < F; ++f) {
    int loc[D];
    int k = 0;
#pragma unroll
    for (int v = 0; v < F; ++v) if (v != f) { if (k < D) loc[k] = v; ++k; }
    float nrm[D], fc[D];
    if (D == 2) {
      const float e0 = p[loc[1]][0] - p[loc[0]][0], e1 = p[loc[1]][1] - p[loc[0]][1];
      nrm[0] = e1; nrm[1] = -e0;
      fc[0] = 0.5f * (p[loc[0]][0] + p[loc[1]][0]); fc[1] = 0.5f * (p[loc[0]][1] + p[loc[1]][1]);
    } else {
      const float u0 = p[loc[1]][0] - p[loc[0]][0], u1 = p[loc[1]][1] - p[loc[0]][1], u2 = p[loc[1]][2 % D] - p[loc[0]][2 % D];
      const float w0 = p[loc[D - 1]][0] - p[loc[0]][0], w1 = p[loc[D - 1]][1] - p[loc[0]][1], w2 = p[loc[D - 1]][2 % D] - p[loc[0]][2 % D];
      nrm[0] = 0.5f * (u1 * w2 - u2 * w1); nrm[1] = 0.5f * (u2 * w0 - u0 * w2); nrm[2 % D] = 0.5f * (u0 * w1 - u1 * w0);
#pragma unroll
      for (int a = 0; a < D; ++a) fc[a] = (p[loc[0]][a] + p[loc[1]][a] + p[loc[D - 1]][a]) / 3.f;
    }
    float dot = 0.f;
#pragma unroll
    for (int a = 0; a < D; ++a) dot += nrm[a] * (fc[a] - cen[a]);
    const float sgn = dot >= 0.f ? 1.f : -1.f;
#pragma unroll
    for (int a = 0; a < D; ++a) coeff[(c * F + f) * D + a] = sgn * nrm[a] / vol;
  }
}

// grad[cell, D, C] = sum_f coeff[cell,f,:] * face_value;  face value = mean with the neighbour (own value on boundaries)
template <int D>
__global__ void green_gauss_apply_kernel(const float* __restrict__ coeff, const long long* __restrict__ nbrs,
                                         const float* __restrict__ vals, float* __restrict__ out, long long n_cells, int C) {
  constexpr int F = D + 1;
  const long long idx = blockIdx.x * (long long)blockDim.x + threadIdx.x;
  if (idx >= n_cells * C) return;
  const long long c = idx / C;
  const int k = int(idx % C);
  float g[D];
#pragma unroll
  for (int a = 0; a < D; ++a) g[a] = 0.f;
  const float own = vals[c * C + k];
#pragma unroll
  for (int f = 0; f < F; ++f) {
    const long long nb = nbrs[c * F + f];
    const float fv = nb >= 0 ? 0.5f * (own + vals[nb * C + k]) : own;
#pragma unroll
    for (int a = 0; a < D; ++a) g[a] += coeff[(c * F + f) * D + a] * fv;
  }
#pragma unroll
  for (int a = 0; a < D; ++a) out[(c * D + a) * C + k] = g[a];
}

template <int D>
__global__ void green_gauss_bwd_values_kernel(const float* __restrict__ coeff, const long long* __restrict__ nbrs,
                                              const float* __restrict__ gout, float* __restrict__ dvals, long long n_cells, int C) {
  constexpr int F = D + 1;
  const long long idx = blockIdx.x * (long long)blockDim.x + threadIdx.x;
  if (idx >= n_cells * C) return;
  const long long c = idx / C;
  const int k = int(idx % C);
  float self = 0.f;
#pragma unroll
  for (int f = 0; f < F; ++f) {
    float t = 0.f;
#pragma unroll
    for (int a = 0; a < D; ++a) t += coeff[(c * F + f) * D + a] * gout[(c * D + a) * C + k];
    const long long nb = nbrs[c * F + f];
    if (nb >= 0) { self += 0.5f * t; atomicAdd(&dvals[nb * C + k], 0.5f * t); }
    else self += t;
  }
  atomicAdd(&dvals[c * C + k], self);
}

}  // namespace pnm

extern "C" {

#define PNM_DISPATCH_D(D_, CALL)          \
  switch (D_) {                           \
    case 1: { constexpr int DD = 1; CALL; } break; \
    case 2: { constexpr int DD = 2; CALL; } break; \
    case 3: { constexpr int DD = 3; CALL; } break; \
    default: return -1;                   \
  }

int pnm_mesh_lsq_gradient(const float* pts, const float* vals, const long long* offs, const long long* nbr, float* out,
                          long long n, int D, int C, float weight_power, float eps, int min_neighbors, int backward,
                          void* stream) {
  if (n <= 0) return 0;
  const int threads = 128;
  const unsigned blocks = (unsigned)((n + threads - 1) / threads);
  cudaStream_t st = (cudaStream_t)stream;
  const float hp = 0.5f * weight_power;
  if (!backward) {
    PNM_DISPATCH_D(D, (pnm::lsq_gradient_fwd_kernel<DD><<<blocks, threads, 0, st>>>(pts, vals, offs, nbr, out, n, C, hp, eps, min_neighbors)))
  } else {
    PNM_DISPATCH_D(D, (pnm::lsq_gradient_bwd_values_kernel<DD><<<blocks, threads, 0, st>>>(pts, vals, offs, nbr, out, n, C, hp, eps, min_neighbors)))
  }
  return (int)cudaGetLastError();
}

// mode 0: coefficients (out = coeff[n_cells, D+1, D]); 1: apply (a = coeff, out = grad); 2: transposed apply (out = dvals)
int pnm_mesh_green_gauss(const float* a, const long long* idx, const float* vals, float* out, long long n_cells, int D,
                         int C, int mode, void* stream) {
  if (n_cells <= 0) return 0;
  if (D != 2 && D != 3) return -1;
  const int threads = 128;
  cudaStream_t st = (cudaStream_t)stream;
  const long long work = mode == 0 ? n_cells : n_cells * C;
  const unsigned blocks = (unsigned)((work + threads - 1) / threads);
  if (D == 2) {
    if (mode == 0) pnm::green_gauss_coeff_kernel<2><<<blocks, threads, 0, st>>>(a, idx, out, n_cells);
    else if (mode == 1) pnm::green_gauss_apply_kernel<2><<<blocks, threads, 0, st>>>(a, idx, vals, out, n_cells, C);
    else pnm::green_gauss_bwd_values_kernel<2><<<blocks, threads, 0, st>>>(a, idx, vals, out, n_cells, C);
  } else {
    if (mode == 0) pnm::green_gauss_coeff_kernel<3><<<blocks, threads, 0, st>>>(a, idx, out, n_cells);
    else if (mode == 1) pnm::green_gauss_apply_kernel<3><<<blocks, threads, 0, st>>>(a, idx, vals, out, n_cells, C);
    else pnm::green_gauss_bwd_values_kernel<3><<<blocks, threads, 0, st>>>(a, idx, vals, out, n_cells, C);
  }
  return (int)cudaGetLastError();
}

}  // extern "C"
