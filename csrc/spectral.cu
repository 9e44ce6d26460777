// Mode-truncated spectral contraction of Fourier neural operators, fused with the corner gather / scatter.
//
//   out[p, q, m] (+)= sum_r  A[p, r, m] * B[r, q, m]        (complex64, optional conjugation of A and / or B)
//
// `m` runs over a block of retained Fourier modes given as up to four mode dimensions with individual strides per tensor,
// so A and `out` can be corners of full spectra (no slice copy, no zero-padded scatter afterwards) while B is the dense
// weight tensor.  The same kernel gives the forward product (A = x_hat corner, B = weights), the input gradient
// (A = dy_hat corner, B = conj(weights) with its channel strides swapped) and the weight gradient (A = conj(x_hat) with
// batch as the contracted index, B = dy_hat).
//
// One thread owns one mode and a tile of four q: every A value it loads is reused four times, the mode index is the fastest
// thread index so that spectra and weights are read along their contiguous last mode dimension.
#include <cuda_runtime.h>
#include <stdint.h>

#include "pnm_api.h"

namespace pnm {

struct SpecDesc {
  int nd;                 // number of mode dimensions (1..4)
  int shape[4];           // extents, slowest first
  long long sa[4], sb[4], so[4];   // element (complex) strides of the mode dimensions
  long long sa_p, sa_r, sb_r, sb_q, so_p, so_q;
  int P, Q, R;
  int conj_a, conj_b, accumulate;
  long long n_modes;
};

__global__ void __launch_bounds__(256) spectral_contract_kernel(const float2* __restrict__ A, const float2* __restrict__ B,
                                                                float2* __restrict__ out, const SpecDesc d) {
  const long long m = (long long)blockIdx.x * blockDim.x + threadIdx.x;
  if (m >= d.n_modes) return;
  const int q0 = blockIdx.y * 4, p = blockIdx.z;
  long long oa = 0, ob = 0, oo = 0, rem = m;
  for (int k = d.nd - 1; k >= 0; --k) {
    const int i = int(rem % d.shape[k]);
    rem /= d.shape[k];
    oa += i * d.sa[k];
    ob += i * d.sb[k];
    oo += i * d.so[k];
  }
  const float2* a = A + oa + p * d.sa_p;
  const float2* b = B + ob + (long long)q0 * d.sb_q;
  float2 acc[4] = {{0.f, 0.f}, {0.f, 0.f}, {0.f, 0.f}, {0.f, 0.f}};
  const float sa = d.conj_a ? -1.f : 1.f, sb = d.conj_b ? -1.f : 1.f;
  const int nq = min(4, d.Q - q0);
  for (int r = 0; r < d.R; ++r) {
    float2 av = a[r * d.sa_r];
    av.y *= sa;
#pragma unroll
    for (int t = 0; t < 4; ++t) {
      if (t < nq) {
        float2 bv = b[r * d.sb_r + t * d.sb_q];
        bv.y *= sb;
        acc[t].x = fmaf(av.x, bv.x, fmaf(-av.y, bv.y, acc[t].x));
        acc[t].y = fmaf(av.x, bv.y, fmaf(av.y, bv.x, acc[t].y));
      }
    }
  }
  float2* o = out + oo + p * d.so_p + (long long)q0 * d.so_q;
  for (int t = 0; t < nq; ++t) {
    float2 v = acc[t];
    if (d.accumulate) {
      const float2 old = o[t * d.so_q];
      v.x += old.x;
      v.y += old.y;
    }
    o[t * d.so_q] = v;
  }
}

}  // namespace pnm

extern "C" int pnm_spectral_contract(const void* A, const void* B, void* out, int nd, const int* shape, const long long* sa,
                                     const long long* sb, const long long* so, const long long* chan_strides, int P, int Q, int R,
                                     int conj_a, int conj_b, int accumulate, void* stream) {
  if (!A || !B || !out || nd < 1 || nd > 4 || P <= 0 || Q <= 0 || R <= 0) return -1;
  pnm::SpecDesc d{};
  d.nd = nd;
  d.n_modes = 1;
  for (int k = 0; k < nd; ++k) {
    if (shape[k] <= 0) return -1;
    d.shape[k] = shape[k];
    d.sa[k] = sa[k];
    d.sb[k] = sb[k];
    d.so[k] = so[k];
    d.n_modes *= shape[k];
  }
  d.sa_p = chan_strides[0]; d.sa_r = chan_strides[1]; d.sb_r = chan_strides[2];
  d.sb_q = chan_strides[3]; d.so_p = chan_strides[4]; d.so_q = chan_strides[5];
  d.P = P; d.Q = Q; d.R = R;
  d.conj_a = conj_a; d.conj_b = conj_b; d.accumulate = accumulate;
  if (P > 65535 || (Q + 3) / 4 > 65535) return -1;
  dim3 grid((unsigned)((d.n_modes + 255) / 256), (unsigned)((Q + 3) / 4), (unsigned)P);
  pnm::spectral_contract_kernel<<<grid, 256, 0, reinterpret_cast<cudaStream_t>(stream)>>>(
      reinterpret_cast<const float2*>(A), reinterpret_cast<const float2*>(B), reinterpret_cast<float2*>(out), d);
  return cudaGetLastError() == cudaSuccess ? 0 : -4;
}
