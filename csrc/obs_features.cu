// Per-observation metadata features of the observation tokenizer (local solar time, time offset, position in the
// column, viewing geometry) as sines / cosines, one row of 28 or 30 floats per observation.
//
//   basic (28):   [sin, cos](k lst), k = 1, 2 | dt, dt^2 | [sin, cos](k h), k = 1..4 | [sin, cos](k p), k = 1..4 |
//                 s, s^2 | cos z_sat, cos^2 z_sat | cos z_sun, sin z_sun
//   extended (30): [sin, cos](k lst), k = 1, 2 | dt, dt^2 | sin dt, cos dt | sin lat, cos lat | then for conventional
//                 observations (finite height) [sin, cos](k h), k = 1..5, [sin, cos](k p), k = 1..5, and for satellite
//                 observations [sin, cos](k s), k = 1..3, [sin, cos](k z_sat), k = 1..4, [sin, cos](k z_sun), k = 1..3
//
// with lst = 2 pi (UTC hours + lon / 15 mod 24) / 24, dt in days relative to the analysis time, h = 2 pi clamp(height /
// 60 km), p = 2 pi clamp(pressure / 1100 hPa), s = scan angle / 50 (basic) or 2 pi scan / 50 (extended), z_sat = 2 pi
// zenith / 90, z_sun = 2 pi zenith / 180 (extended).  A NaN input contributes zeros in the basic scheme.
//
// A block handles 256 observations: each thread computes one row into shared memory, then the block writes the
// 256 x F tile with consecutive threads on consecutive addresses.
#include <cuda_runtime.h>
#include <math.h>
#include <stdint.h>

#include "pnm_api.h"

namespace pnm {

constexpr int kObsBlock = 256;
constexpr float kTwoPi = 6.283185307179586f;
constexpr float kDeg2Rad = 0.017453292519943295f;

template <int N>
__device__ __forceinline__ void fourier_row(float* row, float angle, bool valid) {
#pragma unroll
  for (int k = 1; k <= N; ++k) {
    float s, c;
    __sincosf(angle * float(k), &s, &c);   // arguments stay below 32 rad: the fast path is accurate to ~1e-5 there
    row[k - 1] = valid ? s : 0.f;
    row[N + k - 1] = valid ? c : 0.f;
  }
}

__device__ __forceinline__ float clamp01(float x) { return fminf(fmaxf(x, 0.f), 1.f); }

template <bool EXT>
__global__ void __launch_bounds__(kObsBlock)
obs_metadata_kernel(const float* __restrict__ lat, const float* __restrict__ lon, const long long* __restrict__ time_ns,
                    const long long* __restrict__ target_s, const float* __restrict__ height,
                    const float* __restrict__ pressure, const float* __restrict__ scan, const float* __restrict__ sat_zen,
                    const float* __restrict__ sol_zen, float* __restrict__ out, long long n) {
  constexpr int F = EXT ? 30 : 28;
  __shared__ float tile[kObsBlock][F + 1];
  const long long first = (long long)blockIdx.x * kObsBlock;
  const long long i = first + threadIdx.x;
  if (i < n) {
    float* row = tile[threadIdx.x];
    const long long t = time_ns[i];
    const long long sod = (t / 1000000000LL) % 86400LL;
    float lst = fmodf(float(sod) / 3600.f + lon[i] / 15.f, 24.f);
    if (lst < 0.f) lst += 24.f;
    fourier_row<2>(row, lst / 24.f * kTwoPi, true);
    const float dt = float(t - target_s[i] * 1000000000LL) * 1e-9f / 86400.f;
    row[4] = dt;
    row[5] = dt * dt;
    const float h = height[i], p = pressure[i], sc = scan[i], zs = sat_zen[i], zo = sol_zen[i];
    if (!EXT) {
      const bool hv = !isnan(h), pv = !isnan(p), sv = !isnan(sc), zv = !isnan(zs), ov = !isnan(zo);
      fourier_row<4>(row + 6, hv ? clamp01(h / 60000.f) * kTwoPi : 0.f, hv);
      fourier_row<4>(row + 14, pv ? clamp01(p / 1100.f) * kTwoPi : 0.f, pv);
      const float s = sv ? sc / 50.f : 0.f;
      row[22] = s;
      row[23] = s * s;
      const float cz = zv ? cosf(zs * kDeg2Rad) : 0.f;
      row[24] = cz;
      row[25] = cz * cz;
      float so = 0.f, co = 0.f;
      if (ov) sincosf(zo * kDeg2Rad, &so, &co);
      row[26] = co;
      row[27] = so;
    } else {
      fourier_row<1>(row + 6, dt, true);
      float sl, cl;
      sincosf(lat[i] * kDeg2Rad, &sl, &cl);
      row[8] = sl;
      row[9] = cl;
      if (!isnan(h)) {
        fourier_row<5>(row + 10, clamp01(h / 60000.f) * kTwoPi, true);
        fourier_row<5>(row + 20, clamp01(p / 1100.f) * kTwoPi, true);
      } else {
        fourier_row<3>(row + 10, sc / 50.f * kTwoPi, true);
        fourier_row<4>(row + 16, zs / 90.f * kTwoPi, true);
        fourier_row<3>(row + 24, zo / 180.f * kTwoPi, true);
      }
    }
  }
  __syncthreads();
  const long long rows = (n - first < kObsBlock) ? (n - first) : kObsBlock;
  for (long long e = threadIdx.x; e < rows * F; e += kObsBlock) out[first * F + e] = tile[e / F][e % F];
}

}  // namespace pnm

extern "C" int pnm_obs_metadata(const float* lat, const float* lon, const long long* time_ns, const long long* target_s,
                                const float* height, const float* pressure, const float* scan, const float* sat_zen,
                                const float* sol_zen, float* out, long long n, int extended, void* stream) {
  if (n <= 0) return 0;
  const unsigned blocks = unsigned((n + pnm::kObsBlock - 1) / pnm::kObsBlock);
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  if (extended) {
    if (lat == nullptr) return 1;
    pnm::obs_metadata_kernel<true><<<blocks, pnm::kObsBlock, 0, s>>>(lat, lon, time_ns, target_s, height, pressure, scan,
                                                                    sat_zen, sol_zen, out, n);
  } else {
    pnm::obs_metadata_kernel<false><<<blocks, pnm::kObsBlock, 0, s>>>(lat, lon, time_ns, target_s, height, pressure, scan,
                                                                     sat_zen, sol_zen, out, n);
  }
  return cudaGetLastError() == cudaSuccess ? 0 : 2;
}
