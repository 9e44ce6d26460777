// 2 x 2 box resampling of channels-last bf16 images: the [1, 1] resample filter of the diffusion U-Nets.
//
//   down: y[n, h, w, c] = scale * sum_{i, j < 2} x[n, 2 h + i, 2 w + j, c]        (scale 1/4: the mean)
//   up  : y[n, h, w, c] = scale * x[n, h / 2, w / 2, c]                            (scale 1: replication)
//
// Each is the adjoint of the other up to the scale, so the two kernels also serve as each other's backward
// (d down = up with scale 1/4, d up = down with scale 1).  One pass over the larger tensor at 16 bytes per access;
// the grid is sized from the number of vectors, threads walk the channel vectors of consecutive output pixels.
#include <cuda_bf16.h>
#include <cuda_runtime.h>
#include <stdint.h>

#include "common.cuh"
#include "pnm_api.h"

namespace pnm {

__device__ __forceinline__ void rs_unpack(const uint4& u, float* f) {
  float2 a;
  a = unpack_bf16x2(u.x); f[0] = a.x; f[1] = a.y;
  a = unpack_bf16x2(u.y); f[2] = a.x; f[3] = a.y;
  a = unpack_bf16x2(u.z); f[4] = a.x; f[5] = a.y;
  a = unpack_bf16x2(u.w); f[6] = a.x; f[7] = a.y;
}
__device__ __forceinline__ uint4 rs_pack(const float* f) {
  uint4 u;
  u.x = pack_bf16x2(f[0], f[1]); u.y = pack_bf16x2(f[2], f[3]);
  u.z = pack_bf16x2(f[4], f[5]); u.w = pack_bf16x2(f[6], f[7]);
  return u;
}

// ho, wo: output extent (input is 2 ho x 2 wo); cv = C / 8 vectors per pixel
__global__ void __launch_bounds__(256)
resample_down2x_kernel(const uint4* __restrict__ x, uint4* __restrict__ y, long long total, int ho, int wo, int cv, float scale) {
  for (long long i = blockIdx.x * (long long)blockDim.x + threadIdx.x; i < total; i += (long long)gridDim.x * blockDim.x) {
    const int v = int(i % cv);
    long long p = i / cv;
    const int w = int(p % wo);
    p /= wo;
    const int h = int(p % ho);
    const long long n = p / ho;
    const long long row = 2LL * wo * cv;
    const uint4* src = x + ((n * 2 * ho + 2 * h) * 2LL * wo + 2 * w) * cv + v;
    float a[8], b[8], acc[8];
    rs_unpack(__ldg(src), a);
    rs_unpack(__ldg(src + cv), b);
#pragma unroll
    for (int k = 0; k < 8; ++k) acc[k] = a[k] + b[k];
    rs_unpack(__ldg(src + row), a);
    rs_unpack(__ldg(src + row + cv), b);
#pragma unroll
    for (int k = 0; k < 8; ++k) acc[k] = (acc[k] + a[k] + b[k]) * scale;
    y[i] = rs_pack(acc);
  }
}

// hi, wi: input extent (output is 2 hi x 2 wi); one thread reads a vector and writes its four copies
__global__ void __launch_bounds__(256)
resample_up2x_kernel(const uint4* __restrict__ x, uint4* __restrict__ y, long long total, int hi, int wi, int cv, float scale) {
  for (long long i = blockIdx.x * (long long)blockDim.x + threadIdx.x; i < total; i += (long long)gridDim.x * blockDim.x) {
    const int v = int(i % cv);
    long long p = i / cv;
    const int w = int(p % wi);
    p /= wi;
    const int h = int(p % hi);
    const long long n = p / hi;
    uint4 u = __ldg(x + i);
    if (scale != 1.f) {
      float f[8];
      rs_unpack(u, f);
#pragma unroll
      for (int k = 0; k < 8; ++k) f[k] *= scale;
      u = rs_pack(f);
    }
    const long long row = 2LL * wi * cv;
    uint4* dst = y + ((n * 2 * hi + 2 * h) * 2LL * wi + 2 * w) * cv + v;
    dst[0] = u;
    dst[cv] = u;
    dst[row] = u;
    dst[row + cv] = u;
  }
}

}  // namespace pnm

extern "C" {

// x: [n, h, w, c] bf16 channels-last.  mode 0: y = [n, h/2, w/2, c] (h, w even); mode 1: y = [n, 2h, 2w, c].  c % 8 == 0.
int pnm_resample2x_nhwc(const void* x, void* y, int n, int h, int w, int c, int mode, float scale, void* stream) {
  if (n <= 0 || h <= 0 || w <= 0 || c <= 0 || (c & 7)) return -2;
  if (mode == 0 && ((h | w) & 1)) return -2;
  const int cv = c >> 3;
  cudaStream_t st = (cudaStream_t)stream;
  if (mode == 0) {
    const long long total = (long long)n * (h / 2) * (w / 2) * cv;
    const long long blocks = (total + 255) / 256;
    pnm::resample_down2x_kernel<<<(unsigned)(blocks < 148 * 16 ? blocks : 148 * 16), 256, 0, st>>>((const uint4*)x, (uint4*)y, total,
                                                                                                  h / 2, w / 2, cv, scale);
  } else {
    const long long total = (long long)n * h * w * cv;
    const long long blocks = (total + 255) / 256;
    pnm::resample_up2x_kernel<<<(unsigned)(blocks < 148 * 16 ? blocks : 148 * 16), 256, 0, st>>>((const uint4*)x, (uint4*)y, total, h, w,
                                                                                                cv, scale);
  }
  return cudaGetLastError() == cudaSuccess ? 0 : -3;
}

}  // extern "C"
