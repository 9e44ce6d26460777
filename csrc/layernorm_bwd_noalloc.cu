// Allocation-free LayerNorm backward: same kernels as pnm_layernorm_bwd(), scratch in a
// static device array.  See layernorm_bwd_noalloc.h for who needs this and for the rules.
#include <stdio.h>

#include "norm.cuh"
#include "layernorm_bwd_noalloc.h"

namespace {

constexpr int kMaxBlocks = 160;
constexpr int kMaxC = 1024;
constexpr int kMaxDevices = 64;

// Partial dgamma / dbeta rows, [kMaxBlocks][2][C].  In host code this name is only a handle
// for cudaGetSymbolAddress(); the kernels receive the resolved device pointer.
static __device__ __align__(256) float g_noalloc_scratch[kMaxBlocks * 2 * kMaxC];

float* g_scratch_ptr[kMaxDevices] = {nullptr};

// Resolve (once per device, with that device current) the device address of the scratch.
float* scratch_for_current_device() {
  int dev = -1;
  if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= kMaxDevices) return nullptr;
  if (!g_scratch_ptr[dev]) {
    float* p = nullptr;
    if (cudaGetSymbolAddress(reinterpret_cast<void**>(&p), g_noalloc_scratch) != cudaSuccess) return nullptr;
    g_scratch_ptr[dev] = p;
  }
  return g_scratch_ptr[dev];
}

template <int VEC>
int launch(const void* dy, const void* x, const float* gamma, const float* mean, const float* rstd,
           const void* dres, void* dx, float* scratch, long long M, int C, int grid, cudaStream_t st) {
  pnm::layernorm_bwd_kernel<VEC><<<grid, pnm::kLnWarps * 32, 0, st>>>(
      static_cast<const __nv_bfloat16*>(dy), static_cast<const __nv_bfloat16*>(x), gamma, mean, rstd,
      static_cast<const __nv_bfloat16*>(dres), static_cast<__nv_bfloat16*>(dx), scratch, M, C);
  return cudaGetLastError() == cudaSuccess ? 0 : PNM_NOALLOC_E_LAUNCH;
}

}  // namespace

extern "C" int pnm_layernorm_bwd_noalloc(const void* dy, const void* x, const float* gamma, const float* mean,
                                         const float* rstd, const void* dres, void* dx, float* dgamma,
                                         float* dbeta, long long M, int C, void* stream) {
  if (M < 1 || C < 8 || C > kMaxC || (C % 8) != 0) {
    fprintf(stderr,
            "pnm_layernorm_bwd_noalloc: unsupported size M=%lld C=%d (need M >= 1, C a multiple of 8, C <= %d)\n", M,
            C, kMaxC);
    return PNM_NOALLOC_E_SIZE;
  }
  float* scratch = scratch_for_current_device();
  if (!scratch) {
    fprintf(stderr, "pnm_layernorm_bwd_noalloc: could not resolve the scratch array on the current device\n");
    return PNM_NOALLOC_E_SETUP;
  }
  long long want = (M + pnm::kLnWarps - 1) / pnm::kLnWarps;
  const int grid = static_cast<int>(want < kMaxBlocks ? want : kMaxBlocks);
  cudaStream_t st = reinterpret_cast<cudaStream_t>(stream);
  int rc;
  switch (pnm::ln_vec_for(C)) {
    case 1: rc = launch<1>(dy, x, gamma, mean, rstd, dres, dx, scratch, M, C, grid, st); break;
    case 2: rc = launch<2>(dy, x, gamma, mean, rstd, dres, dx, scratch, M, C, grid, st); break;
    case 3: rc = launch<3>(dy, x, gamma, mean, rstd, dres, dx, scratch, M, C, grid, st); break;
    default: rc = launch<4>(dy, x, gamma, mean, rstd, dres, dx, scratch, M, C, grid, st); break;
  }
  if (rc) return rc;
  // every scratch row [0, grid) was fully written above; the fold reads exactly those rows
  pnm::layernorm_bwd_finalize_kernel<<<(2 * C + 31) / 32, 32 * pnm::kLnFoldRows, 0, st>>>(scratch, grid, C, dgamma, dbeta);
  return cudaGetLastError() == cudaSuccess ? 0 : PNM_NOALLOC_E_LAUNCH;
}
