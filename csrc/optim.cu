// Multi-tensor optimizer kernels: one launch updates every parameter of a group.
//
// The host uploads two small tables per step: `entries` (one per tensor: parameter, gradient,
// first and second moment, element count, gradient dtype) and `blocks` (one per CTA: which
// entry and which chunk of it).  Parameters and moments are fp32; gradients fp32 or bf16.
#include <cuda_bf16.h>
#include <cuda_runtime.h>
#include <stdint.h>

#include "pnm_api.h"

namespace pnm {

struct OptEntry {
  float* p;
  const void* g;
  float* m;
  float* v;
  long long n;
  int g_bf16;
  int pad;
};
static_assert(sizeof(OptEntry) == 48, "table layout is shared with the Python side");

constexpr int kOptChunk = 8192;   // elements per CTA
constexpr int kOptThreads = 256;

__device__ __forceinline__ float load_grad(const void* g, long long i, int bf16) {
  return bf16 ? __bfloat162float(reinterpret_cast<const __nv_bfloat16*>(g)[i]) : reinterpret_cast<const float*>(g)[i];
}

// Adam / AdamW.  step_size = lr / (1 - b1^t); inv_bc2_sqrt = 1 / sqrt(1 - b2^t).
__global__ void __launch_bounds__(kOptThreads)
adam_multi_kernel(const OptEntry* __restrict__ entries, const int2* __restrict__ blocks, float lr, float b1, float b2,
                  float eps, float wd, float step_size, float inv_bc2_sqrt, int decoupled, float grad_scale,
                  const float* __restrict__ hyper) {
  if (hyper) {          // {learning rate, step count} kept on the device: the launch can be replayed from a CUDA graph
    lr = hyper[0];
    const float t = hyper[1];
    step_size = lr / (1.f - powf(b1, t));
    inv_bc2_sqrt = rsqrtf(1.f - powf(b2, t));
  }
  const int2 blk = blocks[blockIdx.x];
  const OptEntry e = entries[blk.x];
  const long long lo = (long long)blk.y * kOptChunk;
  const long long hi = min(lo + (long long)kOptChunk, e.n);
  const bool vec = !e.g_bf16 && ((reinterpret_cast<uintptr_t>(e.p) | reinterpret_cast<uintptr_t>(e.g) |
                                  reinterpret_cast<uintptr_t>(e.m) | reinterpret_cast<uintptr_t>(e.v)) & 15) == 0 &&
                   (hi - lo) == kOptChunk;
  if (vec) {
    for (long long i = lo + threadIdx.x * 4; i < hi; i += kOptThreads * 4) {
      float4 p = *reinterpret_cast<float4*>(e.p + i);
      float4 g = *reinterpret_cast<const float4*>(reinterpret_cast<const float*>(e.g) + i);
      float4 m = *reinterpret_cast<float4*>(e.m + i);
      float4 v = *reinterpret_cast<float4*>(e.v + i);
      float* pp = &p.x; float* gp = &g.x; float* mp = &m.x; float* vp = &v.x;
#pragma unroll
      for (int k = 0; k < 4; ++k) {
        float gr = gp[k] * grad_scale;
        if (decoupled) pp[k] *= (1.f - lr * wd); else gr += wd * pp[k];
        mp[k] = b1 * mp[k] + (1.f - b1) * gr;
        vp[k] = b2 * vp[k] + (1.f - b2) * gr * gr;
        pp[k] -= step_size * mp[k] / (sqrtf(vp[k]) * inv_bc2_sqrt + eps);
      }
      *reinterpret_cast<float4*>(e.p + i) = p;
      *reinterpret_cast<float4*>(e.m + i) = m;
      *reinterpret_cast<float4*>(e.v + i) = v;
    }
    return;
  }
  for (long long i = lo + threadIdx.x; i < hi; i += kOptThreads) {
    float p = e.p[i];
    float gr = load_grad(e.g, i, e.g_bf16) * grad_scale;
    if (decoupled) p *= (1.f - lr * wd); else gr += wd * p;
    const float m = b1 * e.m[i] + (1.f - b1) * gr;
    const float v = b2 * e.v[i] + (1.f - b2) * gr * gr;
    e.m[i] = m;
    e.v[i] = v;
    e.p[i] = p - step_size * m / (sqrtf(v) * inv_bc2_sqrt + eps);
  }
}

// Sum of squares of all gradients (for global-norm clipping); one atomicAdd per CTA.
__global__ void __launch_bounds__(kOptThreads)
grad_sqnorm_multi_kernel(const OptEntry* __restrict__ entries, const int2* __restrict__ blocks, float* __restrict__ out) {
  const int2 blk = blocks[blockIdx.x];
  const OptEntry e = entries[blk.x];
  const long long lo = (long long)blk.y * kOptChunk;
  const long long hi = min(lo + (long long)kOptChunk, e.n);
  float acc = 0.f;
  for (long long i = lo + threadIdx.x; i < hi; i += kOptThreads) {
    const float g = load_grad(e.g, i, e.g_bf16);
    acc += g * g;
  }
  for (int o = 16; o; o >>= 1) acc += __shfl_xor_sync(0xffffffffu, acc, o);
  __shared__ float part[kOptThreads / 32];
  if ((threadIdx.x & 31) == 0) part[threadIdx.x >> 5] = acc;
  __syncthreads();
  if (threadIdx.x < kOptThreads / 32) {
    float s = part[threadIdx.x];
    for (int o = kOptThreads / 64; o; o >>= 1) s += __shfl_xor_sync(0xffu, s, o);
    if (threadIdx.x == 0) atomicAdd(out, s);
  }
}

}  // namespace pnm

extern "C" {

int pnm_opt_chunk() { return pnm::kOptChunk; }

int pnm_adam_multi(const void* entries, const void* blocks, int n_blocks, float lr, float b1, float b2, float eps,
                   float wd, float step_size, float inv_bc2_sqrt, int decoupled, float grad_scale, void* stream,
                   const float* hyper) {
  if (n_blocks <= 0) return 0;
  pnm::adam_multi_kernel<<<n_blocks, pnm::kOptThreads, 0, (cudaStream_t)stream>>>(
      reinterpret_cast<const pnm::OptEntry*>(entries), reinterpret_cast<const int2*>(blocks), lr, b1, b2, eps, wd,
      step_size, inv_bc2_sqrt, decoupled, grad_scale, hyper);
  return (int)cudaGetLastError();
}

int pnm_grad_sqnorm_multi(const void* entries, const void* blocks, int n_blocks, float* out, void* stream) {
  if (n_blocks <= 0) return 0;
  pnm::grad_sqnorm_multi_kernel<<<n_blocks, pnm::kOptThreads, 0, (cudaStream_t)stream>>>(
      reinterpret_cast<const pnm::OptEntry*>(entries), reinterpret_cast<const int2*>(blocks), out);
  return (int)cudaGetLastError();
}

}  // extern "C"
