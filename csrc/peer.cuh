// In-kernel collectives over peer (NVLink / NVSwitch) memory: plain P2P loads and stores on
// buffers that every rank has mapped at rendezvous.  No NCCL call, no multimem, no cluster
// multicast.  One process per GPU runs the same kernel with the same grid; CTA b of every
// rank cooperates only with CTA b of the other ranks, through per-CTA flags, so no grid-wide
// synchronisation is needed and the kernels compose with stream order.
//
// Symmetric buffer layout (bytes), identical on every rank:
//   [0, kFlagBytes)            flags: [slot 2][phase 2][cta kMaxCtas][rank 8] uint32 epochs
//   [kFlagBytes, ...)          two data slots (double buffered by call parity), each
//                              [stage A: capacity floats][stage B: capacity floats]
// Flags carry the monotonically increasing call number ("epoch"); a waiter accepts any value
// >= its epoch, so a stale flag is never mistaken for readiness.  Every wait is bounded:
// when the budget runs out the CTA records ERR_WAIT_PEER and skips the dependent reads.
#pragma once
#include "common.cuh"

namespace pnm {

constexpr int kPeerMaxRanks = 8;
constexpr int kPeerMaxCtas = 64;
constexpr int kFlagBytes = 2 * 2 * kPeerMaxCtas * kPeerMaxRanks * 4;  // 8 KiB

struct PeerArgs {
  uint8_t* base[kPeerMaxRanks];  // symmetric buffer of every rank (peer-mapped pointers)
  int rank, world;
  uint32_t epoch;        // call number, starts at 1 (an offset from *epoch_base when that is set)
  const uint32_t* epoch_base;  // optional device-resident counter: lets a captured CUDA graph advance epochs on replay
  long long capacity;    // floats per stage
  unsigned long long budget_ns;
};

__device__ __forceinline__ void st_release_sys(uint32_t* p, uint32_t v) {
  asm volatile("st.release.sys.global.u32 [%0], %1;" ::"l"(p), "r"(v) : "memory");
}
__device__ __forceinline__ uint32_t ld_acquire_sys(const uint32_t* p) {
  uint32_t v;
  asm volatile("ld.acquire.sys.global.u32 %0, [%1];" : "=r"(v) : "l"(p) : "memory");
  return v;
}
__device__ __forceinline__ uint32_t* peer_flag(const PeerArgs& p, int owner, int slot, int phase, int cta, int from) {
  return reinterpret_cast<uint32_t*>(p.base[owner]) + ((slot * 2 + phase) * kPeerMaxCtas + cta) * kPeerMaxRanks + from;
}
__device__ __forceinline__ float* peer_data(const PeerArgs& p, int owner, int slot, int stage) {
  return reinterpret_cast<float*>(p.base[owner] + kFlagBytes) + (size_t(slot) * 2 + stage) * p.capacity;
}

// Tell every rank that this CTA's data of (slot, phase) is visible; then wait for all of them.
// Called by all threads of the CTA; returns false when a peer did not arrive in time.
__device__ __forceinline__ bool peer_exchange_flags(const PeerArgs& p, uint32_t epoch, int slot, int phase, int* err, int* sh_ok) {
  __syncthreads();
  if (threadIdx.x < p.world) {
    __threadfence_system();
    st_release_sys(peer_flag(p, threadIdx.x, slot, phase, blockIdx.x, p.rank), epoch);
  }
  if (threadIdx.x == 0) *sh_ok = 1;
  __syncthreads();
  if (threadIdx.x < p.world) {
    const uint32_t* f = peer_flag(p, p.rank, slot, phase, blockIdx.x, threadIdx.x);
    unsigned long long t0 = 0;
    uint32_t spins = 0;
    while (int32_t(ld_acquire_sys(f) - epoch) < 0) {
      if ((++spins & 0xff) == 0) {
        unsigned long long now = globaltimer_ns();
        if (t0 == 0) t0 = now;
        else if (now - t0 > p.budget_ns) { atomicCAS(err, 0, ERR_WAIT_PEER); *sh_ok = 0; break; }
      }
    }
  }
  __syncthreads();
  return *sh_ok != 0;
}

// out = scale * sum over ranks of in (fp32), n <= capacity.  two_shot = 0: every rank reads
// every peer's whole vector (latency-optimal for small n); two_shot = 1: reduce-scatter then
// all-gather through peer reads (each rank moves 2 n (P-1)/P floats).
__global__ void __launch_bounds__(512)
peer_allreduce_kernel(const float* __restrict__ in, float* __restrict__ out, long long n, float scale, int two_shot,
                      PeerArgs p, int* err) {
  __shared__ int sh_ok;
  const uint32_t epoch = p.epoch + (p.epoch_base ? *p.epoch_base : 0u);
  const int slot = epoch & 1;
  const int nct = gridDim.x;
  float* mineA = peer_data(p, p.rank, slot, 0);
  if (!two_shot) {
    const long long per = ((n + nct - 1) / nct + 3) & ~3ll;
    const long long lo = per * blockIdx.x;
    const long long hi = lo + per < n ? lo + per : n;
    for (long long i = lo + threadIdx.x; i < hi; i += blockDim.x) mineA[i] = in[i];
    if (!peer_exchange_flags(p, epoch, slot, 0, err, &sh_ok)) return;
    for (long long i = lo + threadIdx.x; i < hi; i += blockDim.x) {
      float s = 0.f;
      for (int r = 0; r < p.world; ++r) s += __ldcg(peer_data(p, r, slot, 0) + i);  // fixed order: same bits on every rank
      out[i] = s * scale;
    }
    return;
  }
  // two-shot: slice s belongs to rank s; CTA b handles sub-chunk b of every slice
  const long long slice = ((n + p.world - 1) / p.world + 3) & ~3ll;
  const long long per = ((slice + nct - 1) / nct + 3) & ~3ll;
  const long long clo = per * blockIdx.x;
  const long long chi = clo + per < slice ? clo + per : slice;
  for (int s = 0; s < p.world; ++s) {
    const long long base = s * slice;
    for (long long i = clo + threadIdx.x; i < chi; i += blockDim.x)
      if (base + i < n) mineA[base + i] = in[base + i];
  }
  if (!peer_exchange_flags(p, epoch, slot, 0, err, &sh_ok)) return;
  {
    const long long base = (long long)p.rank * slice;
    float* mineB = peer_data(p, p.rank, slot, 1);
    for (long long i = clo + threadIdx.x; i < chi; i += blockDim.x) {
      if (base + i >= n) break;
      float s = 0.f;
      for (int r = 0; r < p.world; ++r) s += __ldcg(peer_data(p, r, slot, 0) + base + i);
      mineB[i] = s * scale;
    }
  }
  if (!peer_exchange_flags(p, epoch, slot, 1, err, &sh_ok)) return;
  for (int s = 0; s < p.world; ++s) {
    const long long base = s * slice;
    const float* src = peer_data(p, s, slot, 1);
    for (long long i = clo + threadIdx.x; i < chi; i += blockDim.x)
      if (base + i < n) out[base + i] = __ldcg(src + i);
  }
}

// A wait that nothing satisfies: used by the failure-detection test to check that a bounded
// wait gives up, reports ERR_WAIT_PEER and leaves the context usable.
__global__ void peer_wait_probe_kernel(const uint32_t* flag, uint32_t expect, unsigned long long budget_ns,
                                       int* err, int* status_out) {
  unsigned long long t0 = globaltimer_ns();
  int ok = 1;
  while (int32_t(ld_acquire_sys(flag) - expect) < 0) {
    if (globaltimer_ns() - t0 > budget_ns) { atomicCAS(err, 0, ERR_WAIT_PEER); ok = 0; break; }
  }
  *status_out = ok;
}

inline int launch_peer_allreduce(const float* in, float* out, long long n, float scale, int two_shot,
                                 const PeerArgs& p, int* err, cudaStream_t st) {
  if (n <= 0) return 0;
  if (n > p.capacity || p.world > kPeerMaxRanks || p.world < 1) return -50;
  long long want = (n + 4095) / 4096;
  int grid = (int)(want < kPeerMaxCtas ? want : kPeerMaxCtas);
  if (grid < 1) grid = 1;
  peer_allreduce_kernel<<<grid, 512, 0, st>>>(in, out, n, scale, two_shot, p, err);
  return cudaGetLastError() == cudaSuccess ? 0 : -51;
}

}  // namespace pnm
