// In-kernel collectives over peer (NVLink / NVSwitch) memory: plain P2P loads and stores on
// buffers that every rank has mapped at rendezvous.  No NCCL call, no multimem, no cluster
// multicast.  One process per GPU runs the same kernel with the same grid; CTA b of every
// rank cooperates only with CTA b of the other ranks, through per-CTA flags, so no grid-wide
// synchronisation is needed and the kernels compose with stream order.
//
// Symmetric buffer layout (bytes), identical on every rank:
//   [0, kFlagBytes)            flags: [slot 2][phase 2][cta kPeerMaxCtas][rank 8] uint32 epochs
//   [kFlagBytes, ...)          two data slots (double buffered by call parity), each
//                              [stage A: capacity floats][stage B: capacity floats]
// Flags carry the monotonically increasing call number ("epoch"); a waiter accepts any value
// >= its epoch, so a stale flag is never mistaken for readiness.  Every wait is bounded:
// when the budget runs out the CTA records ERR_WAIT_PEER, fills its share of the output with
// NaN (so that a missed poll of the error word is still visible) and returns.
//
// Why two slots are enough: a rank writes slot (k+2) & 1 == k & 1 only after its own call
// k+1 completed, which needed every peer's flags of call k+1, which every peer raised after
// its call k had finished reading (stream order on each rank).
#pragma once
#include "common.cuh"

namespace pnm {

constexpr int kPeerMaxRanks = 8;
constexpr int kPeerMaxCtas = 128;
constexpr int kPeerSmallCta = kPeerMaxCtas - 1;  // flag row used by the "small reduce" helpers
constexpr int kFlagBytes = 2 * 2 * kPeerMaxCtas * kPeerMaxRanks * 4;  // 16 KiB

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
__device__ __forceinline__ uint32_t peer_epoch(const PeerArgs& p) { return p.epoch + (p.epoch_base ? *p.epoch_base : 0u); }
__device__ __forceinline__ uint32_t* peer_flag(const PeerArgs& p, int owner, int slot, int phase, int cta, int from) {
  return reinterpret_cast<uint32_t*>(p.base[owner]) + ((slot * 2 + phase) * kPeerMaxCtas + cta) * kPeerMaxRanks + from;
}
__device__ __forceinline__ float* peer_data(const PeerArgs& p, int owner, int slot, int stage) {
  return reinterpret_cast<float*>(p.base[owner] + kFlagBytes) + (size_t(slot) * 2 + stage) * p.capacity;
}

// Bounded spin of ONE thread until *f >= epoch.  Returns false when the budget ran out.
__device__ __forceinline__ bool peer_wait_flag(const uint32_t* f, uint32_t epoch, unsigned long long budget_ns, int* err) {
  unsigned long long t0 = 0;
  uint32_t spins = 0;
  while (int32_t(ld_acquire_sys(f) - epoch) < 0) {
    if ((++spins & 0xff) == 0) {
      const unsigned long long now = globaltimer_ns();
      if (t0 == 0) t0 = now;
      else if (now - t0 > budget_ns) { atomicCAS(err, 0, ERR_WAIT_PEER); return false; }
    }
  }
  return true;
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
    if (!peer_wait_flag(peer_flag(p, p.rank, slot, phase, blockIdx.x, threadIdx.x), epoch, p.budget_ns, err)) *sh_ok = 0;
  }
  __syncthreads();
  return *sh_ok != 0;
}

// ---- "small reduce" protocol: a producer kernel leaves a short fp32 vector in its own stage A of the slot and raises
// one flag per peer (row kPeerSmallCta); any number of CTAs of a later kernel wait for all ranks' flags and add up the
// vectors with direct peer loads.  Used where a handful of statistics must be summed over the ranks in the prologue of
// the kernel that consumes them (GroupNorm moments, slice-token sums): there is no stand-alone collective.
// Call from ONE thread after the data has been written and made visible (fence + block barrier by the caller).
__device__ __forceinline__ void peer_small_publish(const PeerArgs& p, uint32_t epoch) {
  __threadfence_system();
  for (int r = 0; r < p.world; ++r) st_release_sys(peer_flag(p, r, epoch & 1, 0, kPeerSmallCta, p.rank), epoch);
}
// All threads of the CTA call this; true when every rank's vector of call `epoch` is readable.
__device__ __forceinline__ bool peer_small_wait(const PeerArgs& p, uint32_t epoch, int* err, int* sh_ok) {
  if (threadIdx.x == 0) *sh_ok = 1;
  __syncthreads();
  if (threadIdx.x < p.world) {
    if (!peer_wait_flag(peer_flag(p, p.rank, epoch & 1, 0, kPeerSmallCta, threadIdx.x), epoch, p.budget_ns, err)) *sh_ok = 0;
  }
  __syncthreads();
  return *sh_ok != 0;
}
__device__ __forceinline__ float peer_small_sum(const PeerArgs& p, uint32_t epoch, long long i) {
  float s = 0.f;
  for (int r = 0; r < p.world; ++r) s += __ldcg(peer_data(p, r, epoch & 1, 0) + i);   // fixed order: same bits on every rank
  return s;
}

__device__ __forceinline__ float4 ldcg4(const float* p) { return __ldcg(reinterpret_cast<const float4*>(p)); }

// out = scale * sum over ranks of in (fp32), n <= capacity.  two_shot = 0: every rank reads
// every peer's whole vector (latency-optimal for small n); two_shot = 1: reduce-scatter then
// all-gather through peer reads (each rank moves 2 n (P-1)/P floats).  vec = 1: in / out are
// 16-byte aligned and the loops move float4.
static __global__ void __launch_bounds__(512)
peer_allreduce_kernel(const float* __restrict__ in, float* __restrict__ out, long long n, float scale, int two_shot,
                      int vec, PeerArgs p, int* err) {
  __shared__ int sh_ok;
  const uint32_t epoch = peer_epoch(p);
  const int slot = epoch & 1;
  const int nct = gridDim.x;
  const float nanv = __int_as_float(0x7fc00000);
  float* mineA = peer_data(p, p.rank, slot, 0);
  if (!two_shot) {
    const long long per = ((n + nct - 1) / nct + 3) & ~3ll;
    const long long lo = per * blockIdx.x;
    const long long hi = lo + per < n ? lo + per : n;
    if (vec) {
      for (long long i = lo + 4 * threadIdx.x; i < hi; i += 4 * blockDim.x) {
        if (i + 4 <= hi) *reinterpret_cast<float4*>(mineA + i) = *reinterpret_cast<const float4*>(in + i);
        else for (long long j = i; j < hi; ++j) mineA[j] = in[j];
      }
    } else {
      for (long long i = lo + threadIdx.x; i < hi; i += blockDim.x) mineA[i] = in[i];
    }
    if (!peer_exchange_flags(p, epoch, slot, 0, err, &sh_ok)) {
      for (long long i = lo + threadIdx.x; i < hi; i += blockDim.x) out[i] = nanv;
      return;
    }
    if (vec) {
      for (long long i = lo + 4 * threadIdx.x; i < hi; i += 4 * blockDim.x) {
        if (i + 4 <= hi) {
          float4 s = make_float4(0.f, 0.f, 0.f, 0.f);
          for (int r = 0; r < p.world; ++r) { const float4 v = ldcg4(peer_data(p, r, slot, 0) + i); s.x += v.x; s.y += v.y; s.z += v.z; s.w += v.w; }
          *reinterpret_cast<float4*>(out + i) = make_float4(s.x * scale, s.y * scale, s.z * scale, s.w * scale);
        } else {
          for (long long j = i; j < hi; ++j) {
            float s = 0.f;
            for (int r = 0; r < p.world; ++r) s += __ldcg(peer_data(p, r, slot, 0) + j);
            out[j] = s * scale;
          }
        }
      }
    } else {
      for (long long i = lo + threadIdx.x; i < hi; i += blockDim.x) {
        float s = 0.f;
        for (int r = 0; r < p.world; ++r) s += __ldcg(peer_data(p, r, slot, 0) + i);  // fixed order: same bits on every rank
        out[i] = s * scale;
      }
    }
    return;
  }
  // two-shot: slice s belongs to rank s; CTA b handles sub-chunk b of every slice.  slice and per are multiples of 4,
  // so every (base + clo) is 16-byte aligned relative to the buffers.
  const long long slice = ((n + p.world - 1) / p.world + 3) & ~3ll;
  const long long per = ((slice + nct - 1) / nct + 3) & ~3ll;
  const long long clo = per * blockIdx.x;
  const long long chi = clo + per < slice ? clo + per : slice;
  for (int s = 0; s < p.world; ++s) {
    const long long base = s * slice;
    if (vec) {
      for (long long i = clo + 4 * threadIdx.x; i < chi; i += 4 * blockDim.x) {
        if (base + i + 4 <= n) *reinterpret_cast<float4*>(mineA + base + i) = *reinterpret_cast<const float4*>(in + base + i);
        else for (long long j = i; j < i + 4 && base + j < n; ++j) mineA[base + j] = in[base + j];
      }
    } else {
      for (long long i = clo + threadIdx.x; i < chi; i += blockDim.x)
        if (base + i < n) mineA[base + i] = in[base + i];
    }
  }
  bool ok = peer_exchange_flags(p, epoch, slot, 0, err, &sh_ok);
  if (ok) {
    const long long base = (long long)p.rank * slice;
    float* mineB = peer_data(p, p.rank, slot, 1);
    for (long long i = clo + 4 * threadIdx.x; i < chi; i += 4 * blockDim.x) {
      if (base + i >= n) break;
      if (base + i + 4 <= n) {
        float4 s = make_float4(0.f, 0.f, 0.f, 0.f);
        for (int r = 0; r < p.world; ++r) { const float4 v = ldcg4(peer_data(p, r, slot, 0) + base + i); s.x += v.x; s.y += v.y; s.z += v.z; s.w += v.w; }
        *reinterpret_cast<float4*>(mineB + i) = make_float4(s.x * scale, s.y * scale, s.z * scale, s.w * scale);
      } else {
        for (long long j = i; j < i + 4 && base + j < n; ++j) {
          float s = 0.f;
          for (int r = 0; r < p.world; ++r) s += __ldcg(peer_data(p, r, slot, 0) + base + j);
          mineB[j] = s * scale;
        }
      }
    }
    ok = peer_exchange_flags(p, epoch, slot, 1, err, &sh_ok);
  }
  for (int s = 0; s < p.world; ++s) {
    const long long base = s * slice;
    const float* src = peer_data(p, s, slot, 1);
    if (!ok) {
      for (long long i = clo + threadIdx.x; i < chi; i += blockDim.x) if (base + i < n) out[base + i] = nanv;
    } else if (vec) {
      for (long long i = clo + 4 * threadIdx.x; i < chi; i += 4 * blockDim.x) {
        if (base + i + 4 <= n) *reinterpret_cast<float4*>(out + base + i) = ldcg4(src + i);
        else for (long long j = i; j < i + 4 && base + j < n; ++j) out[base + j] = __ldcg(src + j);
      }
    } else {
      for (long long i = clo + threadIdx.x; i < chi; i += blockDim.x)
        if (base + i < n) out[base + i] = __ldcg(src + i);
    }
  }
}

// Gradient-bucket all-reduce with a bf16 wire format: io[i] <- sum over ranks of bf16(scale * io[i]), accumulated in
// fp32.  One kernel does the cast + scale into the symmetric staging area, the reduce-scatter over peer loads, and
// the all-gather that writes fp32 back in place.  n % 8 == 0 and io 32-byte aligned; 2 n bytes <= 4 * capacity.
static __global__ void __launch_bounds__(512)
peer_allreduce_bf16_kernel(float* __restrict__ io, long long n, float scale, PeerArgs p, int* err) {
  __shared__ int sh_ok;
  const uint32_t epoch = peer_epoch(p);
  const int slot = epoch & 1;
  const int nct = gridDim.x;
  const float nanv = __int_as_float(0x7fc00000);
  __nv_bfloat16* mineA = reinterpret_cast<__nv_bfloat16*>(peer_data(p, p.rank, slot, 0));
  const long long slice = ((n + p.world - 1) / p.world + 7) & ~7ll;
  const long long per = ((slice + nct - 1) / nct + 7) & ~7ll;
  const long long clo = per * blockIdx.x;
  const long long chi = clo + per < slice ? clo + per : slice;
  for (int s = 0; s < p.world; ++s) {
    const long long base = s * slice;
    for (long long i = clo + 8 * threadIdx.x; i < chi; i += 8 * blockDim.x) {
      if (base + i >= n) break;
      const float4 a = *reinterpret_cast<const float4*>(io + base + i);
      const float4 b = *reinterpret_cast<const float4*>(io + base + i + 4);
      uint4 u;
      u.x = pack_bf16x2(a.x * scale, a.y * scale); u.y = pack_bf16x2(a.z * scale, a.w * scale);
      u.z = pack_bf16x2(b.x * scale, b.y * scale); u.w = pack_bf16x2(b.z * scale, b.w * scale);
      *reinterpret_cast<uint4*>(mineA + base + i) = u;
    }
  }
  bool ok = peer_exchange_flags(p, epoch, slot, 0, err, &sh_ok);
  if (ok) {
    const long long base = (long long)p.rank * slice;
    __nv_bfloat16* mineB = reinterpret_cast<__nv_bfloat16*>(peer_data(p, p.rank, slot, 1));
    for (long long i = clo + 8 * threadIdx.x; i < chi; i += 8 * blockDim.x) {
      if (base + i >= n) break;
      float acc[8] = {0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f};
      for (int r = 0; r < p.world; ++r) {
        const uint4 u = __ldcg(reinterpret_cast<const uint4*>(reinterpret_cast<const __nv_bfloat16*>(peer_data(p, r, slot, 0)) + base + i));
        float2 f;
        f = unpack_bf16x2(u.x); acc[0] += f.x; acc[1] += f.y;
        f = unpack_bf16x2(u.y); acc[2] += f.x; acc[3] += f.y;
        f = unpack_bf16x2(u.z); acc[4] += f.x; acc[5] += f.y;
        f = unpack_bf16x2(u.w); acc[6] += f.x; acc[7] += f.y;
      }
      uint4 o;
      o.x = pack_bf16x2(acc[0], acc[1]); o.y = pack_bf16x2(acc[2], acc[3]);
      o.z = pack_bf16x2(acc[4], acc[5]); o.w = pack_bf16x2(acc[6], acc[7]);
      *reinterpret_cast<uint4*>(mineB + i) = o;
    }
    ok = peer_exchange_flags(p, epoch, slot, 1, err, &sh_ok);
  }
  for (int s = 0; s < p.world; ++s) {
    const long long base = s * slice;
    const __nv_bfloat16* src = reinterpret_cast<const __nv_bfloat16*>(peer_data(p, s, slot, 1));
    for (long long i = clo + 8 * threadIdx.x; i < chi; i += 8 * blockDim.x) {
      if (base + i >= n) break;
      float4 a, b;
      if (ok) {
        const uint4 u = __ldcg(reinterpret_cast<const uint4*>(src + i));
        float2 f;
        f = unpack_bf16x2(u.x); a.x = f.x; a.y = f.y;
        f = unpack_bf16x2(u.y); a.z = f.x; a.w = f.y;
        f = unpack_bf16x2(u.z); b.x = f.x; b.y = f.y;
        f = unpack_bf16x2(u.w); b.z = f.x; b.w = f.y;
      } else {
        a = b = make_float4(nanv, nanv, nanv, nanv);
      }
      *reinterpret_cast<float4*>(io + base + i) = a;
      *reinterpret_cast<float4*>(io + base + i + 4) = b;
    }
  }
}

// Copy `bytes` (multiple of 16) from a (peer-mapped) source into local memory after the "small" flag of call `epoch` has
// arrived from rank flag_from (flag_from >= 0), from every rank (flag_from == -2), or at once (flag_from == -1).  The
// building block of staged transfers: the copy of the next owner's block can run on a side stream while the tensor
// cores work on the current one.  On a time-out the destination is filled with NaN patterns.
static __global__ void __launch_bounds__(512)
peer_pull_kernel(const uint4* __restrict__ src, uint4* __restrict__ dst, long long nvec, PeerArgs p, int flag_from, int* err) {
  __shared__ int sh_ok;
  bool ok = true;
  if (flag_from >= 0) {
    const uint32_t epoch = peer_epoch(p);
    if (threadIdx.x == 0)
      sh_ok = peer_wait_flag(peer_flag(p, p.rank, epoch & 1, 0, kPeerSmallCta, flag_from), epoch, p.budget_ns, err) ? 1 : 0;
    __syncthreads();
    ok = sh_ok != 0;
  } else if (flag_from == -2) {
    ok = peer_small_wait(p, peer_epoch(p), err, &sh_ok);
  }
  const uint4 nan4 = make_uint4(0x7fc07fc0u, 0x7fc07fc0u, 0x7fc07fc0u, 0x7fc07fc0u);
  for (long long i = blockIdx.x * (long long)blockDim.x + threadIdx.x; i < nvec; i += (long long)gridDim.x * blockDim.x)
    dst[i] = ok ? __ldcg(src + i) : nan4;
}

// Raise this rank's "small" flag of call `epoch` on every peer: data written earlier on the stream is then readable.
static __global__ void peer_signal_kernel(PeerArgs p) {
  if (threadIdx.x == 0 && blockIdx.x == 0) peer_small_publish(p, peer_epoch(p));
}

// dst[i] = sum over ranks r of src_r[i] for this rank's own block: every rank keeps a full-length partial result in
// its stage A (written before the flags of call `epoch` were raised by peer_signal_kernel); rank q owns elements
// [q * block, (q + 1) * block).  A reduce-scatter in the pull model: no atomics, fixed summation order.
static __global__ void __launch_bounds__(512)
peer_pull_reduce_kernel(float* __restrict__ dst, long long block, PeerArgs p, int* err) {
  __shared__ int sh_ok;
  const uint32_t epoch = peer_epoch(p);
  if (!peer_small_wait(p, epoch, err, &sh_ok)) {
    const float nanv = __int_as_float(0x7fc00000);
    for (long long i = blockIdx.x * (long long)blockDim.x + threadIdx.x; i < block; i += (long long)gridDim.x * blockDim.x) dst[i] = nanv;
    return;
  }
  const long long off = (long long)p.rank * block;
  for (long long i = 4 * (blockIdx.x * (long long)blockDim.x + threadIdx.x); i < block; i += 4 * (long long)gridDim.x * blockDim.x) {
    float4 s = make_float4(0.f, 0.f, 0.f, 0.f);
    for (int r = 0; r < p.world; ++r) { const float4 v = ldcg4(peer_data(p, r, epoch & 1, 0) + off + i); s.x += v.x; s.y += v.y; s.z += v.z; s.w += v.w; }
    *reinterpret_cast<float4*>(dst + i) = s;
  }
}

// dst[i] = sum over ranks r of srcs.p[r][i], i < n: every rank has left a partial result in symmetric memory before raising
// its flag of call `epoch`; the caller passes, per rank, the address of the block that belongs to THIS rank.  The same
// reduce-scatter in the pull model as above, with explicit addresses instead of the slot layout.
struct PeerSrcs { const float* p[kPeerMaxRanks]; };
static __global__ void __launch_bounds__(512)
peer_sum_blocks_kernel(float* __restrict__ dst, PeerSrcs srcs, long long n, int wait, PeerArgs p, int* err) {
  __shared__ int sh_ok;
  bool ok = true;
  if (wait) ok = peer_small_wait(p, peer_epoch(p), err, &sh_ok);
  const float nanv = __int_as_float(0x7fc00000);
  for (long long i = 4 * (blockIdx.x * (long long)blockDim.x + threadIdx.x); i < n; i += 4 * (long long)gridDim.x * blockDim.x) {
    float4 s = make_float4(0.f, 0.f, 0.f, 0.f);
    if (ok) {
      for (int r = 0; r < p.world; ++r) { const float4 v = ldcg4(srcs.p[r] + i); s.x += v.x; s.y += v.y; s.z += v.z; s.w += v.w; }
    } else {
      s = make_float4(nanv, nanv, nanv, nanv);
    }
    *reinterpret_cast<float4*>(dst + i) = s;
  }
}

// A wait that nothing satisfies: used by the failure-detection test to check that a bounded
// wait gives up, reports ERR_WAIT_PEER and leaves the context usable.
static __global__ void peer_wait_probe_kernel(const uint32_t* flag, uint32_t expect, unsigned long long budget_ns,
                                       int* err, int* status_out) {
  unsigned long long t0 = globaltimer_ns();
  int ok = 1;
  while (int32_t(ld_acquire_sys(flag) - expect) < 0) {
    if (globaltimer_ns() - t0 > budget_ns) { atomicCAS(err, 0, ERR_WAIT_PEER); ok = 0; break; }
  }
  *status_out = ok;
}

inline int peer_grid(long long n_items, long long per_cta, int max_ctas) {
  long long want = (n_items + per_cta - 1) / per_cta;
  int cap = max_ctas > 0 && max_ctas < kPeerMaxCtas - 1 ? max_ctas : kPeerMaxCtas - 1;  // the last flag row is reserved
  int grid = (int)(want < cap ? want : cap);
  return grid < 1 ? 1 : grid;
}

inline int launch_peer_allreduce(const float* in, float* out, long long n, float scale, int two_shot,
                                 const PeerArgs& p, int max_ctas, int* err, cudaStream_t st) {
  if (n <= 0) return 0;
  if (n > p.capacity || p.world > kPeerMaxRanks || p.world < 1) return -50;
  const int vec = ((reinterpret_cast<uintptr_t>(in) | reinterpret_cast<uintptr_t>(out)) & 15) == 0;
  const int grid = peer_grid(n, 4096, max_ctas);
  peer_allreduce_kernel<<<grid, 512, 0, st>>>(in, out, n, scale, two_shot, vec, p, err);
  return cudaGetLastError() == cudaSuccess ? 0 : -51;
}

inline int launch_peer_allreduce_bf16(float* io, long long n, float scale, const PeerArgs& p, int max_ctas, int* err,
                                      cudaStream_t st) {
  if (n <= 0) return 0;
  if ((n & 7) || (reinterpret_cast<uintptr_t>(io) & 31)) return -53;
  // stage A holds n bf16, stage B one slice: both fit when n bf16 <= capacity floats * 2
  if (n > 2 * p.capacity || p.world > kPeerMaxRanks || p.world < 1) return -50;
  const int grid = peer_grid(n, 8192, max_ctas);
  peer_allreduce_bf16_kernel<<<grid, 512, 0, st>>>(io, n, scale, p, err);
  return cudaGetLastError() == cudaSuccess ? 0 : -51;
}

}  // namespace pnm
